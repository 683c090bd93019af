/*
 * winograd_f43.cuh -- fast kernels for the 3x3 transforms, F(4x4,3x3) and F(2x2,3x3), on 16-bit and float32 tensors,
 * the case the ResNet-style layers use.  Same arithmetic as the generic kernels of winograd_nonfused.cu (reference
 * src/winograd_nonfused.cu:302-423, tables :549-557) with the 6-point transforms factored by hand:
 *
 *   B^T d :  c = d4-d2, e = d3-d1, a = d2-d4/4, b = d1-d3/4
 *            [ (d0-d2)+c/4,  a+b,  a-b,  e+c/2,  c/2-e,  (d5-d3)/4-e ]                      12 operations
 *   A^T m :  s = m1+m2, d = m1-m2, u = m3+m4, v = m3-m4
 *            [ m0+s+u/4,  d+v/2,  s+u,  d+2(v+m5) ]                                        10 operations
 *   G' g  :  (gradient, 6x4)  s = g0+g2, t = g1+g3, p = g0/3+4g2/3, q = 2g1/3+8g3/3
 *            [ g0,  2(s+t)/3,  2(s-t)/3,  p+q,  p-q,  2g3 ]                                 11 operations
 *
 * Input transform: a CTA owns a strip of tiles; one thread fetches the strip's halo box of the NHWC input with a
 * single 4-D TMA copy (out-of-range rows, columns and channels arrive as zeros, which is the zero padding), the next
 * strip is in flight while the current one is transformed, every lane reads its two channels from shared memory
 * with compile-time offsets and writes 36 plane rows of 128 (256) contiguous bytes per warp.
 * Output / gradient transforms read and write global memory directly: their accesses are already whole lines.
 */
#ifndef B200_WINOGRAD_F43_CUH_
#define B200_WINOGRAD_F43_CUH_

#include "device_utils.cuh"
#include "umma.cuh"
#include "winograd_tables.cuh"

namespace f43
{
	using namespace bk;

	/* Two float32 values in one 64-bit register pair, operated on by the packed FP32 instructions of sm_100
	 * (add / sub / mul / fma .f32x2): one instruction per two channels.  Every operation rounds each half exactly like
	 * its scalar counterpart, so the transforms below give bit for bit what the scalar formulas give. */
	struct f2
	{
			unsigned long long v;
	};
	__device__ __forceinline__ f2 make_f2(float a, float b)
	{
		f2 r;
		asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(a), "f"(b));
		return r;
	}
	__device__ __forceinline__ f2 make_f2(float2 a)
	{
		return make_f2(a.x, a.y);
	}
	__device__ __forceinline__ f2 splat(float a)
	{
		return make_f2(a, a);
	}
	__device__ __forceinline__ float2 to_float2(f2 a)
	{
		float2 r;
		asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(a.v));
		return r;
	}
	__device__ __forceinline__ f2 add2(f2 a, f2 b)
	{
		f2 r;
		asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
		return r;
	}
	__device__ __forceinline__ f2 sub2(f2 a, f2 b)
	{
		f2 r;
		asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
		return r;
	}
	__device__ __forceinline__ f2 mul2(f2 a, f2 b)
	{
		f2 r;
		asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
		return r;
	}
	__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) /* a * b + c, one rounding */
	{
		f2 r;
		asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v));
		return r;
	}

	__device__ __forceinline__ void input_1d(const f2 (&d)[6], f2 (&o)[6])
	{
		const f2 quarter = splat(0.25f), half_ = splat(0.5f), minus_quarter = splat(-0.25f);
		const f2 c = sub2(d[4], d[2]);
		const f2 e = sub2(d[3], d[1]);
		const f2 minus_e = sub2(d[1], d[3]); /* exactly -e */
		const f2 a = fma2(minus_quarter, d[4], d[2]);
		const f2 b = fma2(minus_quarter, d[3], d[1]);
		o[0] = fma2(quarter, c, sub2(d[0], d[2]));
		o[1] = add2(a, b);
		o[2] = sub2(a, b);
		o[3] = fma2(half_, c, e);
		o[4] = fma2(half_, c, minus_e);
		o[5] = fma2(quarter, sub2(d[5], d[3]), minus_e);
	}
	__device__ __forceinline__ void output_1d(const f2 (&m)[6], f2 (&o)[4])
	{
		const f2 quarter = splat(0.25f), half_ = splat(0.5f), two = splat(2.0f);
		const f2 s = add2(m[1], m[2]);
		const f2 d = sub2(m[1], m[2]);
		const f2 u = add2(m[3], m[4]);
		const f2 v = sub2(m[3], m[4]);
		o[0] = fma2(quarter, u, add2(m[0], s));
		o[1] = fma2(half_, v, d);
		o[2] = add2(s, u);
		o[3] = fma2(two, add2(v, m[5]), d);
	}
	__device__ __forceinline__ void gradient_1d(const f2 (&g)[4], f2 (&o)[6])
	{
		const f2 k13 = splat(1.0f / 3.0f), k23 = splat(2.0f / 3.0f), k43 = splat(4.0f / 3.0f), k83 = splat(8.0f / 3.0f), two = splat(2.0f);
		const f2 s = add2(g[0], g[2]);
		const f2 t = add2(g[1], g[3]);
		const f2 p = fma2(k43, g[2], mul2(k13, g[0]));
		const f2 q = fma2(k83, g[3], mul2(k23, g[1]));
		o[0] = g[0];
		o[1] = mul2(k23, add2(s, t));
		o[2] = mul2(k23, sub2(s, t));
		o[3] = add2(p, q);
		o[4] = sub2(p, q);
		o[5] = mul2(two, g[3]);
	}

	/* F(2x2,3x3) one-dimensional transforms (reference tables src/winograd_nonfused.cu:534-539) */
	__device__ __forceinline__ void input_1d(const f2 (&d)[4], f2 (&o)[4])
	{
		o[0] = sub2(d[0], d[2]);
		o[1] = add2(d[1], d[2]);
		o[2] = sub2(d[2], d[1]);
		o[3] = sub2(d[3], d[1]);
	}
	__device__ __forceinline__ void output_1d(const f2 (&m)[4], f2 (&o)[2])
	{
		const f2 half_ = splat(0.5f);
		o[0] = fma2(half_, add2(m[1], m[2]), m[0]);
		o[1] = fma2(half_, sub2(m[1], m[2]), m[3]);
	}
	__device__ __forceinline__ void gradient_1d(const f2 (&g)[2], f2 (&o)[4])
	{
		o[0] = g[0];
		o[1] = add2(g[0], g[1]);
		o[2] = sub2(g[0], g[1]);
		o[3] = g[1];
	}

	/* two adjacent channels in storage form */
	template<typename T> struct Pair;
	template<> struct Pair<half>
	{
			using type = __half2;
			static __device__ __forceinline__ float2 unpack(__half2 v)
			{
				return __half22float2(v);
			}
			static __device__ __forceinline__ __half2 pack(float a, float b)
			{
				return __floats2half2_rn(a, b);
			}
	};
	template<> struct Pair<__nv_bfloat16>
	{
			using type = __nv_bfloat162;
			static __device__ __forceinline__ float2 unpack(__nv_bfloat162 v)
			{
				return __bfloat1622float2(v);
			}
			static __device__ __forceinline__ __nv_bfloat162 pack(float a, float b)
			{
				return __floats2bfloat162_rn(a, b);
			}
	};
	template<> struct Pair<float>
	{
			using type = float2;
			static __device__ __forceinline__ float2 unpack(float2 v)
			{
				return v;
			}
			static __device__ __forceinline__ float2 pack(float a, float b)
			{
				return make_float2(a, b);
			}
	};

	template<typename T>
	__device__ __forceinline__ f2 load_pair(const T *ptr) /* two adjacent channels, converted to float32 */
	{
		return make_f2(Pair<T>::unpack(*reinterpret_cast<const typename Pair<T>::type*>(ptr)));
	}
	template<>
	__device__ __forceinline__ f2 load_pair<float>(const float *ptr)
	{
		f2 r;
		r.v = *reinterpret_cast<const unsigned long long*>(ptr);
		return r;
	}
	template<typename T>
	__device__ __forceinline__ f2 unpack_pair(typename Pair<T>::type raw)
	{
		return make_f2(Pair<T>::unpack(raw));
	}
	template<typename T>
	__device__ __forceinline__ void store_pair(T *ptr, f2 value) /* rounded once, to nearest even */
	{
		const float2 v = to_float2(value);
		*reinterpret_cast<typename Pair<T>::type*>(ptr) = Pair<T>::pack(v.x, v.y);
	}
	template<>
	__device__ __forceinline__ void store_pair<float>(float *ptr, f2 value)
	{
		*reinterpret_cast<unsigned long long*>(ptr) = value.v;
	}

	/* Q adjacent pairs (2Q channels) of a lane with one access: 4, 8 or 16 bytes */
	template<typename T, int Q>
	__device__ __forceinline__ void load_pairs(const T *ptr, f2 (&out)[Q])
	{
		if constexpr (Q == 1)
			out[0] = load_pair<T>(ptr);
		else
		{
			static_assert(Q == 2, "one or two pairs per lane");
			using P = typename Pair<T>::type;
			if constexpr (sizeof(P) == 4)
			{
				const uint2 raw = *reinterpret_cast<const uint2*>(ptr);
				out[0] = unpack_pair<T>(*reinterpret_cast<const P*>(&raw.x));
				out[1] = unpack_pair<T>(*reinterpret_cast<const P*>(&raw.y));
			}
			else
			{
				const float4 raw = *reinterpret_cast<const float4*>(ptr);
				out[0] = make_f2(raw.x, raw.y);
				out[1] = make_f2(raw.z, raw.w);
			}
		}
	}
	template<typename T, int Q>
	__device__ __forceinline__ void store_pairs(T *ptr, const f2 (&value)[Q]) /* each value rounded once, to nearest even */
	{
		if constexpr (Q == 1)
			store_pair<T>(ptr, value[0]);
		else
		{
			using P = typename Pair<T>::type;
			const float2 a = to_float2(value[0]), b = to_float2(value[1]);
			if constexpr (sizeof(P) == 4)
			{
				const P pa = Pair<T>::pack(a.x, a.y), pb = Pair<T>::pack(b.x, b.y);
				uint2 raw;
				raw.x = *reinterpret_cast<const uint32_t*>(&pa);
				raw.y = *reinterpret_cast<const uint32_t*>(&pb);
				*reinterpret_cast<uint2*>(ptr) = raw;
			}
			else
				*reinterpret_cast<float4*>(ptr) = make_float4(a.x, a.y, b.x, b.y);
		}
	}

	constexpr int kChannelBlock = 64; /* channels per strip and pair of a lane: one warp, two channels per lane and pair */
	constexpr int kThreads = 256;
	constexpr int kMaxStages = 4;
/* Resident blocks per SM of the output transform with 16-bit transform-domain tensors.  Four (64 registers, no spills in
 * the linear and relu forms) against three: the kernel timed alone is slower (17.0 against 15.8 us on 64 x 56 x 56 x 64
 * float16), the pipeline it closes is faster (49.0 against 50.2 us per step), because its blocks then start on the SMs the
 * contraction kernel frees first and find the products in L2.  Five spill 130 bytes per thread. */
#ifndef F43_OUT_BLOCKS
#define F43_OUT_BLOCKS 4
#endif

	/* A weight transform that rides along with an input-transform launch: the first `ctas` blocks of the grid compute
	 * U = G w G^T (3x3 kernels, two channels per thread) instead of input strips.  The transform of 74 KB of weights is
	 * a few microseconds of launch latency as a kernel of its own and nothing inside a launch that is running anyway.
	 * ctas == 0 means no job. */
	struct WeightJob
	{
			const void *weights; /* [K, 3, 3, C] */
			void *matrices; /* [(TS + 2)^2, K, C] */
			int filters, channels;
			int invert; /* 180 degree rotation of the kernel (AVOCADO_CROSS_CORRELATION_MODE) */
			int ctas;
	};

	/* same arithmetic as kernel_weight_transform of winograd_nonfused.cu (winograd::transform_2d on the compile-time
	 * tables), so the result does not depend on which launch computed it */
	template<int TS, typename T, typename MT>
	__device__ __forceinline__ void weight_transform_pairs(const WeightJob &job, int cta, int threads)
	{
		using M = winograd::Matrix<winograd::Transform::Weight, TS, 3>;
		const int cpairs = job.channels / 2;
		const long long total = static_cast<long long>(job.filters) * cpairs;
		const T *weights = reinterpret_cast<const T*>(job.weights);
		MT *matrices = reinterpret_cast<MT*>(job.matrices);
		for (long long g = static_cast<long long>(cta) * threads + threadIdx.x; g < total; g += static_cast<long long>(job.ctas) * threads)
		{
			const int c0 = static_cast<int>(g % cpairs) * 2;
			const int k = static_cast<int>(g / cpairs);
			float in[2][9];
#pragma unroll
			for (int i = 0; i < 9; i++)
			{
				const float2 v = Pair<T>::unpack(*reinterpret_cast<const typename Pair<T>::type*>(weights + (static_cast<size_t>(k) * 9 + i) * job.channels + c0));
				const int dst = job.invert ? (8 - i) : i;
				in[0][dst] = v.x;
				in[1][dst] = v.y;
			}
			float out[2][M::Rows * M::Rows];
			winograd::transform_2d<M, float>(in[0], out[0]);
			winograd::transform_2d<M, float>(in[1], out[1]);
#pragma unroll
			for (int p = 0; p < M::Rows * M::Rows; p++)
				*reinterpret_cast<typename Pair<MT>::type*>(matrices + (static_cast<size_t>(p) * job.filters + k) * job.channels + c0) = Pair<MT>::pack(out[0][p],
						out[1][p]);
		}
	}

	struct InputGeometry
	{
			int batch, tiles_h, tiles_w, channels;
			int pad_h, pad_w;
			int strip_tiles_h, strip_tiles_w; /* tiles per strip */
			int row_groups, w_segments, c_blocks;
			int box_w; /* pixels per box row = transformSize * strip_tiles_w + 2 */
			int stage_bytes;
			int stages; /* depth of the shared-memory ring, 2..kMaxStages */
			int num_items;
			long long nb_tiles;
	};

	/* Q = pairs of channels per lane: 1 (a warp covers 64 channels of a tile) or 2 (128 channels: half as many shared
	 * loads, stores and address computations per byte; the tile's registers double, which F(2x2) affords and F(4x4) does not) */
	template<int TS, typename T, typename MT, int Q>
	/* the halo ring (up to 96 KB per block) lets two blocks share an SM: give each the registers of half an SM (no spills).
	 * Three blocks of 80 registers spill about 90 bytes per thread and were measured slower (25.5 against 19.0 us on the
	 * 64 x 56 x 56 x 64 float16 layer). */
	__global__ void __launch_bounds__(kThreads, 2) kernel_input_tma(const __grid_constant__ CUtensorMap mapX, MT *__restrict__ matrices, InputGeometry g,
			int *deviceStatus, WeightJob weightJob)
	{
		if (static_cast<int>(blockIdx.x) < weightJob.ctas)
		{
			/* a block of the weight transform that rides along (see WeightJob) */
			chain_wait();
			chain_release();
			weight_transform_pairs<TS, T, MT>(weightJob, static_cast<int>(blockIdx.x), static_cast<int>(blockDim.x));
			return;
		}
		const int cta = static_cast<int>(blockIdx.x) - weightJob.ctas;
		const int ncta = static_cast<int>(gridDim.x) - weightJob.ctas;
		extern __shared__ uint8_t smem_raw[];
		uint8_t *smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
		__shared__ __align__(8) uint64_t full_bar[kMaxStages];
		__shared__ __align__(8) uint64_t empty_bar[kMaxStages];
		__shared__ int abort_flag;

		const int tid = threadIdx.x;
		const int warp = tid / 32;
		const int lane = tid % 32;
		const int nwarps = blockDim.x / 32;
		if (tid == 0)
		{
			abort_flag = 0;
			for (int i = 0; i < kMaxStages; i++)
			{
				umma::mbar_init(&full_bar[i], 1);
				umma::mbar_init(&empty_bar[i], static_cast<uint32_t>(nwarps));
			}
			umma::mbar_fence_init();
			umma::prefetch_tensormap(&mapX);
		}
		__syncthreads();
		chain_wait(); /* x and the transform-domain tensor may still be in use by the previous kernel */
		chain_release();

		auto issue = [&](int item, int stage)
		{
			const int cb = item % g.c_blocks;
			const int ws = (item / g.c_blocks) % g.w_segments;
			const int rg = (item / (g.c_blocks * g.w_segments)) % g.row_groups;
			const int n = item / (g.c_blocks * g.w_segments * g.row_groups);
			umma::mbar_arrive_expect_tx(&full_bar[stage], static_cast<uint32_t>(g.stage_bytes));
			umma::tma_load_4d(smem + stage * g.stage_bytes, &mapX, &full_bar[stage], cb * kChannelBlock * Q, g.pad_w + ws * g.strip_tiles_w * TS,
					g.pad_h + rg * g.strip_tiles_h * TS, n);
		};

		/* fill the ring: strips 0 .. stages-2 of this CTA are requested before the first one is consumed */
		if (tid == 0)
			for (int i = 0; i < g.stages - 1; i++)
			{
				const long long item = static_cast<long long>(cta) + static_cast<long long>(i) * ncta;
				if (item < g.num_items)
					issue(static_cast<int>(item), i);
			}

		/* No block-wide barrier inside the loop: every warp waits for a strip on its full barrier by itself and hands the
		 * buffer back on its empty barrier as soon as its tile sits in registers, i.e. before the second transform pass and
		 * the stores, so the refill of a buffer overlaps the arithmetic on what it held and warps drift apart freely. */
		const size_t plane_stride = static_cast<size_t>(g.nb_tiles) * g.channels;
		constexpr int kLaneChannels = 2 * Q;
		constexpr int kWarpChannels = kChannelBlock * Q;
		const int row_pitch = g.box_w * kWarpChannels; /* elements of T per box row */
		volatile int *abort_ptr = &abort_flag;
		int it = 0;
		for (int item = cta; item < g.num_items; item += ncta, it++)
		{
			const int stage = it % g.stages;
			const uint32_t phase = static_cast<uint32_t>(it / g.stages) & 1u;
			if (tid == 0)
			{
				/* the strip stages-1 ahead goes into the buffer of the previous iteration, once every warp has let go of it */
				const long long next = static_cast<long long>(item) + static_cast<long long>(g.stages - 1) * ncta;
				if (next < g.num_items)
				{
					const int refill = (it + g.stages - 1) % g.stages;
					bool free_now = true;
					if (it >= 1)
						free_now = umma::mbar_wait(&empty_bar[refill], static_cast<uint32_t>((it - 1) / g.stages) & 1u, abort_ptr);
					if (free_now)
						issue(static_cast<int>(next), refill);
					else
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorStageWait);
				}
			}
			__syncwarp();
			if (not umma::mbar_wait(&full_bar[stage], phase, abort_ptr))
			{
				umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
				break;
			}

			const int cb = item % g.c_blocks;
			const int ws = (item / g.c_blocks) % g.w_segments;
			const int rg = (item / (g.c_blocks * g.w_segments)) % g.row_groups;
			const int n = item / (g.c_blocks * g.w_segments * g.row_groups);
			const int c0 = cb * kWarpChannels + kLaneChannels * lane;
			const T *box = reinterpret_cast<const T*>(smem + stage * g.stage_bytes);

			const int strip_tiles = g.strip_tiles_h * g.strip_tiles_w;
			bool released = false;
			for (int t = warp; t < strip_tiles; t += nwarps)
			{
				const int tr = t / g.strip_tiles_w;
				const int tc = t - tr * g.strip_tiles_w;
				const int th = rg * g.strip_tiles_h + tr;
				const int tw = ws * g.strip_tiles_w + tc;
				const bool active = th < g.tiles_h and tw < g.tiles_w and c0 < g.channels;
				constexpr int TL = TS + 2;
				const T *src = box + (tr * TS) * row_pitch + (tc * TS) * kWarpChannels + kLaneChannels * lane;

				f2 tmp[Q][TL * TL]; /* B^T d, the lane's pairs of channels */
				if (active)
				{
#pragma unroll
					for (int c = 0; c < TL; c++)
					{
						f2 col[Q][TL];
#pragma unroll
						for (int r = 0; r < TL; r++)
						{
							f2 loaded[Q];
							load_pairs<T, Q>(src + r * row_pitch + c * kWarpChannels, loaded);
#pragma unroll
							for (int q = 0; q < Q; q++)
								col[q][r] = loaded[q];
						}
#pragma unroll
						for (int q = 0; q < Q; q++)
						{
							f2 o[TL];
							input_1d(col[q], o);
#pragma unroll
							for (int i = 0; i < TL; i++)
								tmp[q][i * TL + c] = o[i];
						}
					}
				}
				if (t + nwarps >= strip_tiles)
				{
					/* this warp's last tile of the strip is in registers */
					__syncwarp();
					if (lane == 0)
						umma::mbar_arrive(&empty_bar[stage]);
					released = true;
				}
				if (active)
				{
					const long long tile = (static_cast<long long>(n) * g.tiles_h + th) * g.tiles_w + tw;
					MT *dst = matrices + static_cast<size_t>(tile) * g.channels + c0;
#pragma unroll
					for (int i = 0; i < TL; i++)
					{
						f2 o[Q][TL];
#pragma unroll
						for (int q = 0; q < Q; q++)
						{
							f2 row[TL];
#pragma unroll
							for (int c = 0; c < TL; c++)
								row[c] = tmp[q][i * TL + c];
							input_1d(row, o[q]);
						}
#pragma unroll
						for (int j = 0; j < TL; j++)
						{
							f2 out[Q];
#pragma unroll
							for (int q = 0; q < Q; q++)
								out[q] = o[q][j];
							store_pairs<MT, Q>(dst, out);
							dst += plane_stride;
						}
					}
				}
			}
			if (not released)
			{
				__syncwarp();
				if (lane == 0)
					umma::mbar_arrive(&empty_bar[stage]); /* a warp without a tile in this strip */
			}
		}
		__syncthreads();
		if (abort_flag != 0)
			umma::drain_after_abort();
	}

	struct PlaneGeometry
	{
			int batch, height, width, channels; /* of the NHWC tensor */
			int tiles_h, tiles_w;
			long long nb_tiles;
	};

	/* ACT: 0 linear, 1 relu, 2 any (run-time switch) */
	template<int TS, typename T, typename MT, int ACT>
	/* float32 planes need twice the registers for the tile: two resident blocks without spills beat three with them */
	__global__ void __launch_bounds__(kThreads, sizeof(MT) == 4 ? 2 : F43_OUT_BLOCKS) kernel_output(const MT *__restrict__ matrices, T *output, PlaneGeometry g, const float *__restrict__ bias,
			const T *__restrict__ ext, float alpha1, float alpha2, float beta, avocado::backend::avActivationType_t activation)
	{
		using PT = typename Pair<T>::type;
		using PM = typename Pair<MT>::type;
		chain_wait();
		chain_release();
		/* one warp per tile and block of 64 channels: blockIdx.x counts groups of 8 tiles, blockIdx.y channel blocks */
		const unsigned int tile = blockIdx.x * (kThreads / 32) + threadIdx.x / 32;
		const int c0 = blockIdx.y * kChannelBlock + 2 * (threadIdx.x % 32);
		if (tile >= static_cast<unsigned int>(g.nb_tiles) or c0 >= g.channels)
			return;
		const unsigned int tile_row = tile / static_cast<unsigned int>(g.tiles_w);
		const int tw = static_cast<int>(tile - tile_row * g.tiles_w);
		const int n = static_cast<int>(tile_row / static_cast<unsigned int>(g.tiles_h));
		const int th = static_cast<int>(tile_row - n * g.tiles_h);

		constexpr int TL = TS + 2;
		const size_t plane_stride = static_cast<size_t>(g.nb_tiles) * g.channels;
		const MT *src = matrices + static_cast<size_t>(tile) * g.channels + c0;
		PM raw[TL * TL];
#pragma unroll
		for (int p = 0; p < TL * TL; p++)
		{
			raw[p] = *reinterpret_cast<const PM*>(src);
			src += plane_stride;
		}
		f2 tmp[TS * TL]; /* A^T M: TS x TL, both channels of the lane */
#pragma unroll
		for (int c = 0; c < TL; c++)
		{
			f2 col[TL], o[TS];
#pragma unroll
			for (int r = 0; r < TL; r++)
				col[r] = unpack_pair<MT>(raw[r * TL + c]);
			output_1d(col, o);
#pragma unroll
			for (int i = 0; i < TS; i++)
				tmp[i * TL + c] = o[i];
		}
		f2 b = splat(0.0f);
		if (bias != nullptr)
			b = load_pair<float>(bias + c0);
		const f2 a1 = splat(alpha1), a2 = splat(alpha2), bt = splat(beta), zero = splat(0.0f);

		const int h0 = th * TS, w0 = tw * TS;
		T *tile_ptr = output + ((static_cast<size_t>(n) * g.height + h0) * g.width + w0) * g.channels + c0;
		const T *ext_ptr = (ext == nullptr) ? nullptr : ext + ((static_cast<size_t>(n) * g.height + h0) * g.width + w0) * g.channels + c0;
		const int row_stride = g.width * g.channels;
		const bool interior = (h0 + TS <= g.height) and (w0 + TS <= g.width);
#pragma unroll
		for (int i = 0; i < TS; i++)
		{
			f2 row[TL], o[TS];
#pragma unroll
			for (int c = 0; c < TL; c++)
				row[c] = tmp[i * TL + c];
			output_1d(row, o);
#pragma unroll
			for (int j = 0; j < TS; j++)
			{
				if (interior or (h0 + i < g.height and w0 + j < g.width))
				{
					const int offset = i * row_stride + j * g.channels;
					f2 v = fma2(a1, o[j], b);
					if (ext_ptr != nullptr)
						v = fma2(a2, load_pair<T>(ext_ptr + offset), v);
					if (ACT == 1)
					{
						/* relu as the scalar fmaxf(v, 0) of each half (no packed maximum exists) */
						const float2 u = to_float2(v);
						v = make_f2(fmaxf(u.x, 0.0f), fmaxf(u.y, 0.0f));
					}
					else if (ACT == 2)
					{
						const float2 u = to_float2(v);
						v = make_f2(activation_forward(activation, u.x), activation_forward(activation, u.y));
					}
					if (beta != 0.0f)
						v = fma2(bt, load_pair<T>(tile_ptr + offset), v);
					store_pair<T>(tile_ptr + offset, v);
				}
			}
		}
		(void) zero;
	}

	/* dy[N,H,W,K] -> [tile*tile, tiles, K]: TS x TS tile, zero past the image edge (reference src/winograd_nonfused.cu:424-475) */
	template<int TS, typename T, typename MT>
	__global__ void __launch_bounds__(kThreads, 2) kernel_gradient(MT *__restrict__ matrices, const T *__restrict__ gradient, PlaneGeometry g)
	{
		using PT = typename Pair<T>::type;
		using PM = typename Pair<MT>::type;
		chain_wait();
		chain_release();
		/* one warp per tile and block of 64 channels: blockIdx.x counts groups of 8 tiles, blockIdx.y channel blocks */
		const unsigned int tile = blockIdx.x * (kThreads / 32) + threadIdx.x / 32;
		const int c0 = blockIdx.y * kChannelBlock + 2 * (threadIdx.x % 32);
		if (tile >= static_cast<unsigned int>(g.nb_tiles) or c0 >= g.channels)
			return;
		const unsigned int tile_row = tile / static_cast<unsigned int>(g.tiles_w);
		const int tw = static_cast<int>(tile - tile_row * g.tiles_w);
		const int n = static_cast<int>(tile_row / static_cast<unsigned int>(g.tiles_h));
		const int th = static_cast<int>(tile_row - n * g.tiles_h);
		constexpr int TL = TS + 2;
		const int h0 = th * TS, w0 = tw * TS;
		const T *tile_ptr = gradient + ((static_cast<size_t>(n) * g.height + h0) * g.width + w0) * g.channels + c0;
		const int row_stride = g.width * g.channels;
		const bool interior = (h0 + TS <= g.height) and (w0 + TS <= g.width);

		PT raw[TS * TS];
#pragma unroll
		for (int r = 0; r < TS; r++)
#pragma unroll
			for (int c = 0; c < TS; c++)
			{
				if (interior or (h0 + r < g.height and w0 + c < g.width))
					raw[r * TS + c] = *reinterpret_cast<const PT*>(tile_ptr + r * row_stride + c * g.channels);
				else
					raw[r * TS + c] = Pair<T>::pack(0.0f, 0.0f);
			}
		f2 tmp[TL * TS]; /* G' g: TL x TS, both channels of the lane */
#pragma unroll
		for (int c = 0; c < TS; c++)
		{
			f2 col[TS], o[TL];
#pragma unroll
			for (int r = 0; r < TS; r++)
				col[r] = unpack_pair<T>(raw[r * TS + c]);
			gradient_1d(col, o);
#pragma unroll
			for (int i = 0; i < TL; i++)
				tmp[i * TS + c] = o[i];
		}
		const size_t plane_stride = static_cast<size_t>(g.nb_tiles) * g.channels;
		MT *dst = matrices + static_cast<size_t>(tile) * g.channels + c0;
#pragma unroll
		for (int i = 0; i < TL; i++)
		{
			f2 row[TS], o[TL];
#pragma unroll
			for (int c = 0; c < TS; c++)
				row[c] = tmp[i * TS + c];
			gradient_1d(row, o);
#pragma unroll
			for (int j = 0; j < TL; j++)
			{
				store_pair<MT>(dst, o[j]);
				dst += plane_stride;
			}
		}
	}
} /* namespace f43 */

#endif /* B200_WINOGRAD_F43_CUH_ */
