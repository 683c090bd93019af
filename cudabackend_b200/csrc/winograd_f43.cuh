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

namespace f43
{
	using namespace bk;

	__device__ __forceinline__ void input_1d(const float (&d)[6], float (&o)[6])
	{
		const float c = d[4] - d[2];
		const float e = d[3] - d[1];
		const float a = fmaf(-0.25f, d[4], d[2]);
		const float b = fmaf(-0.25f, d[3], d[1]);
		o[0] = fmaf(0.25f, c, d[0] - d[2]);
		o[1] = a + b;
		o[2] = a - b;
		o[3] = fmaf(0.5f, c, e);
		o[4] = fmaf(0.5f, c, -e);
		o[5] = fmaf(0.25f, d[5] - d[3], -e);
	}
	__device__ __forceinline__ void output_1d(const float (&m)[6], float (&o)[4])
	{
		const float s = m[1] + m[2];
		const float d = m[1] - m[2];
		const float u = m[3] + m[4];
		const float v = m[3] - m[4];
		o[0] = fmaf(0.25f, u, m[0] + s);
		o[1] = fmaf(0.5f, v, d);
		o[2] = s + u;
		o[3] = fmaf(2.0f, v + m[5], d);
	}
	__device__ __forceinline__ void gradient_1d(const float (&g)[4], float (&o)[6])
	{
		constexpr float k13 = 1.0f / 3.0f, k23 = 2.0f / 3.0f, k43 = 4.0f / 3.0f, k83 = 8.0f / 3.0f;
		const float s = g[0] + g[2];
		const float t = g[1] + g[3];
		const float p = fmaf(k43, g[2], k13 * g[0]);
		const float q = fmaf(k83, g[3], k23 * g[1]);
		o[0] = g[0];
		o[1] = k23 * (s + t);
		o[2] = k23 * (s - t);
		o[3] = p + q;
		o[4] = p - q;
		o[5] = 2.0f * g[3];
	}

	/* F(2x2,3x3) one-dimensional transforms (reference tables src/winograd_nonfused.cu:534-539) */
	__device__ __forceinline__ void input_1d(const float (&d)[4], float (&o)[4])
	{
		o[0] = d[0] - d[2];
		o[1] = d[1] + d[2];
		o[2] = d[2] - d[1];
		o[3] = d[3] - d[1];
	}
	__device__ __forceinline__ void output_1d(const float (&m)[4], float (&o)[2])
	{
		o[0] = fmaf(0.5f, m[1] + m[2], m[0]);
		o[1] = fmaf(0.5f, m[1] - m[2], m[3]);
	}
	__device__ __forceinline__ void gradient_1d(const float (&g)[2], float (&o)[4])
	{
		o[0] = g[0];
		o[1] = g[0] + g[1];
		o[2] = g[0] - g[1];
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

	constexpr int kChannelBlock = 64; /* channels per strip: one warp, two channels per lane */
	constexpr int kThreads = 256;
	constexpr int kMaxStages = 4;
#ifndef F43_OUT_BLOCKS
#define F43_OUT_BLOCKS 3
#endif

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

	template<int TS, typename T, typename MT>
	/* float32 stages are twice as large, so only two blocks fit an SM anyway: give them the registers of two (no spills) */
	__global__ void __launch_bounds__(kThreads, sizeof(T) == 4 ? 2 : 3) kernel_input_tma(const __grid_constant__ CUtensorMap mapX, MT *__restrict__ matrices, InputGeometry g,
			int *deviceStatus)
	{
		using PT = typename Pair<T>::type;
		using PM = typename Pair<MT>::type;
		extern __shared__ uint8_t smem_raw[];
		uint8_t *smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
		__shared__ __align__(8) uint64_t full_bar[kMaxStages];
		__shared__ int go_flag;
		__shared__ int abort_flag;

		const int tid = threadIdx.x;
		const int warp = tid / 32;
		const int lane = tid % 32;
		const int nwarps = blockDim.x / 32;
		if (tid == 0)
		{
			abort_flag = 0;
			for (int i = 0; i < kMaxStages; i++)
				umma::mbar_init(&full_bar[i], 1);
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
			umma::tma_load_4d(smem + stage * g.stage_bytes, &mapX, &full_bar[stage], cb * kChannelBlock, g.pad_w + ws * g.strip_tiles_w * TS,
					g.pad_h + rg * g.strip_tiles_h * TS, n);
		};

		/* fill the ring: strips 0 .. stages-2 of this CTA are requested before the first one is consumed */
		if (tid == 0)
			for (int i = 0; i < g.stages - 1; i++)
			{
				const long long item = static_cast<long long>(blockIdx.x) + static_cast<long long>(i) * gridDim.x;
				if (item < g.num_items)
					issue(static_cast<int>(item), i);
			}

		const size_t plane_stride = static_cast<size_t>(g.nb_tiles) * g.channels;
		const int row_pitch = g.box_w * kChannelBlock; /* elements of T per box row */
		int it = 0;
		for (int item = blockIdx.x; item < g.num_items; item += gridDim.x, it++)
		{
			const int stage = it % g.stages;
			const uint32_t phase = static_cast<uint32_t>(it / g.stages) & 1u;
			if (tid == 0)
			{
				/* the buffer consumed in the previous iteration was released by the barrier that closed it */
				const long long next = static_cast<long long>(item) + static_cast<long long>(g.stages - 1) * gridDim.x;
				if (next < g.num_items)
					issue(static_cast<int>(next), (it + g.stages - 1) % g.stages);
				const bool ready = umma::mbar_wait(&full_bar[stage], phase, &abort_flag);
				if (not ready)
					umma::raise_error(&abort_flag, deviceStatus, umma::kErrorTmaWait);
				go_flag = ready ? 1 : 0;
			}
			__syncthreads();
			if (go_flag == 0)
				break;
			umma::mbar_try_wait(&full_bar[stage], phase); /* completed phase: returns at once, orders this thread after the copy */

			const int cb = item % g.c_blocks;
			const int ws = (item / g.c_blocks) % g.w_segments;
			const int rg = (item / (g.c_blocks * g.w_segments)) % g.row_groups;
			const int n = item / (g.c_blocks * g.w_segments * g.row_groups);
			const int c0 = cb * kChannelBlock + 2 * lane;
			const T *box = reinterpret_cast<const T*>(smem + stage * g.stage_bytes);

			const int strip_tiles = g.strip_tiles_h * g.strip_tiles_w;
			for (int t = warp; t < strip_tiles; t += nwarps)
			{
				const int tr = t / g.strip_tiles_w;
				const int tc = t - tr * g.strip_tiles_w;
				const int th = rg * g.strip_tiles_h + tr;
				const int tw = ws * g.strip_tiles_w + tc;
				if (th >= g.tiles_h or tw >= g.tiles_w or c0 >= g.channels)
					continue;
				constexpr int TL = TS + 2;
				const T *src = box + (tr * TS) * row_pitch + (tc * TS) * kChannelBlock + 2 * lane;

				float tmp[2][TL * TL]; /* B^T d, per channel */
#pragma unroll
				for (int c = 0; c < TL; c++)
				{
					float col0[TL], col1[TL];
#pragma unroll
					for (int r = 0; r < TL; r++)
					{
						const float2 v = Pair<T>::unpack(*reinterpret_cast<const PT*>(src + r * row_pitch + c * kChannelBlock));
						col0[r] = v.x;
						col1[r] = v.y;
					}
					float o0[TL], o1[TL];
					input_1d(col0, o0);
					input_1d(col1, o1);
#pragma unroll
					for (int i = 0; i < TL; i++)
					{
						tmp[0][i * TL + c] = o0[i];
						tmp[1][i * TL + c] = o1[i];
					}
				}
				const long long tile = (static_cast<long long>(n) * g.tiles_h + th) * g.tiles_w + tw;
				MT *dst = matrices + static_cast<size_t>(tile) * g.channels + c0;
#pragma unroll
				for (int i = 0; i < TL; i++)
				{
					float row0[TL], row1[TL], o0[TL], o1[TL];
#pragma unroll
					for (int c = 0; c < TL; c++)
					{
						row0[c] = tmp[0][i * TL + c];
						row1[c] = tmp[1][i * TL + c];
					}
					input_1d(row0, o0);
					input_1d(row1, o1);
#pragma unroll
					for (int j = 0; j < TL; j++)
					{
						*reinterpret_cast<PM*>(dst) = Pair<MT>::pack(o0[j], o1[j]);
						dst += plane_stride;
					}
				}
			}
			__syncthreads(); /* every warp is done with this buffer: it may be refilled */
		}
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
		float tmp[2][TS * TL]; /* A^T M: TS x TL per channel */
#pragma unroll
		for (int c = 0; c < TL; c++)
		{
			float col0[TL], col1[TL], o0[TS], o1[TS];
#pragma unroll
			for (int r = 0; r < TL; r++)
			{
				const float2 v = Pair<MT>::unpack(raw[r * TL + c]);
				col0[r] = v.x;
				col1[r] = v.y;
			}
			output_1d(col0, o0);
			output_1d(col1, o1);
#pragma unroll
			for (int i = 0; i < TS; i++)
			{
				tmp[0][i * TL + c] = o0[i];
				tmp[1][i * TL + c] = o1[i];
			}
		}
		float2 b = make_float2(0.0f, 0.0f);
		if (bias != nullptr)
			b = *reinterpret_cast<const float2*>(bias + c0);

		const int h0 = th * TS, w0 = tw * TS;
		T *tile_ptr = output + ((static_cast<size_t>(n) * g.height + h0) * g.width + w0) * g.channels + c0;
		const T *ext_ptr = (ext == nullptr) ? nullptr : ext + ((static_cast<size_t>(n) * g.height + h0) * g.width + w0) * g.channels + c0;
		const int row_stride = g.width * g.channels;
		const bool interior = (h0 + TS <= g.height) and (w0 + TS <= g.width);
#pragma unroll
		for (int i = 0; i < TS; i++)
		{
			float row0[TL], row1[TL], o0[TS], o1[TS];
#pragma unroll
			for (int c = 0; c < TL; c++)
			{
				row0[c] = tmp[0][i * TL + c];
				row1[c] = tmp[1][i * TL + c];
			}
			output_1d(row0, o0);
			output_1d(row1, o1);
#pragma unroll
			for (int j = 0; j < TS; j++)
			{
				if (interior or (h0 + i < g.height and w0 + j < g.width))
				{
					const int offset = i * row_stride + j * g.channels;
					float v0 = fmaf(alpha1, o0[j], b.x);
					float v1 = fmaf(alpha1, o1[j], b.y);
					if (ext_ptr != nullptr)
					{
						const float2 z = Pair<T>::unpack(*reinterpret_cast<const PT*>(ext_ptr + offset));
						v0 = fmaf(alpha2, z.x, v0);
						v1 = fmaf(alpha2, z.y, v1);
					}
					if (ACT == 1)
					{
						v0 = fmaxf(v0, 0.0f);
						v1 = fmaxf(v1, 0.0f);
					}
					else if (ACT == 2)
					{
						v0 = activation_forward(activation, v0);
						v1 = activation_forward(activation, v1);
					}
					if (beta != 0.0f)
					{
						const float2 y = Pair<T>::unpack(*reinterpret_cast<const PT*>(tile_ptr + offset));
						v0 = fmaf(beta, y.x, v0);
						v1 = fmaf(beta, y.y, v1);
					}
					*reinterpret_cast<PT*>(tile_ptr + offset) = Pair<T>::pack(v0, v1);
				}
			}
		}
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
		float tmp[2][TL * TS]; /* G' g: TL x TS per channel */
#pragma unroll
		for (int c = 0; c < TS; c++)
		{
			float col0[TS], col1[TS], o0[TL], o1[TL];
#pragma unroll
			for (int r = 0; r < TS; r++)
			{
				const float2 v = Pair<T>::unpack(raw[r * TS + c]);
				col0[r] = v.x;
				col1[r] = v.y;
			}
			gradient_1d(col0, o0);
			gradient_1d(col1, o1);
#pragma unroll
			for (int i = 0; i < TL; i++)
			{
				tmp[0][i * TS + c] = o0[i];
				tmp[1][i * TS + c] = o1[i];
			}
		}
		const size_t plane_stride = static_cast<size_t>(g.nb_tiles) * g.channels;
		MT *dst = matrices + static_cast<size_t>(tile) * g.channels + c0;
#pragma unroll
		for (int i = 0; i < TL; i++)
		{
			float row0[TS], row1[TS], o0[TL], o1[TL];
#pragma unroll
			for (int c = 0; c < TS; c++)
			{
				row0[c] = tmp[0][i * TS + c];
				row1[c] = tmp[1][i * TS + c];
			}
			gradient_1d(row0, o0);
			gradient_1d(row1, o1);
#pragma unroll
			for (int j = 0; j < TL; j++)
			{
				*reinterpret_cast<PM*>(dst) = Pair<MT>::pack(o0[j], o1[j]);
				dst += plane_stride;
			}
		}
	}
} /* namespace f43 */

#endif /* B200_WINOGRAD_F43_CUH_ */
