/*
 * winograd_fused_f23_tc.cu -- the contraction and the output transform of the one-call F(2x2,3x3) Winograd convolution
 * in ONE kernel: the transform-domain products never leave the SM.
 *
 * The chained form of cudaConvolutionWinogradFusedForward writes M[16][tiles][K] to memory in the batched GEMM and
 * reads it back in the output transform; with float16 tensors every stage of that chain runs at the speed of HBM, and
 * M is 4/9 of all the bytes moved.  Here the 16 products of a block of tiles stay in TMEM:
 *
 *   y(tile) = A^T M A   (A^T is 2 x 4)      =>      y[a][b] = sum_nu ( sum_xi A^T[a][xi] M[xi][nu] ) A^T[b][nu]
 *
 * so the planes are taken in four groups of constant nu.  One work item = 128 tiles x 64 filters:
 *   warp 0      TMA producer: for nu, channel block, pair of xi: two planes V[xi*4+nu] (128 tiles x 64 channels each) and
 *               U[xi*4+nu] (64 filters x 64 channels each) into one of four 128-byte-swizzled stages
 *   warp 1      one thread issues tcgen05.mma (M = 128, N = 64) into the group's four accumulators (4 x 64 TMEM columns);
 *               two groups fit TMEM, so the next group is contracted while the previous one is drained
 *   warps 2..9  drain a group (tcgen05.ld), apply the column transform over xi, and add the group's contribution to
 *               the 2 x 2 outputs of their tile, which live in registers (float32) across the four groups; after the
 *               fourth group: alpha1 * y + bias + alpha2 * z -> activation -> + beta * y, rounded once, 16-byte stores
 *
 * The reference's fused kernel (src/winograd_fused.cu:587-775) was meant to do the same with CUDA-core FMAs on one
 * 8 x 8 x 32 block per CTA and was left unfinished.
 *
 * Bound: HBM.  Per item V is 16 x 128 x C x 2 bytes against 2 x 16 x 128 x C x 64 flop, 16 flop per byte.
 */
#include "conv_kernels.hpp"
#include "winograd_internal.hpp"
#include "umma.cuh"
#include "winograd_tables.cuh"

#include <algorithm>
#include <cstdlib>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;
	using namespace bk;

	constexpr int kBlockTiles = 128;
	constexpr int kBlockFilters = 64;
	constexpr int kBlockChannels = 64; /* 128 bytes of float16 */
	/* A stage holds the operands of two of the four planes of a group for one block of 64 channels: four stages of 48 KB.
	 * What sets the size: the thread that issues the MMAs pays about 100 cycles for a wait on a full barrier and 120 for a
	 * commit, and no MMA of M = 128 retires in less than 86 cycles whatever its N, so a stage has to carry several MMAs
	 * (eight here); and a stage stays occupied for the ~1700 cycles its copies take to land plus the time its MMAs run,
	 * so the bytes in flight, not the size of a stage, bound the fill rate.  Measured on the 128 x 28 x 28 x 128 layer (this
	 * kernel alone, cold): 54 us with one plane per stage (eight stages of 24 KB), 40.5 us with the whole group per stage
	 * (two stages of 96 KB: only one stage is ever in flight while the other is read; 4800 cycles per group), 35-36 us
	 * with this form (3800 cycles per group). */
	constexpr int kStagePlanes = 2;
	constexpr int kStages = 4;
	constexpr int kABytes = kBlockTiles * 128;
	constexpr int kBBytes = kBlockFilters * 128;
	constexpr int kStageBytes = kStagePlanes * (kABytes + kBBytes);
	constexpr int kSmemBytes = kStages * kStageBytes + 1024;
	constexpr int kGroupColumns = 4 * kBlockFilters; /* four planes of one group */
	constexpr int kTmemColumns = 2 * kGroupColumns;
	constexpr int kEpilogueWarps = 8;
	constexpr int kEpilogueThreads = kEpilogueWarps * 32;
	constexpr int kThreads = 64 + kEpilogueThreads;
	constexpr int kFiltersPerThread = kBlockFilters / (kEpilogueWarps / 4); /* 32 */

	struct F23Params
	{
			int tiles, filters, channels;
			int tiles_h, tiles_w, height, width;
			int filter_blocks, channel_blocks, num_items;
			int last_tile_block; /* items walk the blocks of tiles from this one down to the first */
			const float *bias;
			const void *z;
			void *y;
			float alpha1, alpha2, beta;
			int activation;
			int wide_stores; /* y is 32-byte aligned and K a multiple of 16: 16 filters of a pixel go out as one 32-byte store */
	};

	__device__ __noinline__ float activation_slow(avActivationType_t activation, float x)
	{
		return activation_forward(activation, x);
	}

	__device__ __forceinline__ uint32_t pack2(float a, float b, half)
	{
		__half2 v = __floats2half2_rn(a, b);
		return *reinterpret_cast<uint32_t*>(&v);
	}
	__device__ __forceinline__ uint32_t pack2(float a, float b, __nv_bfloat16)
	{
		__nv_bfloat162 v = __floats2bfloat162_rn(a, b);
		return *reinterpret_cast<uint32_t*>(&v);
	}
	__device__ __forceinline__ float2 unpack2(uint32_t raw, half)
	{
		return __half22float2(*reinterpret_cast<__half2*>(&raw));
	}
	__device__ __forceinline__ float2 unpack2(uint32_t raw, __nv_bfloat16)
	{
		return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw));
	}

	/* 32 bytes (16 values of a 16-bit type) with one instruction: a whole sector per lane */
	__device__ __forceinline__ void store_256(void *dst, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t w4, uint32_t w5, uint32_t w6, uint32_t w7)
	{
		asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
				::"l"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3), "r"(w4), "r"(w5), "r"(w6), "r"(w7) : "memory");
	}

	__device__ __forceinline__ void tmem_load_32x8(uint32_t taddr, float (&r)[8])
	{
		uint32_t u[8];
		asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
				: "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]) : "r"(taddr) : "memory");
#pragma unroll
		for (int i = 0; i < 8; i++)
			r[i] = __uint_as_float(u[i]);
	}

	/* A^T of F(2x2,3x3) as the transform tables define it (2 x 4); zero and unit coefficients fold away at compile time */
	__host__ __device__ constexpr float at(int row, int col)
	{
		return static_cast<float>(winograd::Coefficients<2, 3>::output(row, col));
	}
	__device__ __forceinline__ float column_transform(int a, float m0, float m1, float m2, float m3)
	{
		/* sum over xi of A^T[a][xi] * M[xi][nu] */
		float t = 0.0f;
		const float m[4] = { m0, m1, m2, m3 };
#pragma unroll
		for (int xi = 0; xi < 4; xi++)
		{
			const float c = (a == 0) ? at(0, xi) : at(1, xi);
			if (c == 1.0f)
				t += m[xi];
			else if (c == -1.0f)
				t -= m[xi];
			else if (c != 0.0f)
				t = fmaf(c, m[xi], t);
		}
		return t;
	}

	/* adds group NU's contribution to the four outputs: out[a][b] (+)= T[a] * A^T[b][NU]; group 0 initialises */
	template<int NU>
	__device__ __forceinline__ void accumulate_group(float (&out)[2][2][kFiltersPerThread], int k, float t0, float t1)
	{
#pragma unroll
		for (int b = 0; b < 2; b++)
		{
			constexpr float c0 = at(0, NU), c1 = at(1, NU);
			const float c = (b == 0) ? c0 : c1;
			if (NU == 0)
			{
				out[0][b][k] = c * t0;
				out[1][b][k] = c * t1;
			}
			else if (c != 0.0f)
			{
				out[0][b][k] = fmaf(c, t0, out[0][b][k]);
				out[1][b][k] = fmaf(c, t1, out[1][b][k]);
			}
		}
	}

	/* drains the four accumulators of one group for this thread's tile and 32 filters */
	template<int NU>
	__device__ __forceinline__ void drain_group(uint32_t taddr, float (&out)[2][2][kFiltersPerThread])
	{
#pragma unroll
		for (int s = 0; s < kFiltersPerThread / 8; s++)
		{
			float m0[8], m1[8], m2[8], m3[8];
			tmem_load_32x8(taddr + 0 * kBlockFilters + s * 8, m0);
			tmem_load_32x8(taddr + 1 * kBlockFilters + s * 8, m1);
			tmem_load_32x8(taddr + 2 * kBlockFilters + s * 8, m2);
			tmem_load_32x8(taddr + 3 * kBlockFilters + s * 8, m3);
			umma::tmem_load_wait();
#pragma unroll
			for (int j = 0; j < 8; j++)
			{
				const float t0 = column_transform(0, m0[j], m1[j], m2[j], m3[j]);
				const float t1 = column_transform(1, m0[j], m1[j], m2[j], m3[j]);
				accumulate_group<NU>(out, s * 8 + j, t0, t1);
			}
		}
	}

	/* SIMPLE: no z, beta == 0, linear or relu activation -- the epilogue of the common inference layer, without the
	 * per-vector decisions of the general form */
	template<typename T, bool SIMPLE>
	__global__ void __launch_bounds__(kThreads, 1) kernel_f23_contract_output(const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapU,
			F23Params p, int *deviceStatus)
	{
		extern __shared__ uint8_t smem_raw[];
		uint8_t *smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

		__shared__ __align__(8) uint64_t full_bar[kStages];
		__shared__ __align__(8) uint64_t empty_bar[kStages];
		__shared__ __align__(8) uint64_t tmem_full_bar[2];
		__shared__ __align__(8) uint64_t tmem_empty_bar[2];
		__shared__ uint32_t tmem_base_slot;
		__shared__ int abort_flag;
		__shared__ volatile int epilogue_go;
		__shared__ __align__(16) float bias_s[kBlockFilters];

		const int warp = threadIdx.x / 32;
		const int lane = threadIdx.x % 32;

		if (threadIdx.x == 0)
		{
			abort_flag = 0;
			for (int s = 0; s < kStages; s++)
			{
				umma::mbar_init(&full_bar[s], 1);
				umma::mbar_init(&empty_bar[s], 1);
			}
			for (int a = 0; a < 2; a++)
			{
				umma::mbar_init(&tmem_full_bar[a], 1);
				umma::mbar_init(&tmem_empty_bar[a], kEpilogueThreads);
			}
			umma::mbar_fence_init();
			umma::prefetch_tensormap(&mapV);
			umma::prefetch_tensormap(&mapU);
		}
		if (warp == 1)
		{
			umma::tmem_alloc(&tmem_base_slot, kTmemColumns);
			umma::tmem_relinquish();
		}
		umma::tcgen05_fence_before();
		__syncthreads();
		umma::tcgen05_fence_after();
		const uint32_t tmem_base = tmem_base_slot;
		volatile int *abort_ptr = &abort_flag;
		/* everything above touched only this CTA's own resources; V and U come from the kernels before this one */
		chain_wait();
		chain_release();

		if (warp == 0)
		{
			if (lane == 0)
			{
				int stage = 0;
				uint32_t phase = 0;
				bool ok = true;
				for (int item = blockIdx.x; item < p.num_items and ok; item += gridDim.x)
				{
					const int fb = item % p.filter_blocks;
					const int tb = p.last_tile_block - item / p.filter_blocks;
					/* plain nested counters: this thread's own instruction latency bounds how fast stages can be issued, and an
					 * integer division costs it more than the copy it is about to start */
					for (int nu = 0; nu < 4 and ok; nu++)
						for (int cb = 0; cb < p.channel_blocks and ok; cb++)
							for (int half = 0; half < 4 / kStagePlanes; half++)
							{
								if (not umma::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_ptr))
								{
									umma::raise_error(abort_ptr, deviceStatus, umma::kErrorStageWait);
									ok = false;
									break;
								}
								uint8_t *a_dst = smem + stage * kStageBytes;
								uint8_t *b_dst = a_dst + kStagePlanes * kABytes;
								umma::mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
#pragma unroll
								for (int j = 0; j < kStagePlanes; j++)
								{
									const int plane = (half * kStagePlanes + j) * 4 + nu;
									umma::tma_load_3d(a_dst + j * kABytes, &mapV, &full_bar[stage], cb * kBlockChannels, tb * kBlockTiles, plane);
									umma::tma_load_3d(b_dst + j * kBBytes, &mapU, &full_bar[stage], cb * kBlockChannels, fb * kBlockFilters, plane);
								}
								if (++stage == kStages)
								{
									stage = 0;
									phase ^= 1u;
								}
							}
				}
			}
		}
		else if (warp == 1)
		{
			if (lane == 0)
			{
				constexpr uint32_t idesc = umma::make_instr_desc(umma::kAccumF32, umma::kFormatF16, umma::kFormatF16, false, false, kBlockTiles, kBlockFilters);
				int stage = 0;
				uint32_t phase = 0;
				const uint64_t a_desc0 = umma::make_smem_desc(umma::smem_u32(smem), 16, 1024, umma::kSwizzle128B);
				int group = 0; /* counts groups over all items: accumulator buffer = group & 1 */
				bool ok = true;
				for (int item = blockIdx.x; item < p.num_items and ok; item += gridDim.x)
				{
					for (int nu = 0; nu < 4 and ok; nu++, group++)
					{
						const int buf = group & 1;
						const uint32_t buf_phase = static_cast<uint32_t>(group >> 1) & 1u;
						if (not umma::mbar_wait(&tmem_empty_bar[buf], buf_phase ^ 1u, abort_ptr))
						{
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorMmaWait);
							ok = false;
							break;
						}
						umma::tcgen05_fence_after();
						const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kGroupColumns);
						for (int cb = 0; cb < p.channel_blocks and ok; cb++)
							for (int half = 0; half < 4 / kStagePlanes; half++)
							{
								if (not umma::mbar_wait(&full_bar[stage], phase, abort_ptr))
								{
									umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
									ok = false;
									break;
								}
								umma::tcgen05_fence_after();
								/* the address field counts 16-byte units; per plane the four 32-byte steps of the 128-byte swizzle row
								 * go out as one instruction sequence */
								static_assert(kBlockChannels / 16 == 4, "a plane's channel block is four MMAs deep");
								const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage * (kStageBytes / 16));
								const uint64_t b_desc = a_desc + static_cast<uint64_t>(kStagePlanes * (kABytes / 16));
#pragma unroll
								for (int j = 0; j < kStagePlanes; j++)
									umma::mma_f16_k4(tmem_d + static_cast<uint32_t>((half * kStagePlanes + j) * kBlockFilters),
											a_desc + static_cast<uint64_t>(j * (kABytes / 16)), b_desc + static_cast<uint64_t>(j * (kBBytes / 16)), idesc, cb != 0);
								umma::mma_commit(&empty_bar[stage]);
								if (++stage == kStages)
								{
									stage = 0;
									phase ^= 1u;
								}
							}
						if (ok)
							umma::mma_commit(&tmem_full_bar[buf]);
					}
				}
			}
		}
		else
		{
			const int quarter = warp % 4; /* the TMEM lanes this warp may read */
			const int half_block = (warp - 2) / 4; /* which 32 of the 64 filters */
			const int row = quarter * 32 + lane;
			const int epi_thread = threadIdx.x - 64;
			const avActivationType_t activation = static_cast<avActivationType_t>(p.activation);
			const int tiles_per_image = p.tiles_h * p.tiles_w;
			int group = 0;
			int staged_fb = -1;
			bool ok = true;
			for (int item = blockIdx.x; item < p.num_items and ok; item += gridDim.x)
			{
				const int fb = item % p.filter_blocks;
				const int tb = p.last_tile_block - item / p.filter_blocks;
				/* the bias of this filter block, staged once per change of block (read after the fourth group) */
				if (staged_fb != fb)
				{
					if (staged_fb >= 0)
						umma::named_barrier_sync(3, kEpilogueThreads); /* nobody still reads the previous block's values */
					if (epi_thread < kBlockFilters)
					{
						const int k = fb * kBlockFilters + epi_thread;
						bias_s[epi_thread] = (p.bias != nullptr and k < p.filters) ? p.bias[k] : 0.0f;
					}
					staged_fb = fb;
				}
				float out[2][2][kFiltersPerThread];
#pragma unroll
				for (int nu = 0; nu < 4; nu++, group++)
				{
					const int buf = group & 1;
					const uint32_t buf_phase = static_cast<uint32_t>(group >> 1) & 1u;
					if (epi_thread == 0)
					{
						const bool ready = umma::mbar_wait(&tmem_full_bar[buf], buf_phase, abort_ptr);
						if (not ready)
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorEpilogueWait);
						epilogue_go = ready ? 1 : 0;
					}
					umma::named_barrier_sync(1, kEpilogueThreads);
					if (epilogue_go == 0)
					{
						ok = false;
						break;
					}
					umma::tcgen05_fence_after();
					const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16)
							+ static_cast<uint32_t>(buf * kGroupColumns + half_block * kFiltersPerThread);
					if (nu == 0)
						drain_group<0>(taddr, out);
					else if (nu == 1)
						drain_group<1>(taddr, out);
					else if (nu == 2)
						drain_group<2>(taddr, out);
					else
						drain_group<3>(taddr, out);
					umma::tcgen05_fence_before();
					umma::mbar_arrive(&tmem_empty_bar[buf]);
					/* epilogue_go is rewritten for the next group only after everybody has read it */
					umma::named_barrier_sync(2, kEpilogueThreads);
				}
				if (not ok)
					break;

				const int tile = tb * kBlockTiles + row;
				const int k0 = fb * kBlockFilters + half_block * kFiltersPerThread;
				if (tile >= p.tiles or k0 >= p.filters)
					continue;
				const int n = tile / tiles_per_image;
				const int rem = tile - n * tiles_per_image;
				const int th = rem / p.tiles_w;
				const int tw = rem - th * p.tiles_w;
				const T *z = reinterpret_cast<const T*>(p.z);
#pragma unroll
				for (int a = 0; a < 2; a++)
#pragma unroll
					for (int b = 0; b < 2; b++)
					{
						const int h = 2 * th + a, w = 2 * tw + b;
						if (h >= p.height or w >= p.width)
							continue;
						const size_t index = ((static_cast<size_t>(n) * p.height + h) * p.width + w) * p.filters + k0;
						T *dst = reinterpret_cast<T*>(p.y) + index;
						if constexpr (SIMPLE)
						{
							/* a scattered 16-byte store costs the load/store unit as much as a 32-byte one: with whole blocks of
							 * filters the thread's 32 values of this pixel leave as two 32-byte stores instead of four of 16 */
							if (p.wide_stores != 0 and k0 + kFiltersPerThread <= p.filters)
							{
								const bool relu = activation == AVOCADO_ACTIVATION_RELU;
#pragma unroll
								for (int v = 0; v < kFiltersPerThread / 16; v++)
								{
									uint32_t packed[8];
#pragma unroll
									for (int q = 0; q < 8; q++)
									{
										const int j = 16 * v + 2 * q;
										float r0 = fmaf(p.alpha1, out[a][b][j], bias_s[half_block * kFiltersPerThread + j]);
										float r1 = fmaf(p.alpha1, out[a][b][j + 1], bias_s[half_block * kFiltersPerThread + j + 1]);
										r0 = relu ? fmaxf(r0, 0.0f) : r0;
										r1 = relu ? fmaxf(r1, 0.0f) : r1;
										packed[q] = pack2(r0, r1, T());
									}
									store_256(dst + 16 * v, packed[0], packed[1], packed[2], packed[3], packed[4], packed[5], packed[6], packed[7]);
								}
								continue;
							}
						}
#pragma unroll
						for (int v = 0; v < kFiltersPerThread / 8; v++)
						{
							if (k0 + 8 * v + 8 > p.filters)
								continue;
							float r[8];
							const float4 b0 = *reinterpret_cast<const float4*>(bias_s + half_block * kFiltersPerThread + 8 * v);
							const float4 b1 = *reinterpret_cast<const float4*>(bias_s + half_block * kFiltersPerThread + 8 * v + 4);
							r[0] = fmaf(p.alpha1, out[a][b][8 * v + 0], b0.x);
							r[1] = fmaf(p.alpha1, out[a][b][8 * v + 1], b0.y);
							r[2] = fmaf(p.alpha1, out[a][b][8 * v + 2], b0.z);
							r[3] = fmaf(p.alpha1, out[a][b][8 * v + 3], b0.w);
							r[4] = fmaf(p.alpha1, out[a][b][8 * v + 4], b1.x);
							r[5] = fmaf(p.alpha1, out[a][b][8 * v + 5], b1.y);
							r[6] = fmaf(p.alpha1, out[a][b][8 * v + 6], b1.z);
							r[7] = fmaf(p.alpha1, out[a][b][8 * v + 7], b1.w);
							if constexpr (SIMPLE)
							{
								const bool relu = activation == AVOCADO_ACTIVATION_RELU;
#pragma unroll
								for (int q = 0; q < 8; q++)
									r[q] = relu ? fmaxf(r[q], 0.0f) : r[q]; /* a select, not a branch */
								*reinterpret_cast<uint4*>(dst + 8 * v) = make_uint4(pack2(r[0], r[1], T()), pack2(r[2], r[3], T()), pack2(r[4], r[5], T()),
										pack2(r[6], r[7], T()));
								continue;
							}
							if (z != nullptr)
							{
								const uint4 raw = *reinterpret_cast<const uint4*>(z + index + 8 * v);
								const uint32_t zw[4] = { raw.x, raw.y, raw.z, raw.w };
#pragma unroll
								for (int q = 0; q < 4; q++)
								{
									const float2 zz = unpack2(zw[q], T());
									r[2 * q] = fmaf(p.alpha2, zz.x, r[2 * q]);
									r[2 * q + 1] = fmaf(p.alpha2, zz.y, r[2 * q + 1]);
								}
							}
							if (activation == AVOCADO_ACTIVATION_RELU)
							{
#pragma unroll
								for (int q = 0; q < 8; q++)
									r[q] = fmaxf(r[q], 0.0f);
							}
							else if (activation != AVOCADO_ACTIVATION_LINEAR)
							{
#pragma unroll
								for (int q = 0; q < 8; q++)
									r[q] = activation_slow(activation, r[q]);
							}
							if (p.beta != 0.0f)
							{
								const uint4 raw = *reinterpret_cast<const uint4*>(dst + 8 * v);
								const uint32_t yw[4] = { raw.x, raw.y, raw.z, raw.w };
#pragma unroll
								for (int q = 0; q < 4; q++)
								{
									const float2 yy = unpack2(yw[q], T());
									r[2 * q] = fmaf(p.beta, yy.x, r[2 * q]);
									r[2 * q + 1] = fmaf(p.beta, yy.y, r[2 * q + 1]);
								}
							}
							*reinterpret_cast<uint4*>(dst + 8 * v) = make_uint4(pack2(r[0], r[1], T()), pack2(r[2], r[3], T()), pack2(r[4], r[5], T()),
									pack2(r[6], r[7], T()));
						}
					}
			}
		}

		__syncthreads();
		if (abort_flag != 0)
			umma::drain_after_abort();
		if (warp == 1)
		{
			umma::tcgen05_fence_after();
			umma::tmem_dealloc(tmem_base, kTmemColumns);
		}
	}

	template<typename T>
	avStatus_t launch_typed(ContextObject &ctx, const CUtensorMap &mapV, const CUtensorMap &mapU, const F23Params &p, int *deviceStatus)
	{
		const bool simple = p.z == nullptr and p.beta == 0.0f and (p.activation == AVOCADO_ACTIVATION_LINEAR or p.activation == AVOCADO_ACTIVATION_RELU);
		auto kernel = simple ? kernel_f23_contract_output<T, true> : kernel_f23_contract_output<T, false>;
		static PerDeviceOnce configured;
		if (configured.run(ctx.device, [&]() -> cudaError_t { { const cudaError_t e = cudaFuncSetAttribute(kernel_f23_contract_output<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes); if (e != cudaSuccess) return e; } return cudaFuncSetAttribute(kernel_f23_contract_output<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes); }) != cudaSuccess)
		{
			cudaGetLastError();
			return AVOCADO_STATUS_EXECUTION_FAILED;
		}
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		const int grid = std::min(p.num_items, sms);
		launch_chained(kernel, dim3(grid), dim3(kThreads), kSmemBytes, ctx.getStream(), mapV, mapU, p, deviceStatus);
		return checkForErrors();
	}
}

namespace bk
{
	bool winograd_f23_contract_output_covers(const ContextObject &ctx, const ConvArgs &args, avDataType_t yType, long long tiles)
	{
		if (cuda_sm_version(ctx.device) != 100)
			return false;
		if (yType != AVOCADO_DTYPE_FLOAT16 and yType != AVOCADO_DTYPE_BFLOAT16)
			return false;
		/* rows of V and U must be whole 16-byte units for TMA, outputs are stored 8 filters at a time */
		if (args.channels % 8 != 0 or args.filters % 8 != 0 or tiles > 0x7FFFFF00ll)
			return false;
		return reinterpret_cast<uintptr_t>(args.y) % 16 == 0 and (args.z == nullptr or reinterpret_cast<uintptr_t>(args.z) % 16 == 0)
				and (args.bias == nullptr or reinterpret_cast<uintptr_t>(args.bias) % 4 == 0);
	}

	avStatus_t winograd_f23_contract_output(ContextObject &ctx, const ConvArgs &args, avDataType_t yType, long long tiles, const void *vPtr, const void *uPtr,
			const void *alpha1, const void *alpha2, const void *beta, int *deviceStatus)
	{
		if (not winograd_f23_contract_output_covers(ctx, args, yType, tiles))
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (reinterpret_cast<uintptr_t>(vPtr) % 128 != 0 or reinterpret_cast<uintptr_t>(uPtr) % 128 != 0)
			return AVOCADO_STATUS_NOT_SUPPORTED;

		CUtensorMap mapV, mapU;
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(args.channels), static_cast<uint64_t>(tiles), 16 };
			const uint64_t strides[2] = { static_cast<uint64_t>(args.channels) * 2, static_cast<uint64_t>(tiles) * args.channels * 2 };
			const uint32_t box[3] = { kBlockChannels, kBlockTiles, 1 };
			if (not umma::make_tensor_map(&mapV, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(vPtr), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(args.channels), static_cast<uint64_t>(args.filters), 16 };
			const uint64_t strides[2] = { static_cast<uint64_t>(args.channels) * 2, static_cast<uint64_t>(args.filters) * args.channels * 2 };
			const uint32_t box[3] = { kBlockChannels, kBlockFilters, 1 };
			if (not umma::make_tensor_map(&mapU, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(uPtr), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}

		F23Params p;
		p.tiles = static_cast<int>(tiles);
		p.filters = args.filters;
		p.channels = args.channels;
		p.tiles_h = (args.height + 1) / 2;
		p.tiles_w = (args.width + 1) / 2;
		p.height = args.out_height;
		p.width = args.out_width;
		p.filter_blocks = (args.filters + kBlockFilters - 1) / kBlockFilters;
		p.channel_blocks = (args.channels + kBlockChannels - 1) / kBlockChannels;
		const long long items = ((tiles + kBlockTiles - 1) / kBlockTiles) * p.filter_blocks;
		if (items > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		p.num_items = static_cast<int>(items);
		/* the input transform wrote V front to back: its last blocks of tiles are the ones still in L2 (57.6 -> 56.9 us for the
		 * call on the 128 x 28 x 28 x 128 layer against walking them first to last) */
		p.last_tile_block = static_cast<int>(items / p.filter_blocks) - 1;
		p.bias = reinterpret_cast<const float*>(args.bias);
		p.z = args.z;
		p.y = args.y;
		p.alpha1 = getAlphaValue<float>(alpha1);
		p.alpha2 = getAlphaValue<float>(alpha2);
		p.beta = getBetaValue<float>(beta);
		p.activation = static_cast<int>(args.activation);
		p.wide_stores = (args.filters % 16 == 0 and reinterpret_cast<uintptr_t>(args.y) % 32 == 0) ? 1 : 0;
		if (yType == AVOCADO_DTYPE_FLOAT16)
			return launch_typed<half>(ctx, mapV, mapU, p, deviceStatus);
		return launch_typed<__nv_bfloat16>(ctx, mapV, mapU, p, deviceStatus);
	}
} /* namespace bk */
