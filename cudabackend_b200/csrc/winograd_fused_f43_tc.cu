/*
 * winograd_fused_f43_tc.cu -- the transform-domain contraction and the output transform of the non-fused F(4x4,3x3)
 * pipeline in ONE kernel, for 16-bit tensors: the 36 products M[xi][nu] of a block of tiles never leave the SM.
 *
 * The caller of the non-fused API issues cudaGemmBatched (M = V x U^T, reference src/gemm.cpp:126-209) and then
 * cudaWinogradOutputTransform (reference src/winograd_nonfused.cu:703-777) on M.  M is 36 * tiles * K values written
 * by one kernel and read by the next: 2 x 57.8 MB of the 283 MB a 64 x 56 x 56 x 64 float16 layer moves.  When the
 * context has fusion switched on (cudaContextSetWinogradFusion) the batched GEMM is held back, and the output
 * transform that consumes its result launches this kernel instead of both.
 *
 *   y(tile) = A^T M A   (A^T is 4 x 6)      =>      y[a][b] = sum_nu ( sum_xi A^T[a][xi] M[xi][nu] ) A^T[b][nu]
 *
 * so the planes are taken in six groups of constant nu.  One work item = 128 tiles x 16 filters:
 *   warp 0      TMA producer: for nu, xi, channel block: V[xi*6+nu] (128 tiles x 64 channels) and U[xi*6+nu]
 *               (16 filters x 64 channels) into a ring of 128-byte-swizzled stages
 *   warp 1      one thread issues tcgen05.mma (M = 128, N = 16) into the group's six accumulators (6 x 16 TMEM columns);
 *               five groups fit TMEM, so the following groups are contracted while earlier ones are drained and stored
 *   warps 4..11 drain a group (tcgen05.ld), apply the column transform over xi, and add the group's contribution to the
 *               outputs of their tile, which live in registers (float32) across the six groups: a thread owns two of the
 *               four output rows for all 16 filters; after the sixth group: alpha1 * y + bias + alpha2 * z -> activation ->
 *               + beta * y, rounded once, one 32-byte store (a whole sector) per pixel
 *
 * Why 16 filters: the 16 outputs of a (tile, filter) pair accumulate over all six groups, so an item needs
 * 16 float32 registers per pair; 128 x 16 pairs are half of the SM's register file.  The price is that a block of
 * tiles is fetched once per 16 filters (from L2 after the first time: items of one tile block run side by side).
 * The products are never rounded to 16 bits on the way, so the result is closer to the exact convolution than the
 * two-kernel form's.
 *
 * Bound: HBM (V is read once from memory: 36 * tiles * C * 2 bytes; y written once).
 */
#include "conv_kernels.hpp"
#include "winograd_internal.hpp"
#include "umma.cuh"
#include "winograd_f43.cuh"
#include "winograd_tables.cuh"

#include <algorithm>
#include <cstdlib>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;
	using namespace bk;
	using f43::f2;

	constexpr int kBlockTiles = 128;
	constexpr int kBlockFilters = 16;
	constexpr int kBlockChannels = 64; /* 128 bytes of a 16-bit type */
	constexpr int kGroupPlanes = 6;
	/* A stage holds the operands of ALL six planes of one group (for one block of 64 channels), and the MMAs of a stage are
	 * issued contraction step outermost, plane innermost, so that consecutive MMAs go to different accumulators and the
	 * producer moves 108 KB per barrier round trip.  Measured on the 64 x 56 x 56 x 64 layer, everything else equal: one
	 * plane per stage (four MMAs in a row into the same accumulator) 52.7 us, three planes 43.2 us, six planes 37.9 us. */
	constexpr int kStagePlanes = 6;
	constexpr int kStagesPerGroup = kGroupPlanes / kStagePlanes;
	constexpr int kABytes = kBlockTiles * 128;
	constexpr int kBBytes = kBlockFilters * 128;
	constexpr int kStageBytes = kStagePlanes * (kABytes + kBBytes);
	constexpr int kStages = (216 * 1024) / kStageBytes;
	constexpr int kSmemBytes = kStages * kStageBytes + 1024;
	static_assert(kGroupPlanes % kStagePlanes == 0 and kStages >= 2, "stage geometry");
	constexpr int kGroupPitch = kGroupPlanes * kBlockFilters; /* TMEM columns of one accumulator group: 96 */
	/* Five groups fit the 512 columns.  The epilogue warps spend longer storing an item's outputs (16 scattered 16-byte
	 * stores per thread) than draining a group, and nothing can be drained meanwhile: with a deep ring the MMAs of the
	 * next item run on through that time instead of stopping after two groups. */
	constexpr int kGroupBuffers = 5;
	constexpr int kTmemColumns = 512;
	static_assert(kGroupBuffers * kGroupPitch <= kTmemColumns, "accumulator ring exceeds TMEM");
	constexpr int kEpilogueWarps = 8;
	constexpr int kEpilogueThreads = kEpilogueWarps * 32;
	/* Three groups of four warps: {producer, MMA issuer, two idle warps} and two groups of epilogue warps.  Registers are
	 * handed out per group of four warps, so the first group gives most of its share back (setmaxnreg.dec) and the
	 * epilogue groups, whose 128 accumulators per thread do not fit the even share of 168, take it (setmaxnreg.inc). */
	constexpr int kControlThreads = 128;
	constexpr int kThreads = kControlThreads + kEpilogueThreads;
	constexpr int kControlRegisters = 40;
	constexpr int kEpilogueRegisters = 232;
	static_assert(kControlThreads * kControlRegisters + kEpilogueThreads * kEpilogueRegisters <= 65536, "register file");
	/* An epilogue thread owns one tile, two of its four output rows (a = h and a = h + 2, h = which half of the warps) and
	 * all 16 filters: 2 x 4 pixels x 16 filters = 128 float32 accumulators, and every pixel it stores is a whole 32-byte
	 * sector.  Rows {0, 2} need only the sums m1+m2, m3+m4 of the column transform and rows {1, 3} only the differences,
	 * so splitting by rows costs no arithmetic twice. */
	constexpr int kPairsPerThread = kBlockFilters / 2; /* filter pairs (packed float32x2) */

	struct F43Params
	{
			int tiles, filters, channels;
			int tiles_h, tiles_w, height, width;
			int filter_blocks, channel_blocks, num_items;
			const float *bias;
			const void *z;
			void *y;
			float alpha1, alpha2, beta;
			int activation;
			int wide_stores; /* y (and z) are 32-byte aligned and K is a multiple of 16: a pixel's 16 filters go out as one 32-byte store */
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

	/* 32 lanes x 4 consecutive 32-bit columns */
	__device__ __forceinline__ void tmem_load_32x4(uint32_t taddr, float (&r)[4])
	{
		uint32_t u[4];
		asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]) : "r"(taddr) : "memory");
#pragma unroll
		for (int i = 0; i < 4; i++)
			r[i] = __uint_as_float(u[i]);
	}

	/* A^T of F(4x4,3x3) as the transform tables define it (4 x 6) */
	__host__ __device__ constexpr float at(int row, int col)
	{
		return static_cast<float>(winograd::Coefficients<4, 3>::output(row, col));
	}

	/* adds group NU's contribution to the 2 x 4 outputs of one filter pair: out[i][b] (+)= T[i] * A^T[b][NU]; group 0 initialises */
	template<int NU>
	__device__ __forceinline__ void accumulate_group(f2 (&out)[2][4][kPairsPerThread], int pair, const f2 (&t)[2])
	{
#pragma unroll
		for (int b = 0; b < 4; b++)
		{
			constexpr float c0 = at(0, NU), c1 = at(1, NU), c2 = at(2, NU), c3 = at(3, NU);
			const float c = (b == 0) ? c0 : (b == 1) ? c1 : (b == 2) ? c2 : c3;
#pragma unroll
			for (int i = 0; i < 2; i++)
			{
				if (NU == 0)
					out[i][b][pair] = (c == 1.0f) ? t[i] : (c == 0.0f) ? f43::splat(0.0f) : f43::mul2(f43::splat(c), t[i]);
				else if (c == 1.0f)
					out[i][b][pair] = f43::add2(out[i][b][pair], t[i]);
				else if (c == -1.0f)
					out[i][b][pair] = f43::sub2(out[i][b][pair], t[i]);
				else if (c != 0.0f)
					out[i][b][pair] = f43::fma2(f43::splat(c), t[i], out[i][b][pair]);
			}
		}
	}

	/* Column transform (sum over xi of A^T[a][xi] * M[xi][nu]) for the two rows of one half, in the factored form of
	 * f43::output_1d: HALF 0 gives rows a = 0 and 2, HALF 1 rows a = 1 and 3. */
	template<int HALF>
	__device__ __forceinline__ void column_transform(const f2 (&m)[kGroupPlanes], f2 (&t)[2])
	{
		if (HALF == 0)
		{
			const f2 s = f43::add2(m[1], m[2]);
			const f2 u = f43::add2(m[3], m[4]);
			t[0] = f43::fma2(f43::splat(0.25f), u, f43::add2(m[0], s));
			t[1] = f43::add2(s, u);
		}
		else
		{
			const f2 d = f43::sub2(m[1], m[2]);
			const f2 v = f43::sub2(m[3], m[4]);
			t[0] = f43::fma2(f43::splat(0.5f), v, d);
			t[1] = f43::fma2(f43::splat(2.0f), f43::add2(v, m[5]), d);
		}
	}

	/* drains the six accumulators of one group for this thread's tile (all 16 filters) and its two rows */
	template<int NU, int HALF>
	__device__ __forceinline__ void drain_group(uint32_t taddr, f2 (&out)[2][4][kPairsPerThread])
	{
#pragma unroll
		for (int s = 0; s < kBlockFilters / 4; s++)
		{
			float m[kGroupPlanes][4];
#pragma unroll
			for (int xi = 0; xi < kGroupPlanes; xi++)
				tmem_load_32x4(taddr + xi * kBlockFilters + s * 4, m[xi]);
			umma::tmem_load_wait();
#pragma unroll
			for (int j = 0; j < 2; j++)
			{
				f2 column[kGroupPlanes], t[2];
#pragma unroll
				for (int xi = 0; xi < kGroupPlanes; xi++)
					column[xi] = f43::make_f2(m[xi][2 * j], m[xi][2 * j + 1]);
				column_transform<HALF>(column, t);
				accumulate_group<NU>(out, s * 2 + j, t);
			}
		}
	}
	template<int HALF>
	__device__ __forceinline__ void drain_group_of(int nu, uint32_t taddr, f2 (&out)[2][4][kPairsPerThread])
	{
		if (nu == 0)
			drain_group<0, HALF>(taddr, out);
		else if (nu == 1)
			drain_group<1, HALF>(taddr, out);
		else if (nu == 2)
			drain_group<2, HALF>(taddr, out);
		else if (nu == 3)
			drain_group<3, HALF>(taddr, out);
		else if (nu == 4)
			drain_group<4, HALF>(taddr, out);
		else
			drain_group<5, HALF>(taddr, out);
	}

	/* 32 bytes (16 values of a 16-bit type) with one instruction: a whole sector per lane */
	__device__ __forceinline__ void store_256(void *dst, const uint32_t (&w)[8])
	{
		asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
				::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
	}
	__device__ __forceinline__ void load_256(const void *src, uint32_t (&w)[8])
	{
		asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
				: "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "l"(src) : "memory");
	}

	/* SIMPLE: no z, beta == 0, linear or relu activation -- the epilogue of the common inference layer, without the
	 * per-vector decisions of the general form */
	template<typename T, bool IS_BF16_DOMAIN, bool SIMPLE>
	__global__ void __launch_bounds__(kThreads, 1) kernel_f43_contract_output(const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapU,
			F43Params p, int *deviceStatus)
	{
		extern __shared__ uint8_t smem_raw[];
		uint8_t *smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

		__shared__ __align__(8) uint64_t full_bar[kStages];
		__shared__ __align__(8) uint64_t empty_bar[kStages];
		__shared__ __align__(8) uint64_t tmem_full_bar[kGroupBuffers];
		__shared__ __align__(8) uint64_t tmem_empty_bar[kGroupBuffers];
		__shared__ uint32_t tmem_base_slot;
		__shared__ int abort_flag;
		__shared__ volatile int epilogue_go;

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
			for (int a = 0; a < kGroupBuffers; a++)
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

		if (warp < kControlThreads / 32)
		{
			asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegisters));
		}
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
					const int tb = item / p.filter_blocks;
					/* plain nested counters: this thread's own instruction latency bounds how fast stages can be issued */
					for (int nu = 0; nu < kGroupPlanes and ok; nu++)
						for (int part = 0; part < kStagesPerGroup and ok; part++)
							for (int cb = 0; cb < p.channel_blocks; cb++)
							{
								{
									const bool got = umma::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_ptr);
									if (not got)
									{
										umma::raise_error(abort_ptr, deviceStatus, umma::kErrorStageWait);
										ok = false;
										break;
									}
								}
								uint8_t *a_dst = smem + stage * kStageBytes;
								uint8_t *b_dst = a_dst + kStagePlanes * kABytes;
								umma::mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
#pragma unroll
								for (int q = 0; q < kStagePlanes; q++)
								{
									const int plane = (part * kStagePlanes + q) * 6 + nu; /* xi * 6 + nu */
									umma::tma_load_3d(a_dst + q * kABytes, &mapV, &full_bar[stage], cb * kBlockChannels, tb * kBlockTiles, plane);
									umma::tma_load_3d(b_dst + q * kBBytes, &mapU, &full_bar[stage], cb * kBlockChannels, fb * kBlockFilters, plane);
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
				constexpr uint32_t format = IS_BF16_DOMAIN ? umma::kFormatBF16 : umma::kFormatF16;
				constexpr uint32_t idesc = umma::make_instr_desc(umma::kAccumF32, format, format, false, false, kBlockTiles, kBlockFilters);
				int stage = 0;
				uint32_t phase = 0;
				const uint64_t a_desc0 = umma::make_smem_desc(umma::smem_u32(smem), 16, 1024, umma::kSwizzle128B);
				int buf = 0; /* accumulator groups are used round robin over all items */
				uint32_t buf_phase = 0;
				bool ok = true;
				for (int item = blockIdx.x; item < p.num_items and ok; item += gridDim.x)
				{
					for (int nu = 0; nu < kGroupPlanes and ok; nu++)
					{
						{
							const bool got = umma::mbar_wait(&tmem_empty_bar[buf], buf_phase ^ 1u, abort_ptr);
							if (not got)
							{
								umma::raise_error(abort_ptr, deviceStatus, umma::kErrorMmaWait);
								ok = false;
								break;
							}
						}
						umma::tcgen05_fence_after();
						for (int part = 0; part < kStagesPerGroup and ok; part++)
						{
							const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kGroupPitch + part * kStagePlanes * kBlockFilters);
							for (int cb = 0; cb < p.channel_blocks; cb++)
							{
								{
									const bool got = umma::mbar_wait(&full_bar[stage], phase, abort_ptr);
									if (not got)
									{
										umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
										ok = false;
										break;
									}
								}
								umma::tcgen05_fence_after();
								/* the address field counts 16-byte units; a 16-element step along the contraction is 32 bytes of
								 * the 128-byte swizzle row.  Issue order: contraction step outermost, plane innermost, so that an
								 * accumulator is touched again only after the other planes of the stage */
								const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage * (kStageBytes / 16));
								const uint64_t b_desc = a_desc + static_cast<uint64_t>(kStagePlanes * (kABytes / 16));
#pragma unroll
								for (int ks = 0; ks < kBlockChannels / 16; ks++)
#pragma unroll
									for (int q = 0; q < kStagePlanes; q++)
										umma::mma_f16(tmem_d + static_cast<uint32_t>(q * kBlockFilters), a_desc + static_cast<uint64_t>(q * (kABytes / 16) + 2 * ks),
												b_desc + static_cast<uint64_t>(q * (kBBytes / 16) + 2 * ks), idesc, cb != 0 or ks != 0);
								umma::mma_commit(&empty_bar[stage]);
								if (++stage == kStages)
								{
									stage = 0;
									phase ^= 1u;
								}
							}
						}
						if (ok)
							umma::mma_commit(&tmem_full_bar[buf]);
						if (++buf == kGroupBuffers)
						{
							buf = 0;
							buf_phase ^= 1u;
						}
					}
				}
			}
		}
		else if (warp >= kControlThreads / 32)
		{
			asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpilogueRegisters));
			const int quarter = warp % 4; /* the TMEM lanes this warp may read */
			const int half = (warp - kControlThreads / 32) / 4; /* 0: output rows 0 and 2 of the tile, 1: rows 1 and 3 */
			const int row = quarter * 32 + lane;
			const int epi_thread = threadIdx.x - kControlThreads;
			const avActivationType_t activation = static_cast<avActivationType_t>(p.activation);
			const int tiles_per_image = p.tiles_h * p.tiles_w;
			int buf = 0;
			uint32_t buf_phase = 0;
			bool ok = true;
			for (int item = blockIdx.x; item < p.num_items and ok; item += gridDim.x)
			{
				const int fb = item % p.filter_blocks;
				const int tb = item / p.filter_blocks;
				f2 out[2][4][kPairsPerThread];
#pragma unroll 1
				for (int nu = 0; nu < kGroupPlanes; nu++)
				{
					/* one thread waits and publishes the outcome, so that all eight warps take the same branch */
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
					const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * kGroupPitch);
					if (half == 0)
						drain_group_of<0>(nu, taddr, out);
					else
						drain_group_of<1>(nu, taddr, out);
					umma::tcgen05_fence_before();
					umma::mbar_arrive(&tmem_empty_bar[buf]);
					/* epilogue_go is rewritten for the next group only after everybody has read it */
					umma::named_barrier_sync(2, kEpilogueThreads);
					if (++buf == kGroupBuffers)
					{
						buf = 0;
						buf_phase ^= 1u;
					}
				}
				if (not ok)
					break;

				const int tile = tb * kBlockTiles + row;
				const int k0 = fb * kBlockFilters;
				if (tile >= p.tiles or k0 >= p.filters)
					continue;
				/* the last filter block may hold 8 filters only (K is a multiple of 8, not necessarily of 16) */
				const bool whole = (k0 + kBlockFilters <= p.filters) and p.wide_stores != 0;
				const bool upper = (k0 + kBlockFilters <= p.filters);
				const int n = tile / tiles_per_image;
				const int rem = tile - n * tiles_per_image;
				const int th = rem / p.tiles_w;
				const int tw = rem - th * p.tiles_w;
				const T *z = reinterpret_cast<const T*>(p.z);
				/* the bias as packed pairs, multiplied in with one packed FMA per filter pair */
				f2 bias2[kPairsPerThread];
#pragma unroll
				for (int q = 0; q < kBlockFilters / 4; q++)
				{
					float4 bq = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
					if (p.bias != nullptr and (q < 2 or upper))
						bq = __ldg(reinterpret_cast<const float4*>(p.bias + k0 + 4 * q));
					bias2[2 * q] = f43::make_f2(bq.x, bq.y);
					bias2[2 * q + 1] = f43::make_f2(bq.z, bq.w);
				}
				const f2 alpha1_2 = f43::splat(p.alpha1);
				const bool relu = activation == AVOCADO_ACTIVATION_RELU;
#pragma unroll
				for (int i = 0; i < 2; i++)
#pragma unroll
					for (int b = 0; b < 4; b++)
					{
						const int h = 4 * th + half + 2 * i, w = 4 * tw + b;
						if (h >= p.height or w >= p.width)
							continue;
						const size_t index = ((static_cast<size_t>(n) * p.height + h) * p.width + w) * p.filters + k0;
						T *dst = reinterpret_cast<T*>(p.y) + index;
						uint32_t packed[8];
						if constexpr (SIMPLE)
						{
#pragma unroll
							for (int q = 0; q < kPairsPerThread; q++)
							{
								const float2 v = f43::to_float2(f43::fma2(alpha1_2, out[i][b][q], bias2[q]));
								/* a select, not a branch */
								packed[q] = pack2(relu ? fmaxf(v.x, 0.0f) : v.x, relu ? fmaxf(v.y, 0.0f) : v.y, T());
							}
						}
						else
						{
							uint32_t zw[8] = { }, yw[8] = { };
							if (z != nullptr)
							{
								if (whole)
									load_256(z + index, zw);
								else
								{
									const uint4 lo = *reinterpret_cast<const uint4*>(z + index);
									zw[0] = lo.x, zw[1] = lo.y, zw[2] = lo.z, zw[3] = lo.w;
									if (upper)
									{
										const uint4 hi = *reinterpret_cast<const uint4*>(z + index + 8);
										zw[4] = hi.x, zw[5] = hi.y, zw[6] = hi.z, zw[7] = hi.w;
									}
								}
							}
							if (p.beta != 0.0f)
							{
								const uint4 lo = *reinterpret_cast<const uint4*>(dst);
								yw[0] = lo.x, yw[1] = lo.y, yw[2] = lo.z, yw[3] = lo.w;
								if (upper)
								{
									const uint4 hi = *reinterpret_cast<const uint4*>(dst + 8);
									yw[4] = hi.x, yw[5] = hi.y, yw[6] = hi.z, yw[7] = hi.w;
								}
							}
#pragma unroll
							for (int q = 0; q < kPairsPerThread; q++)
							{
								float2 v = f43::to_float2(f43::fma2(alpha1_2, out[i][b][q], bias2[q]));
								if (z != nullptr)
								{
									const float2 zz = unpack2(zw[q], T());
									v.x = fmaf(p.alpha2, zz.x, v.x);
									v.y = fmaf(p.alpha2, zz.y, v.y);
								}
								if (relu)
								{
									v.x = fmaxf(v.x, 0.0f);
									v.y = fmaxf(v.y, 0.0f);
								}
								else if (activation != AVOCADO_ACTIVATION_LINEAR)
								{
									v.x = activation_slow(activation, v.x);
									v.y = activation_slow(activation, v.y);
								}
								if (p.beta != 0.0f)
								{
									const float2 yy = unpack2(yw[q], T());
									v.x = fmaf(p.beta, yy.x, v.x);
									v.y = fmaf(p.beta, yy.y, v.y);
								}
								packed[q] = pack2(v.x, v.y, T());
							}
						}
						{
							if (whole)
								store_256(dst, packed);
							else
							{
								*reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
								if (upper)
									*reinterpret_cast<uint4*>(dst + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
							}
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

	template<typename T, bool IS_BF16_DOMAIN>
	avStatus_t launch_typed(ContextObject &ctx, const CUtensorMap &mapV, const CUtensorMap &mapU, const F43Params &p, int *deviceStatus)
	{
		const bool simple = p.z == nullptr and p.beta == 0.0f and (p.activation == AVOCADO_ACTIVATION_LINEAR or p.activation == AVOCADO_ACTIVATION_RELU);
		auto kernel = simple ? kernel_f43_contract_output<T, IS_BF16_DOMAIN, true> : kernel_f43_contract_output<T, IS_BF16_DOMAIN, false>;
		static PerDeviceOnce configured;
		if (configured.run(ctx.device, [&]() -> cudaError_t
		{
			cudaError_t e = cudaFuncSetAttribute(kernel_f43_contract_output<T, IS_BF16_DOMAIN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
			if (e != cudaSuccess)
				return e;
			return cudaFuncSetAttribute(kernel_f43_contract_output<T, IS_BF16_DOMAIN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
		}) != cudaSuccess)
		{
			cudaGetLastError();
			return AVOCADO_STATUS_EXECUTION_FAILED;
		}
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		const int grid = std::min(p.num_items, sms);
		const cudaError_t launched = launch_chained(kernel, dim3(grid), dim3(kThreads), kSmemBytes, ctx.getStream(), mapV, mapU, p, deviceStatus);
		if (launched != cudaSuccess)
			return convertStatus(launched);
		return checkForErrors();
	}
}


namespace bk
{
	avStatus_t winograd_f43_contract_output(ContextObject &ctx, const TensorObject &v, const void *vPtr, const TensorObject &u, const void *uPtr,
			const TensorObject &y, void *yPtr, const void *biasPtr, const void *zPtr, const void *alpha1, const void *alpha2, const void *beta,
			avActivationType_t activation, int *deviceStatus)
	{
		if (cuda_sm_version(ctx.device) != 100)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (y.dtype != AVOCADO_DTYPE_FLOAT16 and y.dtype != AVOCADO_DTYPE_BFLOAT16)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (v.dtype != u.dtype or (v.dtype != AVOCADO_DTYPE_FLOAT16 and v.dtype != AVOCADO_DTYPE_BFLOAT16))
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (v.nb_dims != 3 or u.nb_dims != 3 or y.nb_dims != 4 or v.dims[0] != 36 or u.dims[0] != 36 or v.dims[2] != u.dims[2] or y.dims[3] != u.dims[1])
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const int channels = v.dims[2], filters = u.dims[1];
		const long long tiles = static_cast<long long>(y.dims[0]) * ((y.dims[1] + 3) / 4) * ((y.dims[2] + 3) / 4);
		if (tiles != v.dims[1] or tiles == 0 or tiles > 0x7FFFFF00ll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		/* rows of V and U must be whole 16-byte units for TMA, outputs are stored 8 filters at a time */
		if (channels % 8 != 0 or filters % 8 != 0)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (reinterpret_cast<uintptr_t>(vPtr) % 16 != 0 or reinterpret_cast<uintptr_t>(uPtr) % 16 != 0 or reinterpret_cast<uintptr_t>(yPtr) % 16 != 0
				or (zPtr != nullptr and reinterpret_cast<uintptr_t>(zPtr) % 16 != 0) or (biasPtr != nullptr and reinterpret_cast<uintptr_t>(biasPtr) % 16 != 0))
			return AVOCADO_STATUS_NOT_SUPPORTED;

		const CUtensorMapDataType type = (v.dtype == AVOCADO_DTYPE_BFLOAT16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
		CUtensorMap mapV, mapU;
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(channels), static_cast<uint64_t>(tiles), 36 };
			const uint64_t strides[2] = { static_cast<uint64_t>(channels) * 2, static_cast<uint64_t>(tiles) * channels * 2 };
			const uint32_t box[3] = { kBlockChannels, kBlockTiles, 1 };
			if (not umma::make_tensor_map(&mapV, type, 3, const_cast<void*>(vPtr), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(channels), static_cast<uint64_t>(filters), 36 };
			const uint64_t strides[2] = { static_cast<uint64_t>(channels) * 2, static_cast<uint64_t>(filters) * channels * 2 };
			const uint32_t box[3] = { kBlockChannels, kBlockFilters, 1 };
			if (not umma::make_tensor_map(&mapU, type, 3, const_cast<void*>(uPtr), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}

		F43Params p;
		p.tiles = static_cast<int>(tiles);
		p.filters = filters;
		p.channels = channels;
		p.tiles_h = (y.dims[1] + 3) / 4;
		p.tiles_w = (y.dims[2] + 3) / 4;
		p.height = y.dims[1];
		p.width = y.dims[2];
		p.filter_blocks = (filters + kBlockFilters - 1) / kBlockFilters;
		p.channel_blocks = (channels + kBlockChannels - 1) / kBlockChannels;
		const long long items = ((tiles + kBlockTiles - 1) / kBlockTiles) * p.filter_blocks;
		if (items > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		p.num_items = static_cast<int>(items);
		p.bias = reinterpret_cast<const float*>(biasPtr);
		p.z = zPtr;
		p.y = yPtr;
		p.alpha1 = getAlphaValue<float>(alpha1);
		p.alpha2 = getAlphaValue<float>(alpha2);
		p.beta = getBetaValue<float>(beta);
		p.activation = static_cast<int>(activation);
		p.wide_stores = (filters % 16 == 0 and reinterpret_cast<uintptr_t>(yPtr) % 32 == 0 and (zPtr == nullptr or reinterpret_cast<uintptr_t>(zPtr) % 32 == 0)) ? 1 : 0;
		ctx.setDevice();
		const bool bf16_domain = (v.dtype == AVOCADO_DTYPE_BFLOAT16);
		if (y.dtype == AVOCADO_DTYPE_FLOAT16)
			return bf16_domain ? launch_typed<half, true>(ctx, mapV, mapU, p, deviceStatus) : launch_typed<half, false>(ctx, mapV, mapU, p, deviceStatus);
		return bf16_domain ? launch_typed<__nv_bfloat16, true>(ctx, mapV, mapU, p, deviceStatus) :
				launch_typed<__nv_bfloat16, false>(ctx, mapV, mapU, p, deviceStatus);
	}
} /* namespace bk */
