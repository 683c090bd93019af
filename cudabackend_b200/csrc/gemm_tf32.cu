/*
 * gemm_tf32.cu -- float32 batched contraction on the tensor cores.
 *
 * The reference runs float32 transform-domain products through cublasSgemmStridedBatched (src/gemm.cpp:178-185).  A
 * single TF32 pass is not accurate enough for Winograd F(4x4,3x3) (the 10-bit mantissa of the operands costs about
 * 4e-2), so every operand is used as a TF32 "hi" part (the landed float32 itself: the MMA ignores the 13 low mantissa
 * bits) plus a TF32 "lo" remainder written beside it, and the product is accumulated as
 * A_hi*B_hi + A_hi*B_lo + A_lo*B_hi  in float32 TMEM accumulators: per 8-deep slice one MMA of double width
 * (A_hi x [B_hi; B_lo]) and one of single width (A_lo x B_hi), error about 1e-6 relative.  The kernels are bound by
 * shared-memory bandwidth first (copy in, remainder out, operand reads), then by HBM.
 *
 * Roles of the 14 warps of a CTA (persistent over output tiles of 128 rows x BLOCK_N columns):
 *   warp 0      TMA producer: raw float32 tiles of A (128 x 32) and B (BLOCK_N x 32) into a ring of stages
 *   warps 2-9   splitters: leave each landed tile as the hi part and write its lo remainder beside it, fence for the async proxy;
 *               every warp waits for the stage by itself and owns a fixed share of it (no barrier between them)
 *   warp 1      issues the MMAs for a stage once it is split, releases the stage when they complete
 *   warps 10-13 epilogue: tcgen05.ld -> alpha -> 128-byte-swizzled shared memory -> TMA store
 *
 * op(B) = B (the dX contraction of the Winograd backward pass, where B is the small transformed filter tensor) is
 * served by transposing B into the context's scratch buffer first.
 */
#include "gemm_internal.hpp"
#include "umma.cuh"

#include <algorithm>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;
	using bk::GemmShape;

	constexpr int kBlockM = 128;
	constexpr int kBlockK = 32; /* float32 elements: 128 bytes */
	/* warp 0 producer, warp 1 MMA issuer, then the split warps, then four epilogue warps.  Eight split warps: with four,
	 * rewriting a stage (24-32 KB, about 20 instructions per 16 bytes) took one warp per scheduler longer than the three
	 * MMAs per slice that consume it, and the split was the pace-setter of both kernels. */
	constexpr int kSplitWarps = 8;
	constexpr int kSplitThreads = kSplitWarps * 32;
	constexpr int kThreads = 64 + kSplitThreads + 128;

	template<int BLOCK_N, int STAGES>
	struct Config
	{
			static constexpr int kATile = kBlockM * 128;
			static constexpr int kBTile = BLOCK_N * 128;
			/* per stage: A hi (landing buffer), A lo, B hi (landing buffer), B lo */
			static constexpr int kStageBytes = 2 * kATile + 2 * kBTile;
			static constexpr int kLoadBytes = kATile + kBTile;
			static constexpr int kSubTiles = BLOCK_N / 32;
			static constexpr int kCBytes = kSubTiles * kBlockM * 128;
			static constexpr int kSmemBytes = STAGES * kStageBytes + kCBytes + 1024;
			static constexpr int kTmemColumns = 4 * BLOCK_N; /* two accumulators of 2 * BLOCK_N columns */
	};

	/* x rounded to TF32 (10 explicit mantissa bits), ties away from zero like cvt.rna.tf32.f32, with two integer
	 * operations: the conversion instruction runs on the slow conversion pipe, and the splitter warps execute it for
	 * every operand element, which made them the pace-setter of the whole kernel. */
	__device__ __forceinline__ uint32_t to_tf32(float x)
	{
		return (__float_as_uint(x) + 0x1000u) & 0xFFFFE000u;
	}
	/* The "lo" part when the landed float32 itself serves as "hi": kind::tf32 reads the sign, the exponent and the top 10
	 * mantissa bits of a 32-bit operand and ignores the 13 bits below, so the raw value acts as x truncated to TF32 and
	 * needs no rewriting; what the MMA then misses is x - trunc(x), exact in float32, rounded to TF32 here.  Half of the
	 * split's shared-memory writes disappear with it. */
	__device__ __forceinline__ uint4 remainder4(uint4 raw)
	{
		const uint32_t in[4] = { raw.x, raw.y, raw.z, raw.w };
		uint32_t l[4];
#pragma unroll
		for (int i = 0; i < 4; i++)
		{
			const float x = __uint_as_float(in[i]);
			l[i] = to_tf32(x - __uint_as_float(in[i] & 0xFFFFE000u));
		}
		return make_uint4(l[0], l[1], l[2], l[3]);
	}

	template<int BLOCK_N, int STAGES>
	__global__ void __launch_bounds__(kThreads, 1) kernel_gemm_nt_tf32x3(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
			const __grid_constant__ CUtensorMap mapC, int mBlocks, int nBlocks, int kBlocks, int numTiles, int N, float alpha, int *deviceStatus)
	{
		using Cfg = Config<BLOCK_N, STAGES>;
		extern __shared__ uint8_t smem_raw[];
		uint8_t *smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
		uint8_t *smem_c = smem + STAGES * Cfg::kStageBytes;

		__shared__ __align__(8) uint64_t full_bar[STAGES]; /* TMA landed */
		__shared__ __align__(8) uint64_t split_bar[STAGES]; /* hi/lo written */
		__shared__ __align__(8) uint64_t empty_bar[STAGES]; /* MMAs done with the stage */
		__shared__ __align__(8) uint64_t tmem_full_bar[2];
		__shared__ __align__(8) uint64_t tmem_empty_bar[2];
		__shared__ uint32_t tmem_base_slot;
		__shared__ int abort_flag;
		__shared__ volatile int epilogue_go;

		const int warp = threadIdx.x / 32;
		const int lane = threadIdx.x % 32;

		if (threadIdx.x == 0)
		{
			abort_flag = 0;
			for (int s = 0; s < STAGES; s++)
			{
				umma::mbar_init(&full_bar[s], 1);
				umma::mbar_init(&split_bar[s], kSplitThreads);
				umma::mbar_init(&empty_bar[s], 1);
			}
			for (int a = 0; a < 2; a++)
			{
				umma::mbar_init(&tmem_full_bar[a], 1);
				umma::mbar_init(&tmem_empty_bar[a], 128);
			}
			umma::mbar_fence_init();
			umma::prefetch_tensormap(&mapA);
			umma::prefetch_tensormap(&mapB);
			umma::prefetch_tensormap(&mapC);
		}
		if (warp == 1)
		{
			umma::tmem_alloc(&tmem_base_slot, Cfg::kTmemColumns);
			umma::tmem_relinquish();
		}
		umma::tcgen05_fence_before();
		__syncthreads();
		umma::tcgen05_fence_after();
		const uint32_t tmem_base = tmem_base_slot;
		volatile int *abort_ptr = &abort_flag;

		if (warp == 0)
		{
			if (lane == 0)
			{
				int stage = 0;
				uint32_t phase = 0;
				bool ok = true;
				/* (plane, row block, column block) of the tile advance by a fixed step: decomposed once, then carried, so that
				 * this thread executes no division per tile */
				int nb = static_cast<int>(blockIdx.x) % nBlocks, mb = (static_cast<int>(blockIdx.x) / nBlocks) % mBlocks,
						p = static_cast<int>(blockIdx.x) / (nBlocks * mBlocks);
				const int step_nb = static_cast<int>(gridDim.x) % nBlocks, step_mb = (static_cast<int>(gridDim.x) / nBlocks) % mBlocks,
						step_p = static_cast<int>(gridDim.x) / (nBlocks * mBlocks);
				for (int tile = blockIdx.x; tile < numTiles and ok; tile += gridDim.x)
				{
					for (int kb = 0; kb < kBlocks; kb++)
					{
						if (not umma::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_ptr))
						{
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorStageWait);
							ok = false;
							break;
						}
						uint8_t *base = smem + stage * Cfg::kStageBytes;
						umma::mbar_arrive_expect_tx(&full_bar[stage], Cfg::kLoadBytes);
						umma::tma_load_3d(base, &mapA, &full_bar[stage], kb * kBlockK, mb * kBlockM, p);
						umma::tma_load_3d(base + 2 * Cfg::kATile, &mapB, &full_bar[stage], kb * kBlockK, nb * BLOCK_N, p);
						if (++stage == STAGES)
						{
							stage = 0;
							phase ^= 1u;
						}
					}
					nb += step_nb;
					mb += step_mb;
					p += step_p;
					if (nb >= nBlocks)
					{
						nb -= nBlocks;
						mb++;
					}
					if (mb >= mBlocks)
					{
						mb -= mBlocks;
						p++;
					}
				}
			}
		}
		else if (warp == 1)
		{
			if (lane == 0)
			{
				constexpr uint32_t idesc = umma::make_instr_desc(umma::kAccumF32, umma::kFormatTF32, umma::kFormatTF32, false, false, kBlockM, BLOCK_N);
				constexpr uint32_t idesc_wide = umma::make_instr_desc(umma::kAccumF32, umma::kFormatTF32, umma::kFormatTF32, false, false, kBlockM, 2 * BLOCK_N);
				int stage = 0;
				uint32_t phase = 0;
				int it = 0;
				bool ok = true;
				for (int tile = blockIdx.x; tile < numTiles and ok; tile += gridDim.x, it++)
				{
					const int acc = it & 1;
					const uint32_t acc_phase = static_cast<uint32_t>(it >> 1) & 1u;
					if (not umma::mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, abort_ptr))
					{
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorMmaWait);
						break;
					}
					umma::tcgen05_fence_after();
					/* 2 * BLOCK_N columns per accumulator: [0, BLOCK_N) collects hi*hi + lo*hi, [BLOCK_N, 2*BLOCK_N) hi*lo */
					const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * 2 * BLOCK_N);
					for (int kb = 0; kb < kBlocks; kb++)
					{
						if (not umma::mbar_wait(&split_bar[stage], phase, abort_ptr))
						{
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
							ok = false;
							break;
						}
						umma::tcgen05_fence_after();
						const uint32_t base = umma::smem_u32(smem + stage * Cfg::kStageBytes);
						const uint64_t a_hi = umma::make_smem_desc(base, 16, 1024, umma::kSwizzle128B);
						const uint64_t a_lo = umma::make_smem_desc(base + Cfg::kATile, 16, 1024, umma::kSwizzle128B);
						/* B_hi and B_lo lie one after the other, so one descriptor with N = 2 * BLOCK_N reads both */
						const uint64_t b_hi = umma::make_smem_desc(base + 2 * Cfg::kATile, 16, 1024, umma::kSwizzle128B);
#pragma unroll
						for (int k = 0; k < kBlockK / 8; k++)
						{
							/* one MMA consumes 8 float32 = 32 bytes of every row: +2 in descriptor units.
							 * A_hi x [B_hi; B_lo] fills both halves of the accumulator with ONE read of A_hi (an MMA of twice the
							 * width costs the pipe no more at these widths), A_lo x B_hi adds to the first half: two MMAs and
							 * 14 KB of operand reads per slice where three separate products need 18 KB.  Shared-memory
							 * bandwidth, not the tensor pipe, is what this kernel runs out of. */
							const uint64_t step = static_cast<uint64_t>(2 * k);
							umma::mma_tf32(tmem_d, a_hi + step, b_hi + step, idesc_wide, (kb | k) != 0);
							umma::mma_tf32(tmem_d, a_lo + step, b_hi + step, idesc, true);
						}
						umma::mma_commit(&empty_bar[stage]);
						if (++stage == STAGES)
						{
							stage = 0;
							phase ^= 1u;
						}
					}
					if (ok)
						umma::mma_commit(&tmem_full_bar[acc]);
				}
			}
		}
		else if (warp < 2 + kSplitWarps)
		{
			/* splitters: each thread owns every kSplitThreads-th 16-byte chunk of the stage's A and B tiles */
			const int split_thread = threadIdx.x - 64;
			int stage = 0;
			uint32_t phase = 0;
			bool ok = true;
			for (int tile = blockIdx.x; tile < numTiles and ok; tile += gridDim.x)
			{
				for (int kb = 0; kb < kBlocks; kb++)
				{
					/* every warp waits by itself (its first lane polls, the outcome is broadcast): the four warps own fixed
					 * quarters of the stage, so nothing else has to be agreed between them */
					int ready = 0;
					if (lane == 0)
					{
						ready = umma::mbar_wait(&full_bar[stage], phase, abort_ptr) ? 1 : 0;
						if (ready == 0)
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
					}
					ready = __shfl_sync(0xFFFFFFFFu, ready, 0);
					if (ready == 0)
					{
						ok = false;
						break;
					}
					umma::mbar_try_wait(&full_bar[stage], phase); /* completed phase: orders this thread after the copy */
					uint4 *a_hi = reinterpret_cast<uint4*>(smem + stage * Cfg::kStageBytes);
					uint4 *a_lo = a_hi + Cfg::kATile / 16;
					uint4 *b_hi = a_hi + 2 * Cfg::kATile / 16;
					uint4 *b_lo = b_hi + Cfg::kBTile / 16;
#pragma unroll 4
					for (int i = split_thread; i < Cfg::kATile / 16; i += kSplitThreads)
						a_lo[i] = remainder4(a_hi[i]);
#pragma unroll 4
					for (int i = split_thread; i < Cfg::kBTile / 16; i += kSplitThreads)
						b_lo[i] = remainder4(b_hi[i]);
					umma::fence_proxy_async_smem();
					umma::mbar_arrive(&split_bar[stage]);
					if (++stage == STAGES)
					{
						stage = 0;
						phase ^= 1u;
					}
				}
			}
		}
		else
		{
			const int quarter = warp % 4;
			const int row = quarter * 32 + lane;
			const int epi_thread = threadIdx.x - (64 + kSplitThreads);
			int it = 0;
			for (int tile = blockIdx.x; tile < numTiles; tile += gridDim.x, it++)
			{
				const int nb = tile % nBlocks;
				const int mb = (tile / nBlocks) % mBlocks;
				const int p = tile / (nBlocks * mBlocks);
				const int acc = it & 1;
				const uint32_t acc_phase = static_cast<uint32_t>(it >> 1) & 1u;
				if (epi_thread == 0)
				{
					const bool ready = umma::mbar_wait(&tmem_full_bar[acc], acc_phase, abort_ptr);
					if (not ready)
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorEpilogueWait);
					else
						umma::tma_store_wait_read<0>(); /* the single staging buffer is free again */
					epilogue_go = ready ? 1 : 0;
				}
				umma::named_barrier_sync(1, 128);
				if (epilogue_go == 0)
					break;
				umma::tcgen05_fence_after();
				const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * 2 * BLOCK_N);
#pragma unroll
				for (int chunk = 0; chunk < BLOCK_N / 32; chunk++)
				{
					/* (hi*hi + lo*hi) + hi*lo; the second half is taken 16 columns at a time to keep the live registers down */
					uint32_t r[32], r_second[16];
					umma::tmem_load_32x32(t_addr + static_cast<uint32_t>(chunk * 32), r);
					umma::tmem_load_32x16(t_addr + static_cast<uint32_t>(BLOCK_N + chunk * 32), r_second);
					umma::tmem_load_wait();
#pragma unroll
					for (int q = 0; q < 16; q++)
						r[q] = __float_as_uint(__uint_as_float(r[q]) + __uint_as_float(r_second[q]));
					umma::tmem_load_32x16(t_addr + static_cast<uint32_t>(BLOCK_N + chunk * 32 + 16), r_second);
					umma::tmem_load_wait();
#pragma unroll
					for (int q = 0; q < 16; q++)
						r[16 + q] = __float_as_uint(__uint_as_float(r[16 + q]) + __uint_as_float(r_second[q]));
					uint8_t *row_ptr = smem_c + chunk * (kBlockM * 128) + row * 128;
#pragma unroll
					for (int j = 0; j < 8; j++)
					{
						uint4 out;
						out.x = __float_as_uint(alpha * __uint_as_float(r[4 * j + 0]));
						out.y = __float_as_uint(alpha * __uint_as_float(r[4 * j + 1]));
						out.z = __float_as_uint(alpha * __uint_as_float(r[4 * j + 2]));
						out.w = __float_as_uint(alpha * __uint_as_float(r[4 * j + 3]));
						*reinterpret_cast<uint4*>(row_ptr + ((j ^ (row & 7)) << 4)) = out;
					}
				}
				umma::tcgen05_fence_before();
				umma::mbar_arrive(&tmem_empty_bar[acc]);
				umma::fence_proxy_async_smem();
				umma::named_barrier_sync(1, 128);
				if (epi_thread == 0)
				{
#pragma unroll
					for (int sub = 0; sub < Cfg::kSubTiles; sub++)
						if (nb * BLOCK_N + sub * 32 < N)
							umma::tma_store_3d(&mapC, smem_c + sub * (kBlockM * 128), nb * BLOCK_N + sub * 32, mb * kBlockM, p);
					umma::tma_store_commit();
				}
			}
			if (epi_thread == 0)
				umma::tma_store_wait_all<0>();
		}

		__syncthreads();
		if (abort_flag != 0)
			umma::drain_after_abort();
		if (warp == 1)
		{
			umma::tcgen05_fence_after();
			umma::tmem_dealloc(tmem_base, Cfg::kTmemColumns);
		}
	}

	/* out[b][c][r] = in[b][r][c] for a small row-major tensor (the transformed filters) */
	__global__ void kernel_transpose_batched(float *__restrict__ out, const float *__restrict__ in, int rows, int cols)
	{
		__shared__ float tile[32][33];
		const int b = blockIdx.z;
		const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
		const float *src = in + static_cast<size_t>(b) * rows * cols;
		float *dst = out + static_cast<size_t>(b) * rows * cols;
		for (int i = threadIdx.y; i < 32; i += blockDim.y)
			if (r0 + i < rows and c0 + static_cast<int>(threadIdx.x) < cols)
				tile[i][threadIdx.x] = src[static_cast<size_t>(r0 + i) * cols + c0 + threadIdx.x];
		__syncthreads();
		for (int i = threadIdx.y; i < 32; i += blockDim.y)
			if (c0 + i < cols and r0 + static_cast<int>(threadIdx.x) < rows)
				dst[static_cast<size_t>(c0 + i) * rows + r0 + threadIdx.x] = tile[threadIdx.x][i];
	}


	/* ---------------------------------------------------------------------------------------------------------
	 * C[i] = alpha * A[i]^T * B[i] + beta * C[i]  with A stored [Kc, M] and B stored [Kc, N]: the weight-gradient
	 * contraction of the Winograd backward pass (A = transformed dy, B = transformed x, Kc = tiles, M = K, N = C).
	 * Both operands are contiguous along their OUTPUT index, i.e. "MN-major" for the tensor core: a TMA box of
	 * 32 float32 (128 bytes) by 32 rows, written with the 128-byte swizzle whose atom is 32 bytes (the only layout the
	 * tensor core accepts for MN-major 32-bit operands), is exactly one column block of the canonical MN-major layout
	 * (4-row groups 512 bytes apart, column blocks 4096 bytes apart), so no transposition happens anywhere.
	 * The contraction is long (thousands of tiles) and the output tiny, so it is split over the grid: CTA (s, tile)
	 * accumulates rows [s*chunk, (s+1)*chunk) into a 128 x 64 TMEM accumulator and writes a partial tile to scratch;
	 * kernel_splitk_reduce sums the partials in a fixed order (deterministic) and applies alpha / beta.
	 * Output rows beyond M inside a 128-row tile come from column blocks that are never loaded and are zeroed once.
	 * --------------------------------------------------------------------------------------------------------- */
	constexpr int kTnBlockN = 64;
	constexpr int kTnBlockBytes = 32 * 128; /* one column block: 32 contraction rows x 32 float32 */
	constexpr int kTnABlocks = kBlockM / 32;
	/* per stage: A hi (4 blocks), A lo, B hi (2 or 4 blocks), B lo: see TnLayout */

	/* Two batch entries per MMA.  When the result has at most 64 rows and 64 columns (the dW product of a 64-channel
	 * layer), half of the 128 accumulator rows of the form above would be padding, and an MMA with N = 64 occupies the
	 * tensor pipe as long as one with N = 128.  The paired form stacks entries 2q and 2q+1: rows 0..63 / 64..127 of A and
	 * columns 0..63 / 64..127 of B come from the two entries, so the two diagonal 64 x 64 blocks of the 128 x 128
	 * accumulator are the two results (the off-diagonal blocks are products of unrelated operands and are dropped).
	 * Every byte of a stage is then real data: twice the bytes in flight and half the MMAs per byte. */
	template<bool PAIR>
	struct TnLayout
	{
			static constexpr int kABlocks = 4;
			static constexpr int kBBlocks = PAIR ? 4 : 2;
			static constexpr int kBlockN = PAIR ? 128 : 64;
			static constexpr int kStages = PAIR ? 3 : 4;
			static constexpr int kALo = kABlocks * kTnBlockBytes;
			static constexpr int kBHi = 2 * kABlocks * kTnBlockBytes;
			static constexpr int kBLo = kBHi + kBBlocks * kTnBlockBytes;
			static constexpr int kStageBytes = 2 * (kABlocks + kBBlocks) * kTnBlockBytes;
			static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
	};

	template<bool PAIR>
	__global__ void __launch_bounds__(kThreads, 1) kernel_gemm_tn_tf32x3(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
			float *__restrict__ partial, int M, int N, int mBlocks, int nBlocks, int kBlocksTotal, int kBlocksPerSplit, int *deviceStatus)
	{
		using L = TnLayout<PAIR>;
		constexpr int kTnStages = L::kStages;
		constexpr int kTnStageBytes = L::kStageBytes;
		constexpr int kTnBlockN = L::kBlockN; /* accumulator columns of this form (the file-scope constant is the 64 of a stored tile) */
		extern __shared__ uint8_t smem_raw[];
		uint8_t *smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
		__shared__ __align__(8) uint64_t full_bar[kTnStages];
		__shared__ __align__(8) uint64_t split_bar[kTnStages];
		__shared__ __align__(8) uint64_t empty_bar[kTnStages];
		__shared__ __align__(8) uint64_t tmem_full_bar;
		__shared__ uint32_t tmem_base_slot;
		__shared__ int abort_flag;

		const int warp = threadIdx.x / 32;
		const int lane = threadIdx.x % 32;
		const int split = blockIdx.x;
		const int tile = blockIdx.y;
		/* unpaired: tile = (batch entry, row block, column block); paired: tile = pair of batch entries, one block each */
		const int nb = PAIR ? 0 : tile % nBlocks;
		const int mb = PAIR ? 0 : (tile / nBlocks) % mBlocks;
		const int p = PAIR ? 2 * tile : tile / (nBlocks * mBlocks);
		const int kb_begin = split * kBlocksPerSplit;
		const int kb_end = min(kBlocksTotal, kb_begin + kBlocksPerSplit);
		const int m0 = mb * kBlockM, n0 = nb * 64;
		/* column blocks (of 32) that hold real data, per batch entry */
		const int a_blocks = min(PAIR ? 2 : kTnABlocks, (M - m0 + 31) / 32);
		const int b_blocks = min(2, (N - n0 + 31) / 32);

		/* column blocks that are never loaded must read as zero, in the hi and the lo copy */
		for (int i = threadIdx.x; i < kTnStages * kTnStageBytes / 16; i += kThreads)
			reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
		if (threadIdx.x == 0)
		{
			abort_flag = 0;
			for (int s = 0; s < kTnStages; s++)
			{
				umma::mbar_init(&full_bar[s], 1);
				umma::mbar_init(&split_bar[s], kSplitThreads);
				umma::mbar_init(&empty_bar[s], 1);
			}
			umma::mbar_init(&tmem_full_bar, 1);
			umma::mbar_fence_init();
			umma::prefetch_tensormap(&mapA);
			umma::prefetch_tensormap(&mapB);
		}
		if (warp == 1)
		{
			umma::tmem_alloc(&tmem_base_slot, 2 * kTnBlockN); /* [0, N) hi*hi + lo*hi, [N, 2N) hi*lo */
			umma::tmem_relinquish();
		}
		umma::fence_proxy_async_smem();
		umma::tcgen05_fence_before();
		__syncthreads();
		umma::tcgen05_fence_after();
		const uint32_t tmem_base = tmem_base_slot;
		volatile int *abort_ptr = &abort_flag;
		constexpr int a_lo_offset = L::kALo;
		constexpr int b_hi_offset = L::kBHi;
		constexpr int b_lo_offset = L::kBLo;

		if (warp == 0)
		{
			if (lane == 0)
			{
				int stage = 0;
				uint32_t phase = 0;
				for (int kb = kb_begin; kb < kb_end; kb++)
				{
					if (not umma::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_ptr))
					{
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorStageWait);
						break;
					}
					uint8_t *base = smem + stage * kTnStageBytes;
					umma::mbar_arrive_expect_tx(&full_bar[stage], static_cast<uint32_t>((PAIR ? 2 : 1) * (a_blocks + b_blocks) * kTnBlockBytes));
					for (int b = 0; b < a_blocks; b++)
						umma::tma_load_3d(base + b * kTnBlockBytes, &mapA, &full_bar[stage], m0 + 32 * b, kb * kBlockK, p);
					for (int b = 0; b < b_blocks; b++)
						umma::tma_load_3d(base + b_hi_offset + b * kTnBlockBytes, &mapB, &full_bar[stage], n0 + 32 * b, kb * kBlockK, p);
					if (PAIR)
					{
						/* the second entry of the pair fills the upper half of the rows of A and of the columns of B */
						for (int b = 0; b < a_blocks; b++)
							umma::tma_load_3d(base + (2 + b) * kTnBlockBytes, &mapA, &full_bar[stage], 32 * b, kb * kBlockK, p + 1);
						for (int b = 0; b < b_blocks; b++)
							umma::tma_load_3d(base + b_hi_offset + (2 + b) * kTnBlockBytes, &mapB, &full_bar[stage], 32 * b, kb * kBlockK, p + 1);
					}
					if (++stage == kTnStages)
					{
						stage = 0;
						phase ^= 1u;
					}
				}
			}
		}
		else if (warp == 1)
		{
			if (lane == 0)
			{
				constexpr uint32_t idesc = umma::make_instr_desc(umma::kAccumF32, umma::kFormatTF32, umma::kFormatTF32, true, true, kBlockM, kTnBlockN);
				constexpr uint32_t idesc_wide = umma::make_instr_desc(umma::kAccumF32, umma::kFormatTF32, umma::kFormatTF32, true, true, kBlockM, 2 * kTnBlockN);
				int stage = 0;
				uint32_t phase = 0;
				bool ok = true;
				for (int kb = kb_begin; kb < kb_end; kb++)
				{
					if (not umma::mbar_wait(&split_bar[stage], phase, abort_ptr))
					{
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
						ok = false;
						break;
					}
					umma::tcgen05_fence_after();
					const uint32_t base = umma::smem_u32(smem + stage * kTnStageBytes);
#pragma unroll
					for (int k = 0; k < kBlockK / 8; k++)
					{
						/* 8 contraction rows = two 512-byte groups of every column block */
						const uint32_t step = static_cast<uint32_t>(k * 1024);
						const uint64_t a_hi = umma::make_smem_desc(base + step, kTnBlockBytes, 512, umma::kSwizzle128BBase32B);
						const uint64_t a_lo = umma::make_smem_desc(base + a_lo_offset + step, kTnBlockBytes, 512, umma::kSwizzle128BBase32B);
						/* the column blocks of B_lo follow those of B_hi at the same 4096-byte pitch: one descriptor with twice the
						 * width reads both (see the (N,T) kernel: two MMAs and fewer operand reads per slice instead of three) */
						const uint64_t b_hi = umma::make_smem_desc(base + b_hi_offset + step, kTnBlockBytes, 512, umma::kSwizzle128BBase32B);
						static_assert(b_lo_offset == b_hi_offset + (kTnBlockN / 32) * kTnBlockBytes, "B_lo must follow B_hi");
						umma::mma_tf32(tmem_base, a_hi, b_hi, idesc_wide, (kb != kb_begin) or (k != 0));
						umma::mma_tf32(tmem_base, a_lo, b_hi, idesc, true);
					}
					umma::mma_commit(&empty_bar[stage]);
					if (++stage == kTnStages)
					{
						stage = 0;
						phase ^= 1u;
					}
				}
				if (ok)
					umma::mma_commit(&tmem_full_bar);
			}
		}
		else if (warp < 2 + kSplitWarps)
		{
			const int split_thread = threadIdx.x - 64;
			int stage = 0;
			uint32_t phase = 0;
			/* paired: the second entry's blocks start at block 2, so the split covers blocks 0 .. 2 + count - 1 (a block in
			 * between that was never loaded holds zeros and splits into zeros) */
			const int a_chunks = (PAIR ? 2 + a_blocks : a_blocks) * kTnBlockBytes / 16;
			const int b_chunks = (PAIR ? 2 + b_blocks : b_blocks) * kTnBlockBytes / 16;
			for (int kb = kb_begin; kb < kb_end; kb++)
			{
				int ready = 0;
				if (lane == 0)
				{
					ready = umma::mbar_wait(&full_bar[stage], phase, abort_ptr) ? 1 : 0;
					if (ready == 0)
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
				}
				ready = __shfl_sync(0xFFFFFFFFu, ready, 0);
				if (ready == 0)
					break;
				umma::mbar_try_wait(&full_bar[stage], phase);
				uint4 *a_hi = reinterpret_cast<uint4*>(smem + stage * kTnStageBytes);
				uint4 *a_lo = a_hi + a_lo_offset / 16;
				uint4 *b_hi = a_hi + b_hi_offset / 16;
				uint4 *b_lo = a_hi + b_lo_offset / 16;
				for (int i = split_thread; i < a_chunks; i += kSplitThreads)
					a_lo[i] = remainder4(a_hi[i]);
				for (int i = split_thread; i < b_chunks; i += kSplitThreads)
					b_lo[i] = remainder4(b_hi[i]);
				umma::fence_proxy_async_smem();
				umma::mbar_arrive(&split_bar[stage]);
				if (++stage == kTnStages)
				{
					stage = 0;
					phase ^= 1u;
				}
			}
		}
		else
		{
			const int quarter = warp % 4;
			const int row = quarter * 32 + lane;
			const bool has_work = kb_end > kb_begin;
			bool ready = has_work;
			if (has_work)
				ready = umma::mbar_wait(&tmem_full_bar, 0, abort_ptr);
			/* a wait that ran out is reported; the (then meaningless) accumulator is still drained so that every warp
			 * takes the same path to the final barrier */
			if (has_work and not ready and lane == 0)
				umma::raise_error(abort_ptr, deviceStatus, umma::kErrorEpilogueWait);
			umma::tcgen05_fence_after();
			/* partial tiles are stored per batch entry as 128 rows x 64 columns whatever the form; in the paired form rows
			 * 0..63 hold entry 2q (accumulator columns 0..63) and rows 64..127 entry 2q+1 (columns 64..127), each written
			 * to rows 0..63 of its own entry's tile */
			const int entry_tile = PAIR ? 2 * tile + (row >= 64 ? 1 : 0) : tile;
			const int entry_tiles = PAIR ? 2 * static_cast<int>(gridDim.y) : static_cast<int>(gridDim.y);
			const int entry_row = PAIR ? (row & 63) : row;
			const int first_column = (PAIR and row >= 64) ? 64 : 0;
			float *dst = partial + ((static_cast<size_t>(split) * entry_tiles + entry_tile) * kBlockM + entry_row) * 64;
#pragma unroll
			for (int chunk = 0; chunk < 2; chunk++)
			{
				uint32_t r[32], r_second[32];
				umma::tmem_load_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(first_column + chunk * 32), r);
				umma::tmem_load_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(kTnBlockN + first_column + chunk * 32), r_second);
				umma::tmem_load_wait();
#pragma unroll
				for (int q = 0; q < 32; q++)
					r[q] = __float_as_uint(__uint_as_float(r[q]) + __uint_as_float(r_second[q])); /* (hi*hi + lo*hi) + hi*lo */
#pragma unroll
				for (int j = 0; j < 8; j++)
				{
					uint4 out = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
					if (not (has_work and ready))
						out = make_uint4(0, 0, 0, 0);
					*reinterpret_cast<uint4*>(dst + chunk * 32 + 4 * j) = out;
				}
			}
		}

		umma::tcgen05_fence_before();
		__syncthreads();
		if (abort_flag != 0)
			umma::drain_after_abort();
		if (warp == 1)
		{
			umma::tcgen05_fence_after();
			umma::tmem_dealloc(tmem_base, 2 * kTnBlockN);
		}
	}

	/* C = alpha * sum over splits of the partial tiles (fixed order) + beta * C */
	__global__ void kernel_splitk_reduce(float *C, const float *__restrict__ partial, int splits, int tiles, int M, int N, int mBlocks, int nBlocks, int ldc,
			long long strideC, float alpha, float beta)
	{
		const long long total = static_cast<long long>(tiles) * kBlockM * kTnBlockN;
		for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			const int col = static_cast<int>(i % kTnBlockN);
			const int row = static_cast<int>((i / kTnBlockN) % kBlockM);
			const int tile = static_cast<int>(i / (kBlockM * kTnBlockN));
			const int nb = tile % nBlocks;
			const int mb = (tile / nBlocks) % mBlocks;
			const int p = tile / (nBlocks * mBlocks);
			const int m = mb * kBlockM + row, n = nb * kTnBlockN + col;
			if (m >= M or n >= N)
				continue;
			float sum = 0.0f;
			for (int s = 0; s < splits; s++)
				sum += partial[(static_cast<size_t>(s) * tiles + tile) * kBlockM * kTnBlockN + row * kTnBlockN + col];
			float *dst = C + p * strideC + static_cast<size_t>(m) * ldc + n;
			float value = alpha * sum;
			if (beta != 0.0f)
				value += beta * *dst;
			*dst = value;
		}
	}

	avStatus_t launch_tn(ContextObject &ctx, const GemmShape &s, const void *A, const void *B, void *C, float alpha, float beta)
	{
		const CUtensorMapDataType type = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
		CUtensorMap mapA, mapB;
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(s.M), static_cast<uint64_t>(s.Kc), static_cast<uint64_t>(s.batch) };
			const uint64_t strides[2] = { static_cast<uint64_t>(s.lda) * 4, static_cast<uint64_t>(s.strideA) * 4 };
			const uint32_t box[3] = { 32, kBlockK, 1 };
			if (not umma::make_tensor_map(&mapA, type, 3, const_cast<void*>(A), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(s.N), static_cast<uint64_t>(s.Kc), static_cast<uint64_t>(s.batch) };
			const uint64_t strides[2] = { static_cast<uint64_t>(s.ldb) * 4, static_cast<uint64_t>(s.strideB) * 4 };
			const uint32_t box[3] = { 32, kBlockK, 1 };
			if (not umma::make_tensor_map(&mapB, type, 3, const_cast<void*>(B), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		const int mBlocks = (s.M + kBlockM - 1) / kBlockM;
		const int nBlocks = (s.N + kTnBlockN - 1) / kTnBlockN;
		const long long tiles = static_cast<long long>(s.batch) * mBlocks * nBlocks;
		if (tiles > 65535)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const int kBlocks = (s.Kc + kBlockK - 1) / kBlockK;
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		/* results of at most 64 x 64 are computed two batch entries at a time */
		const bool paired = s.M <= 64 and s.N <= 64 and s.batch >= 2 and s.batch % 2 == 0;
		const long long grid_tiles = paired ? tiles / 2 : tiles;
		/* as many splits as fit two CTAs' worth of work per SM, but at least 8 contraction blocks per split */
		int splits = static_cast<int>(std::max<long long>(1, std::min<long long>((2 * sms) / grid_tiles, (kBlocks + 7) / 8)));
		const int kBlocksPerSplit = (kBlocks + splits - 1) / splits;
		splits = (kBlocks + kBlocksPerSplit - 1) / kBlocksPerSplit;
		const size_t partial_bytes = static_cast<size_t>(splits) * tiles * kBlockM * kTnBlockN * sizeof(float);
		float *partial = reinterpret_cast<float*>(ctx.getWorkspace(partial_bytes));

		static PerDeviceOnce configured;
		if (configured.run(ctx.device, [&]() -> cudaError_t { { const cudaError_t e = cudaFuncSetAttribute(kernel_gemm_tn_tf32x3<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TnLayout<false>::kSmemBytes); if (e != cudaSuccess) return e; } return cudaFuncSetAttribute(kernel_gemm_tn_tf32x3<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TnLayout<true>::kSmemBytes); }) != cudaSuccess)
		{
			cudaGetLastError();
			return AVOCADO_STATUS_EXECUTION_FAILED;
		}
		const dim3 grid(splits, static_cast<unsigned int>(grid_tiles));
		if (paired)
			kernel_gemm_tn_tf32x3<true> <<<grid, kThreads, TnLayout<true>::kSmemBytes, ctx.getStream()>>>(mapA, mapB, partial, s.M, s.N, mBlocks, nBlocks, kBlocks,
					kBlocksPerSplit, ctx.getDeviceStatus());
		else
			kernel_gemm_tn_tf32x3<false> <<<grid, kThreads, TnLayout<false>::kSmemBytes, ctx.getStream()>>>(mapA, mapB, partial, s.M, s.N, mBlocks, nBlocks, kBlocks,
					kBlocksPerSplit, ctx.getDeviceStatus());
		avStatus_t status = checkForErrors();
		if (status != AVOCADO_STATUS_SUCCESS)
			return status;
		const long long total = tiles * kBlockM * kTnBlockN;
		const int reduce_grid = static_cast<int>(std::min<long long>((total + 255) / 256, 4 * sms));
		kernel_splitk_reduce<<<reduce_grid, 256, 0, ctx.getStream()>>>(reinterpret_cast<float*>(C), partial, splits, static_cast<int>(tiles), s.M, s.N, mBlocks,
				nBlocks, s.ldc, s.strideC, alpha, beta);
		return checkForErrors();
	}

	template<int BLOCK_N, int STAGES>
	avStatus_t launch_config(ContextObject &ctx, const GemmShape &s, const CUtensorMap &mapA, const CUtensorMap &mapB, const CUtensorMap &mapC,
			float alpha)
	{
		using Cfg = Config<BLOCK_N, STAGES>;
		auto kernel = kernel_gemm_nt_tf32x3<BLOCK_N, STAGES>;
		static PerDeviceOnce configured;
		if (configured.run(ctx.device, [&]() -> cudaError_t { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes); }) != cudaSuccess)
		{
			cudaGetLastError();
			return AVOCADO_STATUS_EXECUTION_FAILED;
		}
		const int mBlocks = (s.M + kBlockM - 1) / kBlockM;
		const int nBlocks = (s.N + BLOCK_N - 1) / BLOCK_N;
		const int kBlocks = (s.Kc + kBlockK - 1) / kBlockK;
		const long long tiles = static_cast<long long>(s.batch) * mBlocks * nBlocks;
		if (tiles > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		const int grid = static_cast<int>(std::min<long long>(tiles, sms));
		kernel<<<grid, kThreads, Cfg::kSmemBytes, ctx.getStream()>>>(mapA, mapB, mapC, mBlocks, nBlocks, kBlocks, static_cast<int>(tiles), s.N, alpha,
				ctx.getDeviceStatus());
		return checkForErrors();
	}

	avStatus_t launch_nt(ContextObject &ctx, const GemmShape &s, const void *A, const void *B, void *C, float alpha)
	{
		const CUtensorMapDataType type = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
		const int blockN = (s.N <= 64) ? 64 : 128;
		CUtensorMap mapA, mapB, mapC;
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(s.Kc), static_cast<uint64_t>(s.M), static_cast<uint64_t>(s.batch) };
			const uint64_t strides[2] = { static_cast<uint64_t>(s.lda) * 4, static_cast<uint64_t>(s.strideA) * 4 };
			const uint32_t box[3] = { kBlockK, kBlockM, 1 };
			if (not umma::make_tensor_map(&mapA, type, 3, const_cast<void*>(A), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(s.Kc), static_cast<uint64_t>(s.N), static_cast<uint64_t>(s.batch) };
			const uint64_t strides[2] = { static_cast<uint64_t>(s.ldb) * 4, static_cast<uint64_t>(s.strideB) * 4 };
			const uint32_t box[3] = { kBlockK, static_cast<uint32_t>(blockN), 1 };
			if (not umma::make_tensor_map(&mapB, type, 3, const_cast<void*>(B), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(s.N), static_cast<uint64_t>(s.M), static_cast<uint64_t>(s.batch) };
			const uint64_t strides[2] = { static_cast<uint64_t>(s.ldc) * 4, static_cast<uint64_t>(s.strideC) * 4 };
			const uint32_t box[3] = { 32, kBlockM, 1 };
			if (not umma::make_tensor_map(&mapC, type, 3, C, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		if (blockN == 64)
			return launch_config<64, 4>(ctx, s, mapA, mapB, mapC, alpha);
		return launch_config<128, 2>(ctx, s, mapA, mapB, mapC, alpha);
	}
}

namespace bk
{
	avStatus_t launch_gemm_tf32(ContextObject &ctx, const GemmShape &s, const void *A, const void *B, void *C, float alpha, float beta)
	{
		if (cuda_sm_version(ctx.device) != 100)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (s.transA)
		{
			/* A^T * B: both stored with the contraction index outermost */
			if (s.transB or s.batch < 1 or s.M < 4 or s.N < 4 or s.Kc < 1 or s.M % 4 != 0 or s.N % 4 != 0 or s.lda != s.M or s.ldb != s.N)
				return AVOCADO_STATUS_NOT_SUPPORTED;
			if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) % 16 != 0)
				return AVOCADO_STATUS_NOT_SUPPORTED;
			return launch_tn(ctx, s, A, B, C, alpha, beta);
		}
		if (beta != 0.0f)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (s.batch < 1 or s.M < 1 or s.N < 8 or s.Kc < 8 or s.Kc % 4 != 0 or s.N % 4 != 0)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 != 0)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (s.ldc != s.N)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (s.transB)
		{
			if (s.lda != s.Kc or s.ldb != s.Kc)
				return AVOCADO_STATUS_NOT_SUPPORTED;
			return launch_nt(ctx, s, A, B, C, alpha);
		}
		/* op(B) = B, stored [Kc, N]: transpose the (small) B into scratch and run the same kernel */
		const size_t b_bytes = static_cast<size_t>(s.batch) * s.Kc * s.N * sizeof(float);
		if (s.lda != s.Kc or s.ldb != s.N or b_bytes > (64u << 20))
			return AVOCADO_STATUS_NOT_SUPPORTED;
		float *transposed = reinterpret_cast<float*>(ctx.getWorkspace(b_bytes));
		const dim3 block(32, 8);
		const dim3 grid((s.N + 31) / 32, (s.Kc + 31) / 32, s.batch);
		if (s.batch > 65535)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		kernel_transpose_batched<<<grid, block, 0, ctx.getStream()>>>(transposed, reinterpret_cast<const float*>(B), s.Kc, s.N);
		GemmShape t = s;
		t.transB = true;
		t.ldb = s.Kc;
		t.strideB = static_cast<long long>(s.Kc) * s.N;
		return launch_nt(ctx, t, A, transposed, C, alpha);
	}
} /* namespace bk */
