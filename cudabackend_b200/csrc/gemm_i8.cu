/*
 * gemm_i8.cu -- C[M, N] (int32) = A[M, Kc] (int8) x B[N, Kc]^T (int8) on the tensor cores: the int8 case of cudaGemm
 * (reference src/gemm.cpp:42-57, a cublasGemmEx call with CUDA_R_8I operands and CUDA_R_32I result), which together
 * with cudaIm2Row is the explicit-lowering form of the quantised convolution (reference app/CudaBackend.cu:233-240).
 *
 * Same organisation as the 16-bit kernel of gemm.cu: persistent CTAs, one warp feeding 128-byte-swizzled stages by TMA
 * (128 rows x 128 int8 of A, BLOCK_N rows x 128 int8 of B), one thread issuing tcgen05.mma kind::i8 (K = 32, four per
 * stage) into a double-buffered int32 accumulator in TMEM, four warps draining it (tcgen05.ld) into swizzled shared
 * memory, 32 int32 = 128 bytes per row and sub-tile, and writing it with TMA stores.  Integer arithmetic: the result is
 * exact, whatever the order of accumulation.
 */
#include "gemm_internal.hpp"
#include "device_utils.cuh"
#include "umma.cuh"

#include <algorithm>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;
	using namespace bk;

	constexpr int kBlockM = 128;
	constexpr int kBlockK = 128; /* int8 elements: 128 bytes */
	constexpr int kThreads = 192;
	constexpr int kSubColumns = 32; /* int32 columns per 128-byte row of a C sub-tile */

	template<int BLOCK_N, int STAGES>
	struct Config
	{
			static constexpr int kABytes = kBlockM * 128;
			static constexpr int kBBytes = BLOCK_N * 128;
			static constexpr int kStageBytes = kABytes + kBBytes;
			static constexpr int kSubTiles = BLOCK_N / kSubColumns;
			static constexpr int kCBytes = kSubTiles * kBlockM * 128;
			static constexpr int kSmemBytes = STAGES * kStageBytes + kCBytes + 1024 /* alignment slack */;
			static constexpr int kTmemColumns = 2 * BLOCK_N;
	};

	template<int BLOCK_N, int STAGES>
	__global__ void __launch_bounds__(kThreads) kernel_gemm_nt_i8(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
			const __grid_constant__ CUtensorMap mapC, int mBlocks, int nBlocks, int kBlocks, int numTiles, int N, int *deviceStatus)
	{
		using Cfg = Config<BLOCK_N, STAGES>;
		extern __shared__ uint8_t smem_raw[];
		uint8_t *smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
		uint8_t *smem_c = smem + STAGES * Cfg::kStageBytes;

		__shared__ __align__(8) uint64_t full_bar[STAGES];
		__shared__ __align__(8) uint64_t empty_bar[STAGES];
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
		chain_wait();
		chain_release();

		if (warp == 0)
		{
			if (lane == 0)
			{
				int stage = 0;
				uint32_t phase = 0;
				bool ok = true;
				for (int tile = blockIdx.x; tile < numTiles and ok; tile += gridDim.x)
				{
					const int nb = tile % nBlocks;
					const int mb = tile / nBlocks;
					for (int kb = 0; kb < kBlocks; kb++)
					{
						if (not umma::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_ptr))
						{
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorStageWait);
							ok = false;
							break;
						}
						uint8_t *a_dst = smem + stage * Cfg::kStageBytes;
						uint8_t *b_dst = a_dst + Cfg::kABytes;
						umma::mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
						umma::tma_load_2d(a_dst, &mapA, &full_bar[stage], kb * kBlockK, mb * kBlockM);
						umma::tma_load_2d(b_dst, &mapB, &full_bar[stage], kb * kBlockK, nb * BLOCK_N);
						if (++stage == STAGES)
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
				constexpr uint32_t idesc = umma::make_instr_desc(umma::kAccumS32, umma::kFormatS8, umma::kFormatS8, false, false, kBlockM, BLOCK_N);
				const uint64_t a_desc0 = umma::make_smem_desc(umma::smem_u32(smem), 16, 1024, umma::kSwizzle128B);
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
					const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
					for (int kb = 0; kb < kBlocks; kb++)
					{
						if (not umma::mbar_wait(&full_bar[stage], phase, abort_ptr))
						{
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
							ok = false;
							break;
						}
						umma::tcgen05_fence_after();
						/* four MMAs of 32 int8 (32 bytes of the 128-byte swizzle row each) consume the stage */
						const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage * (Cfg::kStageBytes / 16));
						umma::mma_i8_k4(tmem_d, a_desc, a_desc + Cfg::kABytes / 16, idesc, kb != 0);
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
		else
		{
			const int quarter = warp % 4; /* TMEM lanes this warp may read */
			const int row = quarter * 32 + lane;
			const int epi_thread = threadIdx.x - 64;
			int it = 0;
			for (int tile = blockIdx.x; tile < numTiles; tile += gridDim.x, it++)
			{
				const int nb = tile % nBlocks;
				const int mb = tile / nBlocks;
				const int acc = it & 1;
				const uint32_t acc_phase = static_cast<uint32_t>(it >> 1) & 1u;
				/* one thread waits for the accumulator and for the staging buffer (free once the previous tile's stores
				 * have read it) and publishes the outcome, so that all four warps take the same branch */
				if (epi_thread == 0)
				{
					const bool ready = umma::mbar_wait(&tmem_full_bar[acc], acc_phase, abort_ptr);
					if (not ready)
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorEpilogueWait);
					else
						umma::tma_store_wait_read<0>();
					epilogue_go = ready ? 1 : 0;
				}
				umma::named_barrier_sync(1, 128);
				if (epilogue_go == 0)
					break;
				umma::tcgen05_fence_after();

				const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BLOCK_N);
#pragma unroll
				for (int chunk = 0; chunk < BLOCK_N / kSubColumns; chunk++)
				{
					uint32_t r[32];
					umma::tmem_load_32x32(t_addr + static_cast<uint32_t>(chunk * kSubColumns), r);
					umma::tmem_load_wait();
					uint8_t *row_ptr = smem_c + chunk * (kBlockM * 128) + row * 128;
#pragma unroll
					for (int j = 0; j < 8; j++) /* eight 16-byte pieces of the 128-byte row, in the swizzled order TMA expects */
						*reinterpret_cast<uint4*>(row_ptr + ((j ^ (row & 7)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
				}
				/* accumulator drained: hand it back to the MMA warp */
				umma::tcgen05_fence_before();
				umma::mbar_arrive(&tmem_empty_bar[acc]);

				umma::fence_proxy_async_smem();
				umma::named_barrier_sync(1, 128);
				if (epi_thread == 0)
				{
#pragma unroll
					for (int sub = 0; sub < Cfg::kSubTiles; sub++)
						if (nb * BLOCK_N + sub * kSubColumns < N)
							umma::tma_store_2d(&mapC, smem_c + sub * (kBlockM * 128), nb * BLOCK_N + sub * kSubColumns, mb * kBlockM);
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

	template<int BLOCK_N, int STAGES>
	avStatus_t launch_config(ContextObject &ctx, const GemmShape &s, const CUtensorMap &mapA, const CUtensorMap &mapB, const CUtensorMap &mapC)
	{
		using Cfg = Config<BLOCK_N, STAGES>;
		auto kernel = kernel_gemm_nt_i8<BLOCK_N, STAGES>;
		static PerDeviceOnce configured;
		if (configured.run(ctx.device, [&]() -> cudaError_t { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes); }) != cudaSuccess)
		{
			cudaGetLastError();
			return AVOCADO_STATUS_EXECUTION_FAILED;
		}
		const int mBlocks = (s.M + kBlockM - 1) / kBlockM;
		const int nBlocks = (s.N + BLOCK_N - 1) / BLOCK_N;
		const int kBlocks = (s.Kc + kBlockK - 1) / kBlockK;
		const long long tiles = static_cast<long long>(mBlocks) * nBlocks;
		if (tiles > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		const int grid = static_cast<int>(std::min<long long>(tiles, sms));
		const cudaError_t launched = launch_chained(kernel, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, ctx.getStream(), mapA, mapB, mapC, mBlocks, nBlocks,
				kBlocks, static_cast<int>(tiles), s.N, ctx.getDeviceStatus());
		if (launched != cudaSuccess)
			return convertStatus(launched);
		return checkForErrors();
	}
}

namespace bk
{
	avStatus_t launch_gemm_i8(ContextObject &ctx, const GemmShape &s, const void *A, const void *B, void *C)
	{
		if (cuda_sm_version(ctx.device) != 100)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (s.batch != 1 or s.transA or not s.transB or s.M < 1 or s.N < 16 or s.Kc < 16)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		/* TMA needs 16-byte aligned bases and row pitches: int8 rows of Kc bytes, int32 rows of 4 * N bytes */
		if (s.Kc % 16 != 0 or s.N % 4 != 0 or s.lda != s.Kc or s.ldb != s.Kc or s.ldc != s.N)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 != 0)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const int blockN = (s.N <= 64) ? 64 : 128;
		CUtensorMap mapA, mapB, mapC;
		{
			const uint64_t dims[2] = { static_cast<uint64_t>(s.Kc), static_cast<uint64_t>(s.M) };
			const uint64_t strides[1] = { static_cast<uint64_t>(s.lda) };
			const uint32_t box[2] = { kBlockK, kBlockM };
			if (not umma::make_tensor_map(&mapA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(A), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		{
			const uint64_t dims[2] = { static_cast<uint64_t>(s.Kc), static_cast<uint64_t>(s.N) };
			const uint64_t strides[1] = { static_cast<uint64_t>(s.ldb) };
			const uint32_t box[2] = { kBlockK, static_cast<uint32_t>(blockN) };
			if (not umma::make_tensor_map(&mapB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(B), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		{
			const uint64_t dims[2] = { static_cast<uint64_t>(s.N), static_cast<uint64_t>(s.M) };
			const uint64_t strides[1] = { static_cast<uint64_t>(s.ldc) * 4 };
			const uint32_t box[2] = { kSubColumns, kBlockM };
			if (not umma::make_tensor_map(&mapC, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, C, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		ctx.setDevice();
		if (blockN == 64)
			return launch_config<64, 4>(ctx, s, mapA, mapB, mapC);
		return launch_config<128, 4>(ctx, s, mapA, mapB, mapC);
	}
} /* namespace bk */
