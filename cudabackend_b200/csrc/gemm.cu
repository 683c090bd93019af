/*
 * gemm.cu -- cudaGemm and cudaGemmBatched: C[i] = alpha * op(A[i]) * op(B[i]) + beta * C[i], row-major.
 *
 * Reference counterpart: src/gemm.cpp:25-124 (cudaGemm) and :126-209 (cudaGemmBatched), which forward to
 * cuBLAS.  The batched form is the transform-domain contraction of the non-fused Winograd pipeline
 * (V[p] * U[p]^T for each of the tile*tile planes p), so it is written here as a hand-made kernel:
 *
 *   kernel_gemm_nt_tc  float16 / bfloat16, op(A) = A, op(B) = B^T (both operands contiguous along the
 *                      contraction index, which is how the pipeline stores them).  Persistent, warp-specialised:
 *                      one warp feeds shared memory by TMA through a ring of stages, one thread issues
 *                      tcgen05.mma into a double-buffered float32 accumulator in TMEM, four warps drain the
 *                      accumulator (tcgen05.ld), convert, stage the tile in 128-byte-swizzled shared memory
 *                      and write it with a TMA store.  At the Winograd sizes (C = K = 64..128) the kernel is
 *                      bound by HBM, not by the tensor pipe: 2*C*K/((C+K)*2) = 32..64 flop per byte.
 *   kernel_gemm_simt   every other case (float32 / float64 / int8, transposed A, beta != 0, extents that TMA
 *                      cannot address): a register-tiled CUDA-core kernel with float / double / int32
 *                      accumulation.
 *
 * There is no CPU path and no library call.
 */
#include <Avocado/cuda_backend.h>

#include "objects.hpp"
#include "device_utils.cuh"
#include "umma.cuh"
#include "winograd_internal.hpp"
#include "gemm_internal.hpp"

#include <Avocado/cuda_backend_ext.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;
	using namespace ::bk;

	/* ---------------------------------------------------------------------------------------------------------
	 * CUDA-core kernel: 64 x 64 tile per CTA, 16-deep slices, 4 x 4 results per thread.
	 * --------------------------------------------------------------------------------------------------------- */
	template<typename AT> __device__ __forceinline__ AT to_accum(half x)
	{
		return static_cast<AT>(__half2float(x));
	}
	template<typename AT> __device__ __forceinline__ AT to_accum(__nv_bfloat16 x)
	{
		return static_cast<AT>(__bfloat162float(x));
	}
	template<typename AT> __device__ __forceinline__ AT to_accum(float x)
	{
		return static_cast<AT>(x);
	}
	template<typename AT> __device__ __forceinline__ AT to_accum(double x)
	{
		return static_cast<AT>(x);
	}
	template<typename AT> __device__ __forceinline__ AT to_accum(int8_t x)
	{
		return static_cast<AT>(x);
	}
	template<typename AT> __device__ __forceinline__ AT to_accum(int32_t x)
	{
		return static_cast<AT>(x);
	}
	template<typename OT, typename AT> __device__ __forceinline__ OT from_accum(AT x)
	{
		return static_cast<OT>(x);
	}
	template<> __device__ __forceinline__ half from_accum<half, float>(float x)
	{
		return __float2half_rn(x);
	}
	template<> __device__ __forceinline__ __nv_bfloat16 from_accum<__nv_bfloat16, float>(float x)
	{
		return __float2bfloat16_rn(x);
	}

	constexpr int kSimtTile = 64;
	constexpr int kSimtSlice = 16;
	constexpr int kSimtPitch = kSimtTile + 4;

	template<typename T, typename AT, typename OT>
	__global__ void __launch_bounds__(256) kernel_gemm_simt(const T *__restrict__ A, const T *__restrict__ B, OT *C, int M, int N, int Kc, int lda, int ldb,
			int ldc, long long strideA, long long strideB, long long strideC, bool transA, bool transB, AT alpha, AT beta)
	{
		__shared__ AT As[kSimtSlice][kSimtPitch];
		__shared__ AT Bs[kSimtSlice][kSimtPitch];

		const int batch = blockIdx.z;
		const int m0 = blockIdx.y * kSimtTile;
		const int n0 = blockIdx.x * kSimtTile;
		const int tid = threadIdx.x;
		const int tx = tid % 16, ty = tid / 16;
		A += batch * strideA;
		B += batch * strideB;
		C += batch * strideC;

		AT acc[4][4];
#pragma unroll
		for (int i = 0; i < 4; i++)
#pragma unroll
			for (int j = 0; j < 4; j++)
				acc[i][j] = static_cast<AT>(0);

		for (int k0 = 0; k0 < Kc; k0 += kSimtSlice)
		{
#pragma unroll
			for (int e = tid; e < kSimtTile * kSimtSlice; e += 256)
			{
				/* the thread index runs along whichever index is contiguous in memory */
				const int ka = transA ? e / kSimtTile : e % kSimtSlice;
				const int ma = transA ? e % kSimtTile : e / kSimtSlice;
				AT va = static_cast<AT>(0);
				if (m0 + ma < M and k0 + ka < Kc)
					va = to_accum<AT>(transA ? A[static_cast<size_t>(k0 + ka) * lda + (m0 + ma)] : A[static_cast<size_t>(m0 + ma) * lda + (k0 + ka)]);
				As[ka][ma] = va;

				const int kb = transB ? e % kSimtSlice : e / kSimtTile;
				const int nb = transB ? e / kSimtSlice : e % kSimtTile;
				AT vb = static_cast<AT>(0);
				if (n0 + nb < N and k0 + kb < Kc)
					vb = to_accum<AT>(transB ? B[static_cast<size_t>(n0 + nb) * ldb + (k0 + kb)] : B[static_cast<size_t>(k0 + kb) * ldb + (n0 + nb)]);
				Bs[kb][nb] = vb;
			}
			__syncthreads();
#pragma unroll
			for (int k = 0; k < kSimtSlice; k++)
			{
				AT a[4], b[4];
#pragma unroll
				for (int i = 0; i < 4; i++)
					a[i] = As[k][ty * 4 + i];
#pragma unroll
				for (int j = 0; j < 4; j++)
					b[j] = Bs[k][tx * 4 + j];
#pragma unroll
				for (int i = 0; i < 4; i++)
#pragma unroll
					for (int j = 0; j < 4; j++)
						acc[i][j] += a[i] * b[j];
			}
			__syncthreads();
		}
#pragma unroll
		for (int i = 0; i < 4; i++)
		{
			const int m = m0 + ty * 4 + i;
			if (m >= M)
				continue;
#pragma unroll
			for (int j = 0; j < 4; j++)
			{
				const int n = n0 + tx * 4 + j;
				if (n >= N)
					continue;
				OT *dst = C + static_cast<size_t>(m) * ldc + n;
				AT value = alpha * acc[i][j];
				if (beta != static_cast<AT>(0))
					value += beta * to_accum<AT>(*dst);
				*dst = from_accum<OT, AT>(value);
			}
		}
	}

	template<typename T, typename AT, typename OT>
	avStatus_t launch_simt(cudaStream_t stream, const GemmShape &s, const void *A, const void *B, void *C, AT alpha, AT beta)
	{
		if (s.batch == 0 or s.M == 0 or s.N == 0)
			return AVOCADO_STATUS_SUCCESS;
		for (int b0 = 0; b0 < s.batch; b0 += 65535)
		{
			const int nb = std::min(65535, s.batch - b0);
			dim3 grid((s.N + kSimtTile - 1) / kSimtTile, (s.M + kSimtTile - 1) / kSimtTile, nb);
			kernel_gemm_simt<T, AT, OT> <<<grid, 256, 0, stream>>>(reinterpret_cast<const T*>(A) + b0 * s.strideA, reinterpret_cast<const T*>(B) + b0 * s.strideB,
					reinterpret_cast<OT*>(C) + b0 * s.strideC, s.M, s.N, s.Kc, s.lda, s.ldb, s.ldc, s.strideA, s.strideB, s.strideC, s.transA, s.transB, alpha,
					beta);
		}
		return checkForErrors();
	}

	/* ---------------------------------------------------------------------------------------------------------
	 * Tensor-core kernel, 16-bit operands, C = alpha * A * B^T.
	 *
	 * Shared memory per CTA (1024-byte aligned, 128-byte swizzle everywhere):
	 *   STAGES x { A tile 128 rows x 64 elements (16 KB), B tile BLOCK_N rows x 64 elements }
	 *   EPI_BUFS x { C tile as BLOCK_N/64 sub-tiles of 128 rows x 64 elements (16 KB each) }
	 * TMEM: 2 accumulators of BLOCK_N float32 columns x 128 lanes.
	 * Warps: 0 = TMA producer, 1 = MMA issuer and TMEM owner, 2..5 = epilogue (warp w drains lanes 32*(w%4)..).
	 * --------------------------------------------------------------------------------------------------------- */
	constexpr int kBlockM = 128;
	constexpr int kBlockK = 64; /* elements: 128 bytes of a 16-bit type */
	constexpr int kTcThreads = 192;
/* Stages and epilogue buffers of the 64-column configuration.  Two stages and one buffer (65 KB: three blocks per SM)
 * against three and two (105 KB: two blocks per SM), measured on 36 x [12544 x 64] x [64 x 64] float16: 20.9 against 21.3 us
 * alone, 48.6 against 48.9 us for the Winograd step around it; four stages (one block per SM) 23.1 / 54.6 us. */
#ifndef GEMM64_STAGES
#define GEMM64_STAGES 2
#endif
#ifndef GEMM64_EPI
#define GEMM64_EPI 1
#endif

	template<int BLOCK_N, int STAGES, int EPI_BUFS>
	struct TcConfig
	{
			static constexpr int kABytes = kBlockM * 128;
			static constexpr int kBBytes = BLOCK_N * 128;
			static constexpr int kStageBytes = kABytes + kBBytes;
			static constexpr int kSubTiles = BLOCK_N / 64;
			static constexpr int kCBytes = kSubTiles * kBlockM * 128;
			static constexpr int kSmemBytes = STAGES * kStageBytes + EPI_BUFS * kCBytes + 1024 /* alignment slack */;
			static constexpr int kTmemColumns = 2 * BLOCK_N;
	};

	template<int BLOCK_N, int STAGES, int EPI_BUFS, bool IS_BF16>
	__global__ void __launch_bounds__(kTcThreads) kernel_gemm_nt_tc(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
			const __grid_constant__ CUtensorMap mapC, int mBlocks, int nBlocks, int kBlocks, int numTiles, int N, float alpha, int *deviceStatus)
	{
		using Cfg = TcConfig<BLOCK_N, STAGES, EPI_BUFS>;
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
		/* barriers, TMEM and descriptors are ready: only now wait for the kernel that produces A (and may still read C) */
		chain_wait();
		chain_release();

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
						uint8_t *a_dst = smem + stage * Cfg::kStageBytes;
						uint8_t *b_dst = a_dst + Cfg::kABytes;
						umma::mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
						umma::tma_load_3d(a_dst, &mapA, &full_bar[stage], kb * kBlockK, mb * kBlockM, p);
						umma::tma_load_3d(b_dst, &mapB, &full_bar[stage], kb * kBlockK, nb * BLOCK_N, p);
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
				constexpr uint32_t idesc = umma::make_instr_desc(umma::kAccumF32, IS_BF16 ? umma::kFormatBF16 : umma::kFormatF16,
						IS_BF16 ? umma::kFormatBF16 : umma::kFormatF16, false, false, kBlockM, BLOCK_N);
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
						/* the descriptor's address field counts 16-byte units; four MMAs of 16 elements (32 bytes of the
						 * 128-byte swizzle row each) consume the stage */
						static_assert(kBlockK / 16 == 4, "a stage is four MMAs deep");
						const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage * (Cfg::kStageBytes / 16));
						umma::mma_f16_k4(tmem_d, a_desc, a_desc + Cfg::kABytes / 16, idesc, kb != 0);
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
				const int mb = (tile / nBlocks) % mBlocks;
				const int p = tile / (nBlocks * mBlocks);
				const int acc = it & 1;
				const uint32_t acc_phase = static_cast<uint32_t>(it >> 1) & 1u;
				uint8_t *c_buf = smem_c + (it % EPI_BUFS) * Cfg::kCBytes;

				/* One thread waits for the accumulator and for the staging buffer (free once the store issued
				 * EPI_BUFS tiles ago has read it) and publishes the outcome, so that all four warps take the same
				 * branch: a warp that left alone would strand the others at the named barrier. */
				if (epi_thread == 0)
				{
					const bool ready = umma::mbar_wait(&tmem_full_bar[acc], acc_phase, abort_ptr);
					if (not ready)
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorEpilogueWait);
					else
						umma::tma_store_wait_read<EPI_BUFS - 1>();
					epilogue_go = ready ? 1 : 0;
				}
				umma::named_barrier_sync(1, 128);
				if (epilogue_go == 0)
					break;
				umma::tcgen05_fence_after();

				const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BLOCK_N);
#pragma unroll
				for (int chunk = 0; chunk < BLOCK_N / 32; chunk++)
				{
					uint32_t r[32];
					umma::tmem_load_32x32(t_addr + static_cast<uint32_t>(chunk * 32), r);
					umma::tmem_load_wait();
					const int sub = (chunk * 32) / 64;
					uint8_t *row_ptr = c_buf + sub * (kBlockM * 128) + row * 128;
#pragma unroll
					for (int j = 0; j < 4; j++)
					{
						uint32_t packed[4];
#pragma unroll
						for (int q = 0; q < 4; q++)
						{
							const float lo = alpha * __uint_as_float(r[j * 8 + q * 2]);
							const float hi = alpha * __uint_as_float(r[j * 8 + q * 2 + 1]);
							if (IS_BF16)
							{
								__nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
								packed[q] = *reinterpret_cast<uint32_t*>(&v);
							}
							else
							{
								__half2 v = __floats2half2_rn(lo, hi);
								packed[q] = *reinterpret_cast<uint32_t*>(&v);
							}
						}
						const int chunk16 = ((chunk * 32) % 64) / 8 + j; /* 16-byte chunk inside the 128-byte row */
						*reinterpret_cast<uint4*>(row_ptr + ((chunk16 ^ (row & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
					}
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
						if (nb * BLOCK_N + sub * 64 < N)
							umma::tma_store_3d(&mapC, c_buf + sub * (kBlockM * 128), nb * BLOCK_N + sub * 64, mb * kBlockM, p);
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

	template<int BLOCK_N, int STAGES, int EPI_BUFS, bool IS_BF16>
	avStatus_t launch_tc_config(ContextObject &ctx, const GemmShape &s, const CUtensorMap &mapA, const CUtensorMap &mapB, const CUtensorMap &mapC,
			float alpha, int *deviceStatus)
	{
		using Cfg = TcConfig<BLOCK_N, STAGES, EPI_BUFS>;
		auto kernel = kernel_gemm_nt_tc<BLOCK_N, STAGES, EPI_BUFS, IS_BF16>;
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
		/* as many blocks per SM as TMEM (512 columns) and shared memory (1 KB reserved per block) allow */
		const int ctasPerSm = std::max(1, std::min(512 / Cfg::kTmemColumns, (227 * 1024) / (Cfg::kSmemBytes + 1024)));
		const int grid = static_cast<int>(std::min<long long>(tiles, static_cast<long long>(sms) * ctasPerSm));
		const cudaError_t launched = launch_chained(kernel, dim3(grid), dim3(kTcThreads), Cfg::kSmemBytes, ctx.getStream(), mapA, mapB, mapC, mBlocks,
				nBlocks, kBlocks, static_cast<int>(tiles), s.N, alpha, deviceStatus);
		if (launched != cudaSuccess)
			return convertStatus(launched);
		return checkForErrors();
	}

	/* 0 = choose automatically, 1 = CUDA-core kernel only, 2 = insist on the tensor-core kernel.  Read once from
	 * AVOCADO_B200_GEMM (values "simt", "tensor"); meant for isolating a kernel while debugging. */
	int forced_path()
	{
		static const int value = []()
		{
			const char *env = std::getenv("AVOCADO_B200_GEMM");
			if (env == nullptr)
				return 0;
			if (std::strcmp(env, "simt") == 0)
				return 1;
			if (std::strcmp(env, "tensor") == 0)
				return 2;
			return 0;
		}();
		return value;
	}

	/* out[b][c][r] = in[b][r][c] for a small row-major 16-bit tensor (the transformed filters of a dX pass) */
	__global__ void kernel_transpose_batched_16(uint16_t *__restrict__ out, const uint16_t *__restrict__ in, int rows, int cols)
	{
		__shared__ uint16_t tile[32][34];
		const int b = blockIdx.z;
		const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
		const uint16_t *src = in + static_cast<size_t>(b) * rows * cols;
		uint16_t *dst = out + static_cast<size_t>(b) * rows * cols;
		for (int i = threadIdx.y; i < 32; i += blockDim.y)
			if (r0 + i < rows and c0 + static_cast<int>(threadIdx.x) < cols)
				tile[i][threadIdx.x] = src[static_cast<size_t>(r0 + i) * cols + c0 + threadIdx.x];
		__syncthreads();
		for (int i = threadIdx.y; i < 32; i += blockDim.y)
			if (c0 + i < cols and r0 + static_cast<int>(threadIdx.x) < rows)
				dst[static_cast<size_t>(c0 + i) * rows + r0 + threadIdx.x] = tile[threadIdx.x][i];
	}

	bool tc_eligible(const ContextObject &ctx, const GemmShape &s, avDataType_t dtype, const void *A, const void *B, const void *C, float beta)
	{
		if (dtype != AVOCADO_DTYPE_FLOAT16 and dtype != AVOCADO_DTYPE_BFLOAT16)
			return false;
		if (s.transA or not s.transB or beta != 0.0f)
			return false;
		if (cuda_sm_version(ctx.device) != 100)
			return false;
		if (s.batch < 1 or s.M < 1 or s.N < 8 or s.Kc < 8)
			return false;
		/* TMA needs 16-byte aligned bases and row pitches */
		if (s.Kc % 8 != 0 or s.N % 8 != 0)
			return false;
		if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 != 0)
			return false;
		if (s.lda != s.Kc or s.ldb != s.Kc or s.ldc != s.N)
			return false;
		return true;
	}

	avStatus_t launch_tc(ContextObject &ctx, const GemmShape &s, avDataType_t dtype, const void *A, const void *B, void *C, float alpha, int *deviceStatus)
	{
		const CUtensorMapDataType type = (dtype == AVOCADO_DTYPE_BFLOAT16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
		const int blockN = (s.N <= 64) ? 64 : (s.N <= 128) ? 128 : 256;
		CUtensorMap mapA, mapB, mapC;
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(s.Kc), static_cast<uint64_t>(s.M), static_cast<uint64_t>(s.batch) };
			const uint64_t strides[2] = { static_cast<uint64_t>(s.lda) * 2, static_cast<uint64_t>(s.strideA) * 2 };
			const uint32_t box[3] = { kBlockK, kBlockM, 1 };
			if (not umma::make_tensor_map(&mapA, type, 3, const_cast<void*>(A), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_INTERNAL_ERROR;
		}
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(s.Kc), static_cast<uint64_t>(s.N), static_cast<uint64_t>(s.batch) };
			const uint64_t strides[2] = { static_cast<uint64_t>(s.ldb) * 2, static_cast<uint64_t>(s.strideB) * 2 };
			const uint32_t box[3] = { kBlockK, static_cast<uint32_t>(blockN), 1 };
			if (not umma::make_tensor_map(&mapB, type, 3, const_cast<void*>(B), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_INTERNAL_ERROR;
		}
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(s.N), static_cast<uint64_t>(s.M), static_cast<uint64_t>(s.batch) };
			const uint64_t strides[2] = { static_cast<uint64_t>(s.ldc) * 2, static_cast<uint64_t>(s.strideC) * 2 };
			const uint32_t box[3] = { 64, kBlockM, 1 };
			if (not umma::make_tensor_map(&mapC, type, 3, C, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_INTERNAL_ERROR;
		}
		const bool bf16 = (dtype == AVOCADO_DTYPE_BFLOAT16);
		switch (blockN)
		{
			case 64:
				return bf16 ? launch_tc_config<64, GEMM64_STAGES, GEMM64_EPI, true>(ctx, s, mapA, mapB, mapC, alpha, deviceStatus) : launch_tc_config<64, GEMM64_STAGES, GEMM64_EPI, false>(ctx, s, mapA, mapB, mapC, alpha, deviceStatus);
			case 128:
				return bf16 ? launch_tc_config<128, 3, 2, true>(ctx, s, mapA, mapB, mapC, alpha, deviceStatus) : launch_tc_config<128, 3, 2, false>(ctx, s, mapA, mapB, mapC, alpha, deviceStatus);
			default:
				return bf16 ? launch_tc_config<256, 2, 1, true>(ctx, s, mapA, mapB, mapC, alpha, deviceStatus) : launch_tc_config<256, 2, 1, false>(ctx, s, mapA, mapB, mapC, alpha, deviceStatus);
		}
	}

	avStatus_t gemm_dispatch(ContextObject &ctx, const GemmShape &s, avDataType_t abType, avDataType_t cType, const void *alpha, const void *beta,
			const void *A, const void *B, void *C)
	{
		if (s.batch == 0 or s.M == 0 or s.N == 0)
			return AVOCADO_STATUS_SUCCESS;
		if (A == nullptr or B == nullptr or C == nullptr)
			return AVOCADO_STATUS_BAD_PARAM;
		cudaStream_t stream = ctx.getStream();
		switch (cType)
		{
			case AVOCADO_DTYPE_INT32:
			{
				/* int8 x int8 -> int32, alpha and beta restricted to 0 or 1 as in the reference (src/gemm.cpp:42-57) */
				if (abType != AVOCADO_DTYPE_INT8)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				const int a = static_cast<int>(getAlphaValue<float>(alpha));
				const int b = static_cast<int>(getBetaValue<float>(beta));
				if ((a != 0 and a != 1) or (b != 0 and b != 1))
					return AVOCADO_STATUS_BAD_PARAM;
				if (a == 1 and b == 0 and forced_path() != 1)
				{
					const avStatus_t status = bk::launch_gemm_i8(ctx, s, A, B, C);
					if (status != AVOCADO_STATUS_NOT_SUPPORTED)
						return status;
				}
				if (forced_path() == 2)
					return AVOCADO_STATUS_NOT_SUPPORTED;
				return launch_simt<int8_t, int32_t, int32_t>(stream, s, A, B, C, a, b);
			}
			case AVOCADO_DTYPE_FLOAT16:
			case AVOCADO_DTYPE_BFLOAT16:
			{
				if (abType != cType)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				const float a = getAlphaValue<float>(alpha);
				const float b = getBetaValue<float>(beta);
				const bool eligible = tc_eligible(ctx, s, cType, A, B, C, b);
				if (eligible and forced_path() != 1)
					return launch_tc(ctx, s, cType, A, B, C, a, ctx.getDeviceStatus());
				/* op(B) = B, stored [Kc, N] (the dX contraction: tiles x filters times filters x channels): B is the small
				 * operand there, so it is transposed into scratch and the same tensor-core kernel runs on it */
				if (not s.transA and not s.transB and forced_path() != 1 and s.ldb == s.N and s.batch <= 65535 and s.N % 8 == 0)
				{
					GemmShape t = s;
					t.transB = true;
					t.ldb = s.Kc;
					t.strideB = static_cast<long long>(s.Kc) * s.N;
					const size_t b_bytes = static_cast<size_t>(s.batch) * s.Kc * s.N * 2;
					/* C stands in for the scratch pointer in the test: both are at least 16-byte aligned */
					if (b_bytes <= (64u << 20) and tc_eligible(ctx, t, cType, A, C, C, b))
					{
						uint16_t *transposed = reinterpret_cast<uint16_t*>(ctx.getWorkspace(b_bytes));
						const dim3 block(32, 8);
						const dim3 grid((s.N + 31) / 32, (s.Kc + 31) / 32, s.batch);
						kernel_transpose_batched_16<<<grid, block, 0, stream>>>(transposed, reinterpret_cast<const uint16_t*>(B), s.Kc, s.N);
						return launch_tc(ctx, t, cType, A, transposed, C, a, ctx.getDeviceStatus());
					}
				}
				if (forced_path() == 2)
					return AVOCADO_STATUS_NOT_SUPPORTED;
				if (cType == AVOCADO_DTYPE_FLOAT16)
					return launch_simt<half, float, half>(stream, s, A, B, C, a, b);
				return launch_simt<__nv_bfloat16, float, __nv_bfloat16>(stream, s, A, B, C, a, b);
			}
			case AVOCADO_DTYPE_FLOAT32:
			{
				if (abType != cType)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				const float a = getAlphaValue<float>(alpha);
				const float b = getBetaValue<float>(beta);
				if (forced_path() != 1)
				{
					const avStatus_t status = bk::launch_gemm_tf32(ctx, s, A, B, C, a, b);
					if (status != AVOCADO_STATUS_NOT_SUPPORTED)
						return status;
				}
				if (forced_path() == 2)
					return AVOCADO_STATUS_NOT_SUPPORTED;
				return launch_simt<float, float, float>(stream, s, A, B, C, a, b);
			}
			case AVOCADO_DTYPE_FLOAT64:
			{
				if (abType != cType)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				return launch_simt<double, double, double>(stream, s, A, B, C, getAlphaValue<double>(alpha), getBetaValue<double>(beta));
			}
			default:
				return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
		}
	}
}

namespace
{
	/* the protocol of a tensor-core kernel's wait, reduced to its skeleton: a barrier that never completes */
	__global__ void kernel_bounded_wait_selftest(long long limitCycles, int *deviceStatus)
	{
		__shared__ __align__(8) uint64_t never_signalled;
		__shared__ int abort_flag;
		if (threadIdx.x == 0)
		{
			abort_flag = 0;
			umma::mbar_init(&never_signalled, 1);
			umma::mbar_fence_init();
		}
		__syncthreads();
		if (threadIdx.x == 0)
		{
			if (not umma::mbar_wait(&never_signalled, 0, &abort_flag, limitCycles))
				umma::raise_error(&abort_flag, deviceStatus, umma::kErrorSelfTest);
		}
		__syncthreads();
	}
}

namespace avocado
{
	namespace backend
	{
		static avStatus_t run_bounded_wait_selftest(avContextDescriptor_t context, int limitMicroseconds, bool noAllocWord)
		{
			if (limitMicroseconds < 1 or limitMicroseconds > 1000000)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				ctx.setDevice();
				int *word = noAllocWord ? bk::no_alloc_status_word(ctx.device) : ctx.getDeviceStatus();
				if (word == nullptr)
					return AVOCADO_STATUS_BAD_PARAM; /* the fixed array has not been used on this device yet */
				int khz = 0;
				cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx.device);
				const long long cycles = static_cast<long long>(limitMicroseconds) * std::max(khz, 1000) / 1000;
				kernel_bounded_wait_selftest<<<1, 32, 0, ctx.getStream()>>>(cycles, word);
				return checkForErrors();
			AVOCADO_API_END
		}
		avStatus_t cudaRunBoundedWaitSelfTest(avContextDescriptor_t context, int limitMicroseconds)
		{
			return run_bounded_wait_selftest(context, limitMicroseconds, false);
		}
		avStatus_t cudaRunBoundedWaitSelfTestNoAlloc(avContextDescriptor_t context, int limitMicroseconds)
		{
			return run_bounded_wait_selftest(context, limitMicroseconds, true);
		}
	}
}

namespace bk
{
	avStatus_t gemm_batched(ContextObject &ctx, bool transA, bool transB, const void *alpha, const TensorObject &a, const void *aPtr, const TensorObject &b,
			const void *bPtr, const void *beta, const TensorObject &c, void *cPtr)
	{
		if (a.nb_dims != 3 or b.nb_dims != 3 or c.nb_dims != 3)
			return AVOCADO_STATUS_BAD_PARAM;
		if (a.dtype != b.dtype)
			return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
		/* the int8 case exists only in the non-batched call of the reference (src/gemm.cpp:146-208) */
		if (c.dtype == AVOCADO_DTYPE_INT32 or c.dtype == AVOCADO_DTYPE_INT8)
			return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
		GemmShape s;
		s.batch = a.dims[0];
		s.transA = transA;
		s.transB = transB;
		s.M = s.transA ? a.dims[2] : a.dims[1];
		s.Kc = s.transA ? a.dims[1] : a.dims[2];
		s.N = s.transB ? b.dims[1] : b.dims[2];
		const int kb = s.transB ? b.dims[2] : b.dims[1];
		if (b.dims[0] != s.batch or c.dims[0] != s.batch or kb != s.Kc or c.dims[1] != s.M or c.dims[2] != s.N)
			return AVOCADO_STATUS_BAD_PARAM;
		s.lda = a.dims[2];
		s.ldb = b.dims[2];
		s.ldc = c.dims[2];
		s.strideA = a.volumeWithoutFirstDim();
		s.strideB = b.volumeWithoutFirstDim();
		s.strideC = c.volumeWithoutFirstDim();
		ctx.setDevice();
		return gemm_dispatch(ctx, s, a.dtype, c.dtype, alpha, beta, aPtr, bPtr, cPtr);
	}

	avStatus_t flush_deferred_gemm(ContextObject &ctx)
	{
		if (not ctx.deferred.valid)
			return AVOCADO_STATUS_SUCCESS;
		const DeferredGemm d = ctx.deferred;
		ctx.deferred.valid = false;
		noteDeferred(-1);
		return gemm_batched(ctx, false, true, nullptr, d.a, d.aPtr, d.b, d.bPtr, nullptr, d.c, d.cPtr);
	}

	/* Whether this cudaGemmBatched call is the contraction M = V x U^T of an F(4x4,3x3) pipeline in a form the fused
	 * contraction + output transform kernel can take over: 36 planes, (N, T), 16-bit, alpha = 1, beta = 0, and within what
	 * the tensor-core kernel covers (so that launching it later, unfused, behaves exactly like launching it now). */
	static bool deferrable(const ContextObject &ctx, bool transA, bool transB, const void *alpha, const TensorObject &a, const void *aPtr,
			const TensorObject &b, const void *bPtr, const void *beta, const TensorObject &c, const void *cPtr)
	{
		if (not ctx.fuse_winograd or ctx.is_default or transA or not transB)
			return false;
		if (a.nb_dims != 3 or b.nb_dims != 3 or c.nb_dims != 3 or a.dims[0] != 36 or b.dims[0] != 36 or c.dims[0] != 36)
			return false;
		if (a.dtype != b.dtype or a.dtype != c.dtype or (a.dtype != AVOCADO_DTYPE_FLOAT16 and a.dtype != AVOCADO_DTYPE_BFLOAT16))
			return false;
		if (getAlphaValue<float>(alpha) != 1.0f or getBetaValue<float>(beta) != 0.0f)
			return false;
		if (a.dims[2] != b.dims[2] or c.dims[1] != a.dims[1] or c.dims[2] != b.dims[1] or a.dims[1] < 1)
			return false;
		if (aPtr == nullptr or bPtr == nullptr or cPtr == nullptr)
			return false;
		GemmShape s;
		s.batch = 36;
		s.transA = false;
		s.transB = true;
		s.M = a.dims[1];
		s.Kc = a.dims[2];
		s.N = b.dims[1];
		s.lda = s.Kc;
		s.ldb = s.Kc;
		s.ldc = s.N;
		s.strideA = a.volumeWithoutFirstDim();
		s.strideB = b.volumeWithoutFirstDim();
		s.strideC = c.volumeWithoutFirstDim();
		return tc_eligible(ctx, s, c.dtype, aPtr, bPtr, cPtr, 0.0f);
	}

	bool defer_gemm_batched(ContextObject &ctx, bool transA, bool transB, const void *alpha, const TensorObject &a, const void *aPtr, const TensorObject &b,
			const void *bPtr, const void *beta, const TensorObject &c, void *cPtr)
	{
		if (not deferrable(ctx, transA, transB, alpha, a, aPtr, b, bPtr, beta, c, cPtr))
			return false;
		ctx.deferred.valid = true;
		ctx.deferred.a = a;
		ctx.deferred.b = b;
		ctx.deferred.c = c;
		ctx.deferred.aPtr = aPtr;
		ctx.deferred.bPtr = bPtr;
		ctx.deferred.cPtr = cPtr;
		noteDeferred(+1);
		return true;
	}

	avStatus_t gemm_batched_nt_tensor_core(ContextObject &ctx, const TensorObject &a, const void *aPtr, const TensorObject &b, const void *bPtr,
			const TensorObject &c, void *cPtr, int *deviceStatus)
	{
		if (a.nb_dims != 3 or b.nb_dims != 3 or c.nb_dims != 3 or a.dtype != b.dtype or a.dtype != c.dtype)
			return AVOCADO_STATUS_BAD_PARAM;
		GemmShape s;
		s.batch = a.dims[0];
		s.transA = false;
		s.transB = true;
		s.M = a.dims[1];
		s.Kc = a.dims[2];
		s.N = b.dims[1];
		if (b.dims[0] != s.batch or c.dims[0] != s.batch or b.dims[2] != s.Kc or c.dims[1] != s.M or c.dims[2] != s.N)
			return AVOCADO_STATUS_BAD_PARAM;
		s.lda = s.Kc;
		s.ldb = s.Kc;
		s.ldc = s.N;
		s.strideA = a.volumeWithoutFirstDim();
		s.strideB = b.volumeWithoutFirstDim();
		s.strideC = c.volumeWithoutFirstDim();
		if (not tc_eligible(ctx, s, c.dtype, aPtr, bPtr, cPtr, 0.0f))
			return AVOCADO_STATUS_NOT_SUPPORTED;
		ctx.setDevice();
		return launch_tc(ctx, s, c.dtype, aPtr, bPtr, cPtr, 1.0f, deviceStatus);
	}
} /* namespace bk */

namespace avocado
{
	namespace backend
	{
		avStatus_t cudaGemm(avContextDescriptor_t context, avGemmOperation_t aOp, avGemmOperation_t bOp, const void *alpha, const avTensorDescriptor_t aDesc,
				const avMemoryDescriptor_t aMem, const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const void *beta,
				const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				const TensorObject &a = getTensor(aDesc);
				const TensorObject &b = getTensor(bDesc);
				const TensorObject &c = getTensor(cDesc);
				if (a.nb_dims != 2 or b.nb_dims != 2 or c.nb_dims != 2)
					return AVOCADO_STATUS_BAD_PARAM;
				if (a.dtype != b.dtype)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				GemmShape s;
				s.batch = 1;
				s.transA = is_transpose(aOp);
				s.transB = is_transpose(bOp);
				s.M = s.transA ? a.dims[1] : a.dims[0];
				s.Kc = s.transA ? a.dims[0] : a.dims[1];
				s.N = s.transB ? b.dims[0] : b.dims[1];
				const int kb = s.transB ? b.dims[1] : b.dims[0];
				if (kb != s.Kc or c.dims[0] != s.M or c.dims[1] != s.N)
					return AVOCADO_STATUS_BAD_PARAM;
				s.lda = a.dims[1];
				s.ldb = b.dims[1];
				s.ldc = c.dims[1];
				s.strideA = a.volume();
				s.strideB = b.volume();
				s.strideC = c.volume();
				if (a.dtype == AVOCADO_DTYPE_INT8 and (s.lda % 4 != 0 or s.ldb % 4 != 0))
					return AVOCADO_STATUS_BAD_PARAM;
				ctx.setDevice();
				return gemm_dispatch(ctx, s, a.dtype, c.dtype, alpha, beta, getPointer(aMem), getPointer(bMem), getPointer(cMem));
			AVOCADO_API_END
		}

		avStatus_t cudaGemmBatched(avContextDescriptor_t context, avGemmOperation_t aOp, avGemmOperation_t bOp, const void *alpha,
				const avTensorDescriptor_t aDesc, const avMemoryDescriptor_t aMem, const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem,
				const void *beta, const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context); /* a call held back earlier is launched first */
				/* with fusion switched on, the contraction of an F(4x4,3x3) pipeline is held back until the next call shows
				 * whether the output transform consumes it directly */
				if (ctx.fuse_winograd and bk::defer_gemm_batched(ctx, is_transpose(aOp), is_transpose(bOp), alpha, getTensor(aDesc), getPointer(aMem),
						getTensor(bDesc), getPointer(bMem), beta, getTensor(cDesc), getPointer(cMem)))
					return AVOCADO_STATUS_SUCCESS;
				return bk::gemm_batched(ctx, is_transpose(aOp), is_transpose(bOp), alpha, getTensor(aDesc), getPointer(aMem), getTensor(bDesc),
						getPointer(bMem), beta, getTensor(cDesc), getPointer(cMem));
			AVOCADO_API_END
		}
	} /* namespace backend */
} /* namespace avocado */
