/*
 * umma.cuh -- thin inline-PTX layer over the Blackwell (sm_100a) data-movement and tensor-core instructions
 * used by the contraction kernels: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM allocation, MMA,
 * commit, TMEM load) and the shared-memory / instruction descriptors they take.
 *
 * The reference has nothing comparable: its only contractions are cuBLAS calls (src/gemm.cpp:155-205) and
 * dp4a / FFMA loops (src/conv2d_implicit_gemm.cu:115-138).
 *
 * Every wait in this file is bounded: a wait that does not complete within kWaitLimitCycles SM cycles returns
 * false, the caller records an error code in the context's device status word and leaves its loop, so a
 * protocol error ends the kernel instead of hanging the GPU.
 */
#ifndef B200_UMMA_CUH_
#define B200_UMMA_CUH_

#include <cuda.h>
#include <cuda_runtime_api.h>
#include <cstdint>

namespace umma
{
	/* about one second at 2 GHz; a healthy wait lasts microseconds */
	constexpr long long kWaitLimitCycles = 2000000000ll;

	enum DeviceError
	{
		kErrorNone = 0, kErrorTmaWait = 1, kErrorMmaWait = 2, kErrorEpilogueWait = 3, kErrorStageWait = 4, kErrorSelfTest = 5
	};

	__device__ __forceinline__ uint32_t smem_u32(const void *ptr)
	{
		return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
	}
	__device__ __forceinline__ bool elect_one()
	{
		uint32_t pred = 0;
		asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(pred));
		return pred != 0;
	}

	/* ---- mbarrier ------------------------------------------------------------------------------------- */
	__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
	{
		asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
	}
	__device__ __forceinline__ void mbar_fence_init()
	{
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
	{
		asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
	}
	__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
	{
		asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
	}
	__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
	{
		uint32_t done = 0;
		asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
				: "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
		return done != 0;
	}
	/* Waits for the phase with the given parity to complete.  Returns false when the limit ran out or when
	 * another role of the CTA has raised *abortFlag (a shared-memory word) because its own wait ran out. */
	__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abortFlag, long long limitCycles = kWaitLimitCycles)
	{
		if (mbar_try_wait(bar, parity))
			return true;
		const long long start = clock64();
		while (true)
		{
#pragma unroll 1
			for (int i = 0; i < 64; i++)
				if (mbar_try_wait(bar, parity))
					return true;
			if (*abortFlag != 0 or clock64() - start > limitCycles)
				return false;
		}
	}
	/* Records a failed wait: sets the CTA's abort flag and ORs the code into the context's status word. */
	__device__ __forceinline__ void raise_error(volatile int *abortFlag, int *deviceStatus, int code)
	{
		*abortFlag = 1;
		if (deviceStatus != nullptr)
			atomicOr(deviceStatus, 1 << code);
	}
	/* After an abort: gives copies and MMAs that are still in flight time to land before shared memory and
	 * TMEM are released (they complete within microseconds; this waits about 200). */
	__device__ __forceinline__ void drain_after_abort()
	{
		for (int i = 0; i < 200; i++)
			__nanosleep(1000);
	}

	/* ---- proxies and tcgen05 fences ------------------------------------------------------------------- */
	__device__ __forceinline__ void fence_proxy_async_smem()
	{
		asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
	}
	__device__ __forceinline__ void tcgen05_fence_before()
	{
		asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	}
	__device__ __forceinline__ void tcgen05_fence_after()
	{
		asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	}
	__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads)
	{
		asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
	}

	/* ---- TMA --------------------------------------------------------------------------------------------
	 * The innermost coordinate times the element size must be a multiple of 16 bytes; callers only pass
	 * multiples of the 128-byte box width.  No multicast variant is provided on purpose. */
	__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map)
	{
		asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
	}
	__device__ __forceinline__ void tma_load_3d(void *smemDst, const CUtensorMap *map, uint64_t *bar, int c0, int c1, int c2)
	{
		asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
				::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
	}
	__device__ __forceinline__ void tma_load_4d(void *smemDst, const CUtensorMap *map, uint64_t *bar, int c0, int c1, int c2, int c3)
	{
		asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
				::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
	}
	__device__ __forceinline__ void tma_load_2d(void *smemDst, const CUtensorMap *map, uint64_t *bar, int c0, int c1)
	{
		asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
				::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
	}
	/* im2col mode over an NHWC tensor: (c, w, h, n) is the first base pixel (in input coordinates, may be negative
	 * inside the bounding box of the map), (offW, offH) the filter tap added to every base pixel; the copy walks
	 * pixelsPerColumn base pixels along w, then h, then n, and delivers channelsPerPixel channels of each. */
	__device__ __forceinline__ void tma_load_im2col_4d(void *smemDst, const CUtensorMap *map, uint64_t *bar, int c, int w, int h, int n, uint16_t offW,
			uint16_t offH)
	{
		asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
				::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(offW), "h"(offH)
				: "memory");
	}
	__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, const void *smemSrc, int c0, int c1, int c2)
	{
		asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
				::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smemSrc)), "r"(c0), "r"(c1), "r"(c2) : "memory");
	}
	__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *smemSrc, int c0, int c1)
	{
		asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
				::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smemSrc)), "r"(c0), "r"(c1) : "memory");
	}
	__device__ __forceinline__ void tma_store_commit()
	{
		asm volatile("cp.async.bulk.commit_group;" ::: "memory");
	}
	/* waits until at most N of this thread's store groups still READ their shared-memory source */
	template<int N>
	__device__ __forceinline__ void tma_store_wait_read()
	{
		asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
	}
	template<int N>
	__device__ __forceinline__ void tma_store_wait_all()
	{
		asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
	}

	/* ---- TMEM ------------------------------------------------------------------------------------------- */
	/* whole-warp call; columns is a power of two in [32, 512]; the base address lands in *smemResult */
	__device__ __forceinline__ void tmem_alloc(uint32_t *smemResult, uint32_t columns)
	{
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smemResult)), "r"(columns) : "memory");
	}
	__device__ __forceinline__ void tmem_relinquish()
	{
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns)
	{
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
	}

	/* ---- descriptors ------------------------------------------------------------------------------------
	 * Shared-memory matrix descriptor (64 bit): [13:0] start address >> 4, [29:16] leading byte offset >> 4,
	 * [45:32] stride byte offset >> 4, [47:46] = 1 (Blackwell), [51:49] base offset, [63:61] swizzle mode. */
	constexpr uint64_t kSwizzleNone = 0, kSwizzle128BBase32B = 1, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6;

	__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smemAddr, uint32_t leadingBytes, uint32_t strideBytes, uint64_t swizzle)
	{
		uint64_t desc = 0;
		desc |= static_cast<uint64_t>((smemAddr & 0x3FFFFu) >> 4);
		desc |= static_cast<uint64_t>((leadingBytes >> 4) & 0x3FFFu) << 16;
		desc |= static_cast<uint64_t>((strideBytes >> 4) & 0x3FFFu) << 32;
		desc |= static_cast<uint64_t>(1) << 46;
		desc |= swizzle << 61;
		return desc;
	}

	/* Instruction descriptor (32 bit) of tcgen05.mma kind::f16 / kind::tf32 / kind::i8:
	 * [5:4] accumulator format (1 = f32, 2 = s32), [9:7] A format, [12:10] B format, [15] A is MN-major,
	 * [16] B is MN-major, [22:17] N >> 3, [28:24] M >> 4. */
	constexpr uint32_t kFormatF16 = 0, kFormatBF16 = 1, kFormatTF32 = 2, kFormatS8 = 1;
	constexpr uint32_t kAccumF32 = 1, kAccumS32 = 2;

	__host__ __device__ constexpr uint32_t make_instr_desc(uint32_t accum, uint32_t aFormat, uint32_t bFormat, bool aMnMajor, bool bMnMajor, uint32_t m,
			uint32_t n)
	{
		return (accum << 4) | (aFormat << 7) | (bFormat << 10) | ((aMnMajor ? 1u : 0u) << 15) | ((bMnMajor ? 1u : 0u) << 16) | ((n >> 3) << 17)
				| ((m >> 4) << 24);
	}

	/* ---- MMA, commit, TMEM load -------------------------------------------------------------------------- */
	/* D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread */
	__device__ __forceinline__ void mma_f16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulate)
	{
		asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
				::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate ? 1u : 0u) : "memory");
	}
	__device__ __forceinline__ void mma_tf32(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulate)
	{
		asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
				::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate ? 1u : 0u) : "memory");
	}
	__device__ __forceinline__ void mma_i8(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulate)
	{
		asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
				::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate ? 1u : 0u) : "memory");
	}
	/* Four MMAs over one 128-byte-wide K-major stage (descriptor + 0, 2, 4, 6 = 32-byte steps along the contraction) in
	 * one instruction sequence.  The issuing thread is a single thread whose own instruction latency adds to every MMA it
	 * issues (measured: about 55 cycles per MMA issued this way, 100-120 for a wait on a barrier, 120-150 for a commit),
	 * while an MMA of M = 128 retires in 86 cycles for any N up to 128 and in 140 at N = 256: with one such group per
	 * barrier round trip the thread, not the tensor pipe, sets the pace, so the per-MMA predicate set-up and descriptor
	 * arithmetic of the single-MMA wrappers is folded here and kernels put two or more groups behind one wait and commit. */
#define B200_UMMA_K4(NAME, KIND) \
	__device__ __forceinline__ void NAME(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulateFirst) \
	{ \
		asm volatile("{\n\t.reg .pred p, q;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t" \
				"setp.ne.b32 p, %4, 0;\n\tsetp.eq.u32 q, %3, %3;\n\t" \
				"add.s64 a1, %1, 2;\n\tadd.s64 b1, %2, 2;\n\tadd.s64 a2, %1, 4;\n\tadd.s64 b2, %2, 4;\n\tadd.s64 a3, %1, 6;\n\tadd.s64 b3, %2, 6;\n\t" \
				"tcgen05.mma.cta_group::1.kind::" KIND " [%0], %1, %2, %3, p;\n\t" \
				"tcgen05.mma.cta_group::1.kind::" KIND " [%0], a1, b1, %3, q;\n\t" \
				"tcgen05.mma.cta_group::1.kind::" KIND " [%0], a2, b2, %3, q;\n\t" \
				"tcgen05.mma.cta_group::1.kind::" KIND " [%0], a3, b3, %3, q;\n\t}" \
				::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulateFirst ? 1u : 0u) : "memory"); \
	}
	B200_UMMA_K4(mma_f16_k4, "f16")
	B200_UMMA_K4(mma_i8_k4, "i8")
#undef B200_UMMA_K4
	/* makes the mbarrier track completion of all MMAs issued so far by this thread (one arrival) */
	__device__ __forceinline__ void mma_commit(uint64_t *bar)
	{
		asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
	}
	__device__ __forceinline__ void tmem_load_wait()
	{
		asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
	}
	/* 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane (base lane + t) */
	__device__ __forceinline__ void tmem_load_32x32(uint32_t taddr, uint32_t (&r)[32])
	{
		asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
				"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
				"%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
				: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
				"=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
				"=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
				"=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
				: "r"(taddr) : "memory");
	}
	__device__ __forceinline__ void tmem_load_32x16(uint32_t taddr, uint32_t (&r)[16])
	{
		asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
				"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
				: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
				"=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
				: "r"(taddr) : "memory");
	}

	/* ---- CTA pairs (clusters of two) ---------------------------------------------------------------------
	 * A pair of CTAs on neighbouring SMs can issue one tcgen05.mma over both SMs' shared memory and TMEM
	 * (cta_group::2): each CTA supplies half of the rows of A and half of the rows of B, and receives its half of
	 * the accumulator rows.  The helpers below are what such a kernel needs on top of the single-CTA ones.  Only
	 * the commit is multicast (an mbarrier arrival at the same offset in both CTAs); no load is. */
	__device__ __forceinline__ uint32_t cluster_cta_rank()
	{
		uint32_t rank;
		asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
		return rank;
	}
	/* shared::cluster address of the given shared::cta address in the CTA of the given rank */
	__device__ __forceinline__ uint32_t map_to_cta(uint32_t smemAddr, uint32_t rank)
	{
		uint32_t result;
		asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(result) : "r"(smemAddr), "r"(rank));
		return result;
	}
	/* all threads of all CTAs of the cluster */
	__device__ __forceinline__ void cluster_sync_all()
	{
		asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
	}
	__device__ __forceinline__ void mbar_arrive_cluster(uint32_t clusterAddr)
	{
		asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
	}
	/* loads into THIS CTA's shared memory whose byte count is reported to an mbarrier of either CTA of the pair */
	__device__ __forceinline__ void tma_load_2d_pair(void *smemDst, const CUtensorMap *map, uint32_t barClusterAddr, int c0, int c1)
	{
		asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%3, %4}], [%2];"
				::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(barClusterAddr), "r"(c0), "r"(c1) : "memory");
	}
	__device__ __forceinline__ void tma_load_3d_pair(void *smemDst, const CUtensorMap *map, uint32_t barClusterAddr, int c0, int c1, int c2)
	{
		asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%3, %4, %5}], [%2];"
				::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(barClusterAddr), "r"(c0), "r"(c1), "r"(c2) : "memory");
	}
	__device__ __forceinline__ void tma_load_im2col_4d_pair(void *smemDst, const CUtensorMap *map, uint32_t barClusterAddr, int c, int w, int h, int n,
			uint16_t offW, uint16_t offH)
	{
		asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
				::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(barClusterAddr), "r"(c), "r"(w), "r"(h), "r"(n), "h"(offW), "h"(offH)
				: "memory");
	}
	/* the same warp index of BOTH CTAs calls these; *smemResult sits at the same offset in both */
	__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smemResult, uint32_t columns)
	{
		asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smemResult)), "r"(columns) : "memory");
	}
	__device__ __forceinline__ void tmem_relinquish_pair()
	{
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
	}
	__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns)
	{
		asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
	}
	/* issued by ONE thread of the pair's first CTA; descriptors hold offsets that are valid in both CTAs */
	__device__ __forceinline__ void mma_f16_pair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulate)
	{
		asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
				::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate ? 1u : 0u) : "memory");
	}
	__device__ __forceinline__ void mma_i8_pair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulate)
	{
		asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
				::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate ? 1u : 0u) : "memory");
	}
	/* four cta_group::2 MMAs over one 128-byte-wide K-major stage, as mma_*_k4 below do for a single CTA */
#define B200_UMMA_PAIR_K4(NAME, KIND) \
	__device__ __forceinline__ void NAME(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulateFirst) \
	{ \
		asm volatile("{\n\t.reg .pred p, q;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t" \
				"setp.ne.b32 p, %4, 0;\n\tsetp.eq.u32 q, %3, %3;\n\t" \
				"add.s64 a1, %1, 2;\n\tadd.s64 b1, %2, 2;\n\tadd.s64 a2, %1, 4;\n\tadd.s64 b2, %2, 4;\n\tadd.s64 a3, %1, 6;\n\tadd.s64 b3, %2, 6;\n\t" \
				"tcgen05.mma.cta_group::2.kind::" KIND " [%0], %1, %2, %3, p;\n\t" \
				"tcgen05.mma.cta_group::2.kind::" KIND " [%0], a1, b1, %3, q;\n\t" \
				"tcgen05.mma.cta_group::2.kind::" KIND " [%0], a2, b2, %3, q;\n\t" \
				"tcgen05.mma.cta_group::2.kind::" KIND " [%0], a3, b3, %3, q;\n\t}" \
				::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulateFirst ? 1u : 0u) : "memory"); \
	}
	B200_UMMA_PAIR_K4(mma_f16_pair_k4, "f16")
	B200_UMMA_PAIR_K4(mma_i8_pair_k4, "i8")
#undef B200_UMMA_PAIR_K4
	/* one arrival on the mbarrier at this offset in every CTA named by the mask, once all MMAs issued so far are done */
	__device__ __forceinline__ void mma_commit_pair(uint64_t *bar, uint16_t ctaMask)
	{
		asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
				::"r"(smem_u32(bar)), "h"(ctaMask) : "memory");
	}

	/* ---- host side: tensor maps ------------------------------------------------------------------------- */
	typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
			const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

	/* cuTensorMapEncodeTiled looked up through the runtime, so the library does not link against libcuda */
	inline EncodeTiledFn encode_tiled_fn()
	{
		static EncodeTiledFn fn = []() -> EncodeTiledFn
		{
			void *ptr = nullptr;
			cudaDriverEntryPointQueryResult result;
			if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess or result != cudaDriverEntryPointSuccess)
			{
				cudaGetLastError();
				return nullptr;
			}
			return reinterpret_cast<EncodeTiledFn>(ptr);
		}();
		return fn;
	}

	/* rank <= 5; dims/box innermost first; strides in bytes for dims 1..rank-1.  Returns false on failure. */
	inline bool make_tensor_map(CUtensorMap *map, CUtensorMapDataType dtype, int rank, void *base, const uint64_t *dims, const uint64_t *stridesBytes,
			const uint32_t *box, CUtensorMapSwizzle swizzle)
	{
		EncodeTiledFn fn = encode_tiled_fn();
		if (fn == nullptr)
			return false;
		cuuint64_t gdims[5], gstrides[4];
		cuuint32_t gbox[5], estrides[5];
		for (int i = 0; i < rank; i++)
		{
			gdims[i] = dims[i];
			gbox[i] = box[i];
			estrides[i] = 1;
			if (i > 0)
				gstrides[i - 1] = stridesBytes[i - 1];
		}
		const CUresult status = fn(map, dtype, static_cast<cuuint32_t>(rank), base, gdims, gstrides, gbox, estrides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
				CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
		return status == CUDA_SUCCESS;
	}

	typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*, const int*,
			cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

	inline EncodeIm2colFn encode_im2col_fn()
	{
		static EncodeIm2colFn fn = []() -> EncodeIm2colFn
		{
			void *ptr = nullptr;
			cudaDriverEntryPointQueryResult result;
			if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &ptr, cudaEnableDefault, &result) != cudaSuccess or result != cudaDriverEntryPointSuccess)
			{
				cudaGetLastError();
				return nullptr;
			}
			return reinterpret_cast<EncodeIm2colFn>(ptr);
		}();
		return fn;
	}

	/* im2col map over an NHWC tensor (dims innermost first: C, W, H, N).  lower/upper corner are the offsets of the
	 * bounding box of base pixels from (0,0) and from (W-1,H-1), in {W, H} order. */
	inline bool make_im2col_map(CUtensorMap *map, CUtensorMapDataType dtype, void *base, const uint64_t dims[4], const uint64_t stridesBytes[3],
			const int lowerCorner[2], const int upperCorner[2], uint32_t channelsPerPixel, uint32_t pixelsPerColumn, CUtensorMapSwizzle swizzle)
	{
		EncodeIm2colFn fn = encode_im2col_fn();
		if (fn == nullptr)
			return false;
		cuuint64_t gdims[4] = { dims[0], dims[1], dims[2], dims[3] };
		cuuint64_t gstrides[3] = { stridesBytes[0], stridesBytes[1], stridesBytes[2] };
		cuuint32_t estrides[4] = { 1, 1, 1, 1 };
		const CUresult status = fn(map, dtype, 4, base, gdims, gstrides, lowerCorner, upperCorner, channelsPerPixel, pixelsPerColumn, estrides,
				CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
		return status == CUDA_SUCCESS;
	}
} /* namespace umma */

#endif /* B200_UMMA_CUH_ */
