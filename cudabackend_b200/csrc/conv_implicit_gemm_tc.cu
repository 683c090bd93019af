/*
 * conv_implicit_gemm_tc.cu -- implicit-GEMM convolution on the Blackwell tensor cores.
 *
 * Counterpart of the reference's kernel_conv_implicit_gemm (src/conv2d_implicit_gemm.cu:150-289), which was meant to
 * compute a 3x3 convolution as a GEMM with the im2col matrix formed on the fly (dp4a for int8) and was left
 * unfinished.  Here:
 *
 *   GEMM view     rows = output pixels (N*Ho*Wo), columns = filters K, contraction = taps x channels (kh*kw*C)
 *   A operand     never materialised: for each (tap, channel block) a TMA copy in im2col mode gathers 128
 *                 consecutive output pixels' input vectors (128 bytes each) straight from the NHWC tensor into
 *                 128-byte-swizzled shared memory; pixels that fall outside the image arrive as zeros (= padding)
 *   B operand     the filters [K, kh*kw, C], contiguous along the contraction: tiled TMA copy of one tap's channel
 *                 block of N filters (a three-dimensional map, so that channels past the end of a partial block
 *                 arrive as zeros like those of the pixels)
 *   MMA           tcgen05.mma, N = 64/128/256; kind::i8 with int32 accumulation for int8, kind::f16 with float32
 *                 accumulation for float16 / bfloat16; accumulator double-buffered in TMEM.  Layers of at least 256
 *                 output pixels run on CTA pairs (cta_group::2, M = 256, each CTA holding half of the filter block),
 *                 smaller ones on single CTAs (cta_group::1, M = 128)
 *   epilogue      four warps drain TMEM: + bias, (requantisation | alpha/z/activation/beta), 16-byte stores
 *
 * Roofline: with C = K = 256 the contraction is 2*9*C*K = 1.18 MFLOP per output pixel against 512 bytes moved, so
 * the kernel is bound by the tensor pipe, not by HBM.
 */
#include "conv_kernels.hpp"
#include "umma.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;
	using namespace bk;

	constexpr int kBlockM = 128;
	constexpr int kBlockKBytes = 128;
	constexpr int kEpilogueWarps = 8;
	constexpr int kEpilogueThreads = kEpilogueWarps * 32;
	constexpr int kThreads = 64 + kEpilogueThreads;

	struct IgParams
	{
			int pixels; /* N * Ho * Wo */
			int filters, channels;
			int out_h, out_w;
			int pad_h, pad_w;
			int kernel_h, kernel_w;
			int rotate;
			int m_blocks, n_blocks, c_blocks, k_blocks;
			int num_tiles;
			const void *bias;
			const float *scales;
			const void *z;
			void *y;
			float alpha1, alpha2, beta;
			int activation;
			int int8_output;
	};

	template<typename T> struct Element;
	template<> struct Element<int8_t>
	{
			static constexpr bool kInteger = true;
			static constexpr uint32_t kFormat = umma::kFormatS8;
			static constexpr uint32_t kAccum = umma::kAccumS32;
			static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_UINT8;
	};
	template<> struct Element<half>
	{
			static constexpr bool kInteger = false;
			static constexpr uint32_t kFormat = umma::kFormatF16;
			static constexpr uint32_t kAccum = umma::kAccumF32;
			static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
	};
	template<> struct Element<__nv_bfloat16>
	{
			static constexpr bool kInteger = false;
			static constexpr uint32_t kFormat = umma::kFormatBF16;
			static constexpr uint32_t kAccum = umma::kAccumF32;
			static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
	};

	template<int BLOCK_N, int STAGES>
	struct IgConfig
	{
			static constexpr int kABytes = kBlockM * kBlockKBytes;
			static constexpr int kBBytes = BLOCK_N * kBlockKBytes;
			static constexpr int kStageBytes = kABytes + kBBytes;
			static constexpr int kSmemBytes = STAGES * kStageBytes + 1024;
			static constexpr int kTmemColumns = 2 * BLOCK_N;
	};

	__device__ __forceinline__ uint32_t pack_half2(float a, float b, half)
	{
		__half2 v = __floats2half2_rn(a, b);
		return *reinterpret_cast<uint32_t*>(&v);
	}
	__device__ __forceinline__ uint32_t pack_half2(float a, float b, __nv_bfloat16)
	{
		__nv_bfloat162 v = __floats2bfloat162_rn(a, b);
		return *reinterpret_cast<uint32_t*>(&v);
	}
	__device__ __forceinline__ float2 unpack_half2(uint32_t raw, half)
	{
		return __half22float2(*reinterpret_cast<__half2*>(&raw));
	}
	__device__ __forceinline__ float2 unpack_half2(uint32_t raw, __nv_bfloat16)
	{
		return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw));
	}

	/* Finishes 32 consecutive filters of one output pixel: r holds the accumulators of filters kc .. kc+31 of pixel m,
	 * scale_s / bias_s the staged per-filter values of the current column block (chunk = 32-filter group inside it). */
	template<typename T>
	__device__ __forceinline__ void epilogue_chunk(const IgParams &p, const uint32_t (&r)[32], int m, int kc, int chunk, const float *scale_s,
			const float *bias_s, avActivationType_t activation)
	{
		const size_t index = static_cast<size_t>(m) * p.filters + kc;
		if constexpr (Element<T>::kInteger)
		{
			if (p.int8_output)
			{
				const int8_t *z = reinterpret_cast<const int8_t*>(p.z);
				uint32_t packed[8];
#pragma unroll
				for (int w = 0; w < 8; w++)
				{
					uint32_t word = 0;
#pragma unroll
					for (int b = 0; b < 4; b++)
					{
						const int j = w * 4 + b;
						const int32_t t = static_cast<int32_t>(r[j]) + __float_as_int(bias_s[chunk * 32 + j]);
						float v = int_to_float_rn(t);
						if (p.alpha1 != 1.0f)
							v = __fmul_rn(p.alpha1, v);
						if (p.scales != nullptr)
							v = __fmul_rn(v, scale_s[chunk * 32 + j]);
						if (z != nullptr)
							v = __fadd_rn(v, __fmul_rn(p.alpha2, small_int_to_float(z[index + j])));
						if (activation == AVOCADO_ACTIVATION_RELU)
							v = fmaxf(v, 0.0f);
						else if (activation != AVOCADO_ACTIVATION_LINEAR)
							v = activation_forward_call(activation, v);
						word |= (static_cast<uint32_t>(float_to_int8_rn_sat(v)) & 0xFFu) << (8 * b);
					}
					packed[w] = word;
				}
				int8_t *dst = reinterpret_cast<int8_t*>(p.y) + index;
				if (kc + 16 <= p.filters)
					*reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
				if (kc + 32 <= p.filters)
					*reinterpret_cast<uint4*>(dst + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
			}
			else
			{
				int32_t *dst = reinterpret_cast<int32_t*>(p.y) + index;
#pragma unroll
				for (int w = 0; w < 8; w++)
					if (kc + 4 * w + 4 <= p.filters)
					{
						uint4 out;
						out.x = static_cast<uint32_t>(static_cast<int32_t>(r[4 * w + 0]) + __float_as_int(bias_s[chunk * 32 + 4 * w + 0]));
						out.y = static_cast<uint32_t>(static_cast<int32_t>(r[4 * w + 1]) + __float_as_int(bias_s[chunk * 32 + 4 * w + 1]));
						out.z = static_cast<uint32_t>(static_cast<int32_t>(r[4 * w + 2]) + __float_as_int(bias_s[chunk * 32 + 4 * w + 2]));
						out.w = static_cast<uint32_t>(static_cast<int32_t>(r[4 * w + 3]) + __float_as_int(bias_s[chunk * 32 + 4 * w + 3]));
						*reinterpret_cast<uint4*>(dst + 4 * w) = out;
					}
			}
		}
		else
		{
			/* 16-bit floating tensors: 32 results = 64 bytes = 4 stores of 8 elements */
			using H = T;
			H *dst = reinterpret_cast<H*>(p.y) + index;
			const H *z = reinterpret_cast<const H*>(p.z);
#pragma unroll
			for (int w = 0; w < 4; w++)
			{
				if (kc + 8 * w + 8 > p.filters)
					continue;
				uint4 zraw = make_uint4(0, 0, 0, 0), yraw = make_uint4(0, 0, 0, 0);
				if (z != nullptr)
					zraw = *reinterpret_cast<const uint4*>(z + index + 8 * w);
				if (p.beta != 0.0f)
					yraw = *reinterpret_cast<const uint4*>(dst + 8 * w);
				const uint32_t zw[4] = { zraw.x, zraw.y, zraw.z, zraw.w };
				const uint32_t yw[4] = { yraw.x, yraw.y, yraw.z, yraw.w };
				uint32_t out[4];
#pragma unroll
				for (int q = 0; q < 4; q++)
				{
					const int j = 8 * w + 2 * q;
					float v0 = fmaf(p.alpha1, __uint_as_float(r[j]), bias_s[chunk * 32 + j]);
					float v1 = fmaf(p.alpha1, __uint_as_float(r[j + 1]), bias_s[chunk * 32 + j + 1]);
					if (z != nullptr)
					{
						const float2 zz = unpack_half2(zw[q], H());
						v0 = fmaf(p.alpha2, zz.x, v0);
						v1 = fmaf(p.alpha2, zz.y, v1);
					}
					if (activation == AVOCADO_ACTIVATION_RELU)
					{
						v0 = fmaxf(v0, 0.0f);
						v1 = fmaxf(v1, 0.0f);
					}
					else if (activation != AVOCADO_ACTIVATION_LINEAR)
					{
						v0 = activation_forward_call(activation, v0);
						v1 = activation_forward_call(activation, v1);
					}
					if (p.beta != 0.0f)
					{
						const float2 yy = unpack_half2(yw[q], H());
						v0 = fmaf(p.beta, yy.x, v0);
						v1 = fmaf(p.beta, yy.y, v1);
					}
					out[q] = pack_half2(v0, v1, H());
				}
				*reinterpret_cast<uint4*>(dst + 8 * w) = make_uint4(out[0], out[1], out[2], out[3]);
			}
		}
	}

	/*
	 * Short forms of the epilogue for the common cases.  The general form below decides per element what to apply; with
	 * 32 elements unrolled that is several hundred branches and an instruction footprint beyond the instruction cache,
	 * and the eight epilogue warps then take longer over a tile than the tensor pipe does.  The short forms are
	 * branch-free, take bias and scale from shared memory four at a time and pack with byte permutes.
	 *
	 * int8 -> int8 with alpha1 == 1 and linear or relu activation.  Same roundings as the general form: int32 + bias,
	 * to float (round to nearest even), * scale, [+ alpha2 * z], max(lower), min(127), round to nearest even.
	 * lower is 0 for relu and -128 otherwise (a NaN becomes lower, as in the general form).
	 */
	template<bool HAS_Z>
	__device__ __forceinline__ void epilogue_chunk_int8_short(const IgParams &p, const uint32_t (&r)[32], int m, int kc, int chunk, const float *scale_s,
			const float *bias_s, float lower)
	{
		const size_t index = static_cast<size_t>(m) * p.filters + kc;
		const int4 *bias4 = reinterpret_cast<const int4*>(bias_s + chunk * 32);
		const float4 *scale4 = reinterpret_cast<const float4*>(scale_s + chunk * 32);
		const bool first_half = kc + 16 <= p.filters, second_half = kc + 32 <= p.filters;
		uint32_t zw[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
		if constexpr (HAS_Z)
		{
			const int8_t *z = reinterpret_cast<const int8_t*>(p.z) + index;
			if (first_half)
			{
				const uint4 t = *reinterpret_cast<const uint4*>(z);
				zw[0] = t.x, zw[1] = t.y, zw[2] = t.z, zw[3] = t.w;
			}
			if (second_half)
			{
				const uint4 t = *reinterpret_cast<const uint4*>(z + 16);
				zw[4] = t.x, zw[5] = t.y, zw[6] = t.z, zw[7] = t.w;
			}
		}
		uint32_t packed[8];
#pragma unroll
		for (int w = 0; w < 8; w++)
		{
			const int4 b = bias4[w];
			const float4 sc = scale4[w];
			float v0 = __fmul_rn(__int2float_rn(static_cast<int32_t>(r[4 * w + 0]) + b.x), sc.x);
			float v1 = __fmul_rn(__int2float_rn(static_cast<int32_t>(r[4 * w + 1]) + b.y), sc.y);
			float v2 = __fmul_rn(__int2float_rn(static_cast<int32_t>(r[4 * w + 2]) + b.z), sc.z);
			float v3 = __fmul_rn(__int2float_rn(static_cast<int32_t>(r[4 * w + 3]) + b.w), sc.w);
			if constexpr (HAS_Z)
			{
				/* sign-extended bytes of the z word; |z| <= 128 is exact in float */
				v0 = __fadd_rn(v0, __fmul_rn(p.alpha2, small_int_to_float(static_cast<int32_t>(zw[w] << 24) >> 24)));
				v1 = __fadd_rn(v1, __fmul_rn(p.alpha2, small_int_to_float(static_cast<int32_t>(zw[w] << 16) >> 24)));
				v2 = __fadd_rn(v2, __fmul_rn(p.alpha2, small_int_to_float(static_cast<int32_t>(zw[w] << 8) >> 24)));
				v3 = __fadd_rn(v3, __fmul_rn(p.alpha2, small_int_to_float(static_cast<int32_t>(zw[w]) >> 24)));
			}
			/* after the clamp, adding 1.5 * 2^23 leaves the rounded integer (two's complement) in the low byte */
			const uint32_t u0 = __float_as_uint(__fadd_rn(fminf(fmaxf(v0, lower), 127.0f), 12582912.0f));
			const uint32_t u1 = __float_as_uint(__fadd_rn(fminf(fmaxf(v1, lower), 127.0f), 12582912.0f));
			const uint32_t u2 = __float_as_uint(__fadd_rn(fminf(fmaxf(v2, lower), 127.0f), 12582912.0f));
			const uint32_t u3 = __float_as_uint(__fadd_rn(fminf(fmaxf(v3, lower), 127.0f), 12582912.0f));
			packed[w] = __byte_perm(__byte_perm(u0, u1, 0x0040), __byte_perm(u2, u3, 0x0040), 0x5410);
		}
		int8_t *dst = reinterpret_cast<int8_t*>(p.y) + index;
		if (first_half)
			*reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
		if (second_half)
			*reinterpret_cast<uint4*>(dst + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
	}

	/* 16-bit floating tensors without z and with beta == 0: y = act(alpha1 * acc + bias), linear or relu */
	template<typename H, bool RELU>
	__device__ __forceinline__ void epilogue_chunk_half_short(const IgParams &p, const uint32_t (&r)[32], int m, int kc, int chunk, const float *bias_s)
	{
		H *dst = reinterpret_cast<H*>(p.y) + static_cast<size_t>(m) * p.filters + kc;
		const float4 *bias4 = reinterpret_cast<const float4*>(bias_s + chunk * 32);
#pragma unroll
		for (int w = 0; w < 4; w++)
		{
			const float4 b0 = bias4[2 * w], b1 = bias4[2 * w + 1];
			float v[8];
			v[0] = fmaf(p.alpha1, __uint_as_float(r[8 * w + 0]), b0.x);
			v[1] = fmaf(p.alpha1, __uint_as_float(r[8 * w + 1]), b0.y);
			v[2] = fmaf(p.alpha1, __uint_as_float(r[8 * w + 2]), b0.z);
			v[3] = fmaf(p.alpha1, __uint_as_float(r[8 * w + 3]), b0.w);
			v[4] = fmaf(p.alpha1, __uint_as_float(r[8 * w + 4]), b1.x);
			v[5] = fmaf(p.alpha1, __uint_as_float(r[8 * w + 5]), b1.y);
			v[6] = fmaf(p.alpha1, __uint_as_float(r[8 * w + 6]), b1.z);
			v[7] = fmaf(p.alpha1, __uint_as_float(r[8 * w + 7]), b1.w);
			if constexpr (RELU)
			{
#pragma unroll
				for (int q = 0; q < 8; q++)
					v[q] = fmaxf(v[q], 0.0f);
			}
			if (kc + 8 * w + 8 <= p.filters)
				*reinterpret_cast<uint4*>(dst + 8 * w) = make_uint4(pack_half2(v[0], v[1], H()), pack_half2(v[2], v[3], H()), pack_half2(v[4], v[5], H()),
						pack_half2(v[6], v[7], H()));
		}
	}

	enum EpilogueForm
	{
		kFormGeneral = 0, kFormInt8Short = 1, kFormInt8ShortZ = 2, kFormHalfShortLinear = 3, kFormHalfShortRelu = 4
	};
	template<typename T>
	__device__ __forceinline__ int epilogue_form(const IgParams &p)
	{
		const bool simple_activation = p.activation == AVOCADO_ACTIVATION_LINEAR or p.activation == AVOCADO_ACTIVATION_RELU;
		if constexpr (Element<T>::kInteger)
		{
			if (p.int8_output and p.alpha1 == 1.0f and simple_activation)
				return (p.z != nullptr) ? kFormInt8ShortZ : kFormInt8Short;
		}
		else
		{
			if (p.z == nullptr and p.beta == 0.0f and simple_activation)
				return (p.activation == AVOCADO_ACTIVATION_RELU) ? kFormHalfShortRelu : kFormHalfShortLinear;
		}
		return kFormGeneral;
	}
	template<typename T>
	__device__ __forceinline__ void epilogue_chunk_any(int form, const IgParams &p, const uint32_t (&r)[32], int m, int kc, int chunk, const float *scale_s,
			const float *bias_s, avActivationType_t activation)
	{
		if constexpr (Element<T>::kInteger)
		{
			const float lower = (activation == AVOCADO_ACTIVATION_RELU) ? 0.0f : -128.0f;
			if (form == kFormInt8Short)
				epilogue_chunk_int8_short<false>(p, r, m, kc, chunk, scale_s, bias_s, lower);
			else if (form == kFormInt8ShortZ)
				epilogue_chunk_int8_short<true>(p, r, m, kc, chunk, scale_s, bias_s, lower);
			else
				epilogue_chunk<T>(p, r, m, kc, chunk, scale_s, bias_s, activation);
		}
		else
		{
			if (form == kFormHalfShortLinear)
				epilogue_chunk_half_short<T, false>(p, r, m, kc, chunk, bias_s);
			else if (form == kFormHalfShortRelu)
				epilogue_chunk_half_short<T, true>(p, r, m, kc, chunk, bias_s);
			else
				epilogue_chunk<T>(p, r, m, kc, chunk, scale_s, bias_s, activation);
		}
	}

	template<typename T, int BLOCK_N, int STAGES>
	__global__ void __launch_bounds__(kThreads, 1) kernel_implicit_gemm_tc(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW,
			IgParams p, int *deviceStatus)
	{
		using Cfg = IgConfig<BLOCK_N, STAGES>;
		constexpr int kElemsPerBlock = kBlockKBytes / static_cast<int>(sizeof(T)); /* channels per contraction block */
		constexpr int kMmaK = 32 / static_cast<int>(sizeof(T)); /* elements consumed by one tcgen05.mma */
		extern __shared__ uint8_t smem_raw[];
		uint8_t *smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

		__shared__ __align__(8) uint64_t full_bar[STAGES];
		__shared__ __align__(8) uint64_t empty_bar[STAGES];
		__shared__ __align__(8) uint64_t tmem_full_bar[2];
		__shared__ __align__(8) uint64_t tmem_empty_bar[2];
		__shared__ uint32_t tmem_base_slot;
		__shared__ int abort_flag;
		__shared__ volatile int epilogue_go;
		__shared__ __align__(16) float scale_s[BLOCK_N];
		__shared__ __align__(16) float bias_s[BLOCK_N]; /* int32 bit patterns in the integer case */

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
				umma::mbar_init(&tmem_empty_bar[a], kEpilogueThreads);
			}
			umma::mbar_fence_init();
			umma::prefetch_tensormap(&mapX);
			umma::prefetch_tensormap(&mapW);
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
		const int taps = p.kernel_h * p.kernel_w;
		/* everything above touched only shared memory, barriers and TMEM: the kernel after this one on the stream may
		 * start its own set-up now, and this one waits here for the kernel before it */
		chain_release();
		chain_wait();

		if (warp == 0)
		{
			if (lane == 0)
			{
				int stage = 0;
				uint32_t phase = 0;
				bool ok = true;
				const int image = p.out_h * p.out_w;
				for (int tile = blockIdx.x; tile < p.num_tiles and ok; tile += gridDim.x)
				{
					const int nb = tile % p.n_blocks;
					const int mb = tile / p.n_blocks;
					const int m0 = mb * kBlockM;
					const int n = m0 / image;
					const int rem = m0 - n * image;
					const int oh = rem / p.out_w;
					const int ow = rem - oh * p.out_w;
					/* counters instead of divisions: this single thread's instruction latency is part of every stage's cost */
					int r = 0, s = 0, cb = 0, tap = 0;
					for (int kb = 0; kb < p.k_blocks; kb++)
					{
						const int wtap = p.rotate ? (taps - 1 - tap) : tap;
						if (not umma::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_ptr))
						{
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorStageWait);
							ok = false;
							break;
						}
						uint8_t *a_dst = smem + stage * Cfg::kStageBytes;
						uint8_t *b_dst = a_dst + Cfg::kABytes;
						umma::mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
						umma::tma_load_im2col_4d(a_dst, &mapX, &full_bar[stage], cb * kElemsPerBlock, ow + p.pad_w, oh + p.pad_h, n, static_cast<uint16_t>(s),
								static_cast<uint16_t>(r));
						umma::tma_load_3d(b_dst, &mapW, &full_bar[stage], cb * kElemsPerBlock, wtap, nb * BLOCK_N);
						if (++stage == STAGES)
						{
							stage = 0;
							phase ^= 1u;
						}
						if (++cb == p.c_blocks)
						{
							cb = 0;
							tap++;
							if (++s == p.kernel_w)
							{
								s = 0;
								r++;
							}
						}
					}
				}
			}
		}
		else if (warp == 1)
		{
			if (lane == 0)
			{
				constexpr uint32_t idesc = umma::make_instr_desc(Element<T>::kAccum, Element<T>::kFormat, Element<T>::kFormat, false, false, kBlockM, BLOCK_N);
				/* the descriptor's address field counts 16-byte units: the descriptor of a later stage is this one plus a constant */
				const uint64_t a_desc0 = umma::make_smem_desc(umma::smem_u32(smem), 16, 1024, umma::kSwizzle128B);
				int stage = 0;
				uint32_t phase = 0;
				int it = 0;
				bool ok = true;
				for (int tile = blockIdx.x; tile < p.num_tiles and ok; tile += gridDim.x, it++)
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
					for (int kb = 0; kb < p.k_blocks; kb++)
					{
						if (not umma::mbar_wait(&full_bar[stage], phase, abort_ptr))
						{
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
							ok = false;
							break;
						}
						umma::tcgen05_fence_after();
						const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage * (Cfg::kStageBytes / 16));
						const uint64_t b_desc = a_desc + Cfg::kABytes / 16;
						/* four MMAs, each consuming 32 bytes of every row of the 128-byte-wide stage */
						static_assert(kElemsPerBlock / kMmaK == 4, "a stage is four MMAs deep");
						if constexpr (Element<T>::kInteger)
							umma::mma_i8_k4(tmem_d, a_desc, b_desc, idesc, kb != 0);
						else
							umma::mma_f16_k4(tmem_d, a_desc, b_desc, idesc, kb != 0);
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
			/* eight warps: warp w drains TMEM lanes 32*(w%4).. (the only lanes it may read) and, of the BLOCK_N columns,
			 * the half given by (w-2)/4 */
			const int quarter = warp % 4;
			const int column_half = (warp - 2) / 4;
			const int row = quarter * 32 + lane;
			const int epi_thread = threadIdx.x - 64;
			const avActivationType_t activation = static_cast<avActivationType_t>(p.activation);
			const int form = epilogue_form<T>(p);
			int it = 0;
			int staged_nb = -1;
			for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, it++)
			{
				const int nb = tile % p.n_blocks;
				const int mb = tile / p.n_blocks;
				const int acc = it & 1;
				const uint32_t acc_phase = static_cast<uint32_t>(it >> 1) & 1u;
				const int k0 = nb * BLOCK_N;

				/* per-filter scale and bias of this column block: staged once per change of block */
				if (staged_nb != nb)
				{
					if (staged_nb >= 0)
						umma::named_barrier_sync(1, kEpilogueThreads); /* nobody still reads the previous block's values */
					for (int j = epi_thread; j < BLOCK_N; j += kEpilogueThreads)
					{
						const int k = k0 + j;
						float sc = 1.0f, bi = 0.0f;
						if (k < p.filters)
						{
							if (p.scales != nullptr)
								sc = p.scales[k];
							if (p.bias != nullptr)
								bi = reinterpret_cast<const float*>(p.bias)[k]; /* float, or int32 bit pattern */
						}
						scale_s[j] = sc;
						bias_s[j] = bi;
					}
					staged_nb = nb;
				}
				if (epi_thread == 0)
				{
					const bool ready = umma::mbar_wait(&tmem_full_bar[acc], acc_phase, abort_ptr);
					if (not ready)
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorEpilogueWait);
					epilogue_go = ready ? 1 : 0;
				}
				umma::named_barrier_sync(1, kEpilogueThreads);
				if (epilogue_go == 0)
					break;
				umma::tcgen05_fence_after();

				const int m = mb * kBlockM + row;
				const bool row_valid = m < p.pixels;
				const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BLOCK_N);
#pragma unroll 1
				for (int chunk = column_half * (BLOCK_N / 64); chunk < (column_half + 1) * (BLOCK_N / 64); chunk++)
				{
					uint32_t r[32];
					umma::tmem_load_32x32(t_addr + static_cast<uint32_t>(chunk * 32), r);
					umma::tmem_load_wait();
					const int kc = k0 + chunk * 32; /* first filter of this chunk */
					if (not row_valid or kc >= p.filters)
						continue;
					epilogue_chunk_any<T>(form, p, r, m, kc, chunk, scale_s, bias_s, activation);
				}
				/* accumulator drained: hand it back to the MMA warp */
				umma::tcgen05_fence_before();
				umma::mbar_arrive(&tmem_empty_bar[acc]);
			}
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

	/*
	 * The same convolution on CTA pairs: two CTAs on neighbouring SMs share one tile of 256 pixels x BLOCK_N filters.  Each
	 * loads its own 128 pixels and only HALF of the filter block; the first CTA of the pair issues tcgen05.mma
	 * cta_group::2 (M = 256), which reads both halves in place and leaves each CTA with the accumulator rows of its own
	 * pixels.
	 *
	 * Why this is the default form.  Measured on this kernel's loads and MMAs without an epilogue (148 CTAs, int8, 256
	 * filters): the thread that issues the MMAs spends about 100 cycles in a wait on a full barrier, 55 per MMA and 120 in
	 * a commit, and the thread that issues the copies about 370 per 128-byte contraction block; a shared-memory stage
	 * stays occupied for the 1500-1900 cycles its copies take to land plus the time its MMAs run.  With one 128-byte
	 * block per stage the single-CTA kernel is therefore paced by those two threads and by the four stages that fit
	 * (600 cycles per block and 128 pixels, 870 with the epilogue warps running) and not by the tensor pipe (4 MMAs of
	 * 139 cycles).  A pair halves the filter bytes per SM, so a stage can hold KB = 2 blocks three or four deep: one wait
	 * and one commit per eight MMAs, half as many copies per SM and pixel, and the pipe sets the pace (560 cycles per
	 * block and 256 pixels).
	 *
	 *   full_bar[s]        first CTA only: one arrival (its producer, which also posts the bytes of BOTH CTAs' copies);
	 *                      the second CTA's copies report their bytes to it
	 *   empty_bar[s]       both CTAs: the commit after a stage's MMAs arrives on both
	 *   tmem_full_bar[a]   both CTAs: the commit after a tile's last MMA arrives on both
	 *   tmem_empty_bar[a]  first CTA only: one arrival per epilogue warp of both CTAs
	 */
	/* RES > 0: the filters stay in shared memory.  When the layer has a single block of filters and at most RES contraction
	 * blocks, every tile multiplies by the same B operand: each CTA copies its half of it once (RES x kBBytes) and the ring
	 * carries only the pixels.  The producer issues half as many copies per tile and the filters cross from L2 once per CTA
	 * instead of once per tile; measured on 64 x 56 x 56 x 64 -> 64 float16: 34.6 -> 33.4 us (those layers are paced by the
	 * MMA thread and the per-tile hand-over, not by the copies). */
	template<int BLOCK_N, int KB, int STAGES, int RES>
	struct IgPairConfig
	{
			static constexpr int kHalfN = BLOCK_N / 2;
			static constexpr int kABytes = kBlockM * kBlockKBytes;
			static constexpr int kBBytes = kHalfN * kBlockKBytes;
			static constexpr int kBlockBytes = (RES > 0) ? kABytes : kABytes + kBBytes; /* what the ring holds per 128-byte contraction block */
			static constexpr int kStageBytes = KB * kBlockBytes;
			static constexpr int kResidentBytes = RES * kBBytes;
			static constexpr int kSmemBytes = kResidentBytes + STAGES * kStageBytes + 1024;
			static constexpr int kTmemColumns = 2 * BLOCK_N;
			static_assert(kSmemBytes <= 232448, "stages exceed the shared memory of an SM");
	};

	template<typename T, int BLOCK_N, int KB, int STAGES, int RES>
	__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) kernel_implicit_gemm_tc_pair(const __grid_constant__ CUtensorMap mapX,
			const __grid_constant__ CUtensorMap mapW, IgParams p, int *deviceStatus)
	{
		using Cfg = IgPairConfig<BLOCK_N, KB, STAGES, RES>;
		constexpr int kElemsPerBlock = kBlockKBytes / static_cast<int>(sizeof(T));
		constexpr int kMmaK = 32 / static_cast<int>(sizeof(T));
		extern __shared__ uint8_t smem_raw[];
		uint8_t *smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

		__shared__ __align__(8) uint64_t full_bar[STAGES];
		__shared__ __align__(8) uint64_t empty_bar[STAGES];
		__shared__ __align__(8) uint64_t tmem_full_bar[2];
		__shared__ __align__(8) uint64_t tmem_empty_bar[2];
		__shared__ __align__(8) uint64_t resident_bar; /* first CTA only: the resident filters of both CTAs have landed */
		__shared__ uint32_t tmem_base_slot;
		__shared__ int abort_flag;
		__shared__ volatile int epilogue_go;
		__shared__ __align__(16) float scale_s[BLOCK_N];
		__shared__ __align__(16) float bias_s[BLOCK_N];

		const int warp = threadIdx.x / 32;
		const int lane = threadIdx.x % 32;
		const uint32_t rank = umma::cluster_cta_rank();
		const int pair = blockIdx.x / 2;
		const int num_pairs = gridDim.x / 2;

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
				umma::mbar_init(&tmem_empty_bar[a], 2 * kEpilogueWarps);
			}
			umma::mbar_init(&resident_bar, 1);
			umma::mbar_fence_init();
			umma::prefetch_tensormap(&mapX);
			umma::prefetch_tensormap(&mapW);
		}
		if (warp == 1)
		{
			umma::tmem_alloc_pair(&tmem_base_slot, Cfg::kTmemColumns);
			umma::tmem_relinquish_pair();
		}
		umma::tcgen05_fence_before();
		__syncthreads();
		umma::cluster_sync_all(); /* both CTAs' barriers exist before anything arrives on them */
		umma::tcgen05_fence_after();
		const uint32_t tmem_base = tmem_base_slot;
		volatile int *abort_ptr = &abort_flag;
		const int taps = p.kernel_h * p.kernel_w;
		uint8_t *resident = smem;                       /* RES > 0: this CTA's half of the filters, one kBBytes tile per contraction block */
		uint8_t *ring = smem + Cfg::kResidentBytes;     /* the stages */
		/* everything above touched only shared memory, barriers and TMEM: the kernel after this one on the stream may
		 * start its own set-up now, and this one waits here for the kernel before it */
		chain_release();
		chain_wait();

		if (warp == 0)
		{
			if (lane == 0)
			{
				int stage = 0;
				uint32_t phase = 0;
				bool ok = true;
				const int image = p.out_h * p.out_w;
				if constexpr (RES > 0)
				{
					/* the whole filter operand once: contraction block kb = (tap, channel block) in the order the tiles walk them */
					const uint32_t bar = umma::map_to_cta(umma::smem_u32(&resident_bar), 0);
					if (rank == 0)
						umma::mbar_arrive_expect_tx(&resident_bar, static_cast<uint32_t>(2 * p.k_blocks * Cfg::kBBytes));
					int cb = 0, tap = 0;
					for (int kb = 0; kb < p.k_blocks; kb++)
					{
						const int wtap = p.rotate ? (taps - 1 - tap) : tap;
						umma::tma_load_3d_pair(resident + kb * Cfg::kBBytes, &mapW, bar, cb * kElemsPerBlock, wtap, static_cast<int>(rank) * Cfg::kHalfN);
						if (++cb == p.c_blocks)
						{
							cb = 0;
							tap++;
						}
					}
				}
				for (int tile = pair; tile < p.num_tiles and ok; tile += num_pairs)
				{
					const int nb = tile % p.n_blocks;
					const int mb = tile / p.n_blocks;
					int m0 = mb * (2 * kBlockM) + static_cast<int>(rank) * kBlockM;
					if (m0 >= p.pixels)
						m0 = 0; /* the odd half block past the end: any valid pixels will do, its rows are never stored */
					const int n = m0 / image;
					const int rem = m0 - n * image;
					const int oh = rem / p.out_w;
					const int ow = rem - oh * p.out_w;
					const int filter0 = nb * BLOCK_N + static_cast<int>(rank) * Cfg::kHalfN;
					int r = 0, s = 0, cb = 0, tap = 0;
					for (int kb = 0; kb < p.k_blocks; kb += KB)
					{
						const int count = min(KB, p.k_blocks - kb);
						if (not umma::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_ptr))
						{
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorStageWait);
							ok = false;
							break;
						}
						const uint32_t bar = umma::map_to_cta(umma::smem_u32(&full_bar[stage]), 0);
						if (rank == 0)
							umma::mbar_arrive_expect_tx(&full_bar[stage], static_cast<uint32_t>(2 * count * Cfg::kBlockBytes));
#pragma unroll
						for (int j = 0; j < KB; j++)
							if (j < count)
							{
								uint8_t *a_dst = ring + stage * Cfg::kStageBytes + j * Cfg::kBlockBytes;
								umma::tma_load_im2col_4d_pair(a_dst, &mapX, bar, cb * kElemsPerBlock, ow + p.pad_w, oh + p.pad_h, n, static_cast<uint16_t>(s),
										static_cast<uint16_t>(r));
								if constexpr (RES == 0)
								{
									const int wtap = p.rotate ? (taps - 1 - tap) : tap;
									umma::tma_load_3d_pair(a_dst + Cfg::kABytes, &mapW, bar, cb * kElemsPerBlock, wtap, filter0);
								}
								if (++cb == p.c_blocks)
								{
									cb = 0;
									tap++;
									if (++s == p.kernel_w)
									{
										s = 0;
										r++;
									}
								}
							}
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
			if (lane == 0 and rank == 0)
			{
				constexpr uint32_t idesc = umma::make_instr_desc(Element<T>::kAccum, Element<T>::kFormat, Element<T>::kFormat, false, false, 2 * kBlockM,
						BLOCK_N);
				const uint64_t a_desc0 = umma::make_smem_desc(umma::smem_u32(ring), 16, 1024, umma::kSwizzle128B);
				const uint64_t resident_desc0 = umma::make_smem_desc(umma::smem_u32(resident), 16, 1024, umma::kSwizzle128B);
				int stage = 0;
				uint32_t phase = 0;
				int it = 0;
				bool ok = true;
				if constexpr (RES > 0)
				{
					if (not umma::mbar_wait(&resident_bar, 0, abort_ptr))
					{
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
						ok = false;
					}
				}
				for (int tile = pair; tile < p.num_tiles and ok; tile += num_pairs, it++)
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
					for (int kb = 0; kb < p.k_blocks; kb += KB)
					{
						const int count = min(KB, p.k_blocks - kb);
						if (not umma::mbar_wait(&full_bar[stage], phase, abort_ptr))
						{
							umma::raise_error(abort_ptr, deviceStatus, umma::kErrorTmaWait);
							ok = false;
							break;
						}
						umma::tcgen05_fence_after();
						static_assert(kElemsPerBlock / kMmaK == 4, "a contraction block is four MMAs deep");
#pragma unroll
						for (int j = 0; j < KB; j++)
							if (j < count)
							{
								const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((stage * Cfg::kStageBytes + j * Cfg::kBlockBytes) / 16);
								const uint64_t b_desc = (RES > 0) ? resident_desc0 + static_cast<uint64_t>(((kb + j) * Cfg::kBBytes) / 16) : a_desc + Cfg::kABytes / 16;
								if constexpr (Element<T>::kInteger)
									umma::mma_i8_pair_k4(tmem_d, a_desc, b_desc, idesc, (kb + j) != 0);
								else
									umma::mma_f16_pair_k4(tmem_d, a_desc, b_desc, idesc, (kb + j) != 0);
							}
						umma::mma_commit_pair(&empty_bar[stage], 3);
						if (++stage == STAGES)
						{
							stage = 0;
							phase ^= 1u;
						}
					}
					if (ok)
						umma::mma_commit_pair(&tmem_full_bar[acc], 3);
				}
			}
		}
		else
		{
			const int quarter = warp % 4;
			const int column_half = (warp - 2) / 4;
			const int row = quarter * 32 + lane;
			const int epi_thread = threadIdx.x - 64;
			const avActivationType_t activation = static_cast<avActivationType_t>(p.activation);
			const int form = epilogue_form<T>(p);
			int it = 0;
			int staged_nb = -1;
			for (int tile = pair; tile < p.num_tiles; tile += num_pairs, it++)
			{
				const int nb = tile % p.n_blocks;
				const int mb = tile / p.n_blocks;
				const int acc = it & 1;
				const uint32_t acc_phase = static_cast<uint32_t>(it >> 1) & 1u;
				const int k0 = nb * BLOCK_N;

				if (staged_nb != nb)
				{
					if (staged_nb >= 0)
						umma::named_barrier_sync(1, kEpilogueThreads);
					for (int j = epi_thread; j < BLOCK_N; j += kEpilogueThreads)
					{
						const int k = k0 + j;
						float sc = 1.0f, bi = 0.0f;
						if (k < p.filters)
						{
							if (p.scales != nullptr)
								sc = p.scales[k];
							if (p.bias != nullptr)
								bi = reinterpret_cast<const float*>(p.bias)[k];
						}
						scale_s[j] = sc;
						bias_s[j] = bi;
					}
					staged_nb = nb;
				}
				if (epi_thread == 0)
				{
					const bool ready = umma::mbar_wait(&tmem_full_bar[acc], acc_phase, abort_ptr);
					if (not ready)
						umma::raise_error(abort_ptr, deviceStatus, umma::kErrorEpilogueWait);
					epilogue_go = ready ? 1 : 0;
				}
				umma::named_barrier_sync(1, kEpilogueThreads);
				if (epilogue_go == 0)
					break;
				umma::tcgen05_fence_after();

				const int m = mb * (2 * kBlockM) + static_cast<int>(rank) * kBlockM + row;
				const bool row_valid = m < p.pixels;
				const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BLOCK_N);
#pragma unroll 1
				for (int chunk = column_half * (BLOCK_N / 64); chunk < (column_half + 1) * (BLOCK_N / 64); chunk++)
				{
					uint32_t r[32];
					umma::tmem_load_32x32(t_addr + static_cast<uint32_t>(chunk * 32), r);
					umma::tmem_load_wait();
					const int kc = k0 + chunk * 32;
					if (not row_valid or kc >= p.filters)
						continue;
					epilogue_chunk_any<T>(form, p, r, m, kc, chunk, scale_s, bias_s, activation);
				}
				/* accumulator drained: each warp tells the first CTA's MMA thread */
				umma::tcgen05_fence_before();
				__syncwarp();
				if (lane == 0)
					umma::mbar_arrive_cluster(umma::map_to_cta(umma::smem_u32(&tmem_empty_bar[acc]), 0));
			}
		}

		/* neither CTA may leave (or free TMEM) while the other can still touch its shared memory, barriers or TMEM */
		__syncthreads();
		if (abort_flag != 0)
			umma::drain_after_abort();
		umma::tcgen05_fence_before();
		umma::cluster_sync_all();
		if (warp == 1)
		{
			umma::tcgen05_fence_after();
			umma::tmem_dealloc_pair(tmem_base, Cfg::kTmemColumns);
		}
	}

	template<typename T, int BLOCK_N, int KB, int STAGES, int RES = 0>
	avStatus_t launch_pair(ContextObject &ctx, const CUtensorMap &mapX, const CUtensorMap &mapW, IgParams &p)
	{
		using Cfg = IgPairConfig<BLOCK_N, KB, STAGES, RES>;
		auto kernel = kernel_implicit_gemm_tc_pair<T, BLOCK_N, KB, STAGES, RES>;
		static PerDeviceOnce configured;
		if (configured.run(ctx.device, [&]() -> cudaError_t { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes); }) != cudaSuccess)
		{
			cudaGetLastError();
			return AVOCADO_STATUS_EXECUTION_FAILED;
		}
		p.n_blocks = (p.filters + BLOCK_N - 1) / BLOCK_N;
		const int m_pairs = (p.pixels + 2 * kBlockM - 1) / (2 * kBlockM);
		const long long tiles = static_cast<long long>(m_pairs) * p.n_blocks;
		if (tiles > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		p.num_tiles = static_cast<int>(tiles);
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		const int pairs = std::max(1, std::min(p.num_tiles, sms / 2));
		const cudaError_t launched = launch_chained(kernel, dim3(2 * pairs), dim3(kThreads), Cfg::kSmemBytes, ctx.getStream(), mapX, mapW, p,
				ctx.getDeviceStatus());
		if (launched != cudaSuccess)
			return convertStatus(launched);
		return checkForErrors();
	}

	template<typename T, int BLOCK_N, int STAGES>
	avStatus_t launch_config(ContextObject &ctx, const CUtensorMap &mapX, const CUtensorMap &mapW, IgParams &p)
	{
		using Cfg = IgConfig<BLOCK_N, STAGES>;
		auto kernel = kernel_implicit_gemm_tc<T, BLOCK_N, STAGES>;
		static PerDeviceOnce configured;
		if (configured.run(ctx.device, [&]() -> cudaError_t { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes); }) != cudaSuccess)
		{
			cudaGetLastError();
			return AVOCADO_STATUS_EXECUTION_FAILED;
		}
		p.n_blocks = (p.filters + BLOCK_N - 1) / BLOCK_N;
		const long long tiles = static_cast<long long>(p.m_blocks) * p.n_blocks;
		if (tiles > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		p.num_tiles = static_cast<int>(tiles);
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		const int grid = std::min(p.num_tiles, sms);
		const cudaError_t launched = launch_chained(kernel, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, ctx.getStream(), mapX, mapW, p,
				ctx.getDeviceStatus());
		if (launched != cudaSuccess)
			return convertStatus(launched);
		return checkForErrors();
	}

	bool tensor_cores_enabled()
	{
		static const bool enabled = []()
		{
			const char *env = std::getenv("AVOCADO_B200_CONV");
			return not (env != nullptr and std::strcmp(env, "direct") == 0);
		}();
		return enabled;
	}

	/* AVOCADO_B200_CONV=single keeps every layer on the single-CTA kernel (for A/B timing); the default sends layers of
	 * at least two 128-pixel blocks to the CTA-pair kernel */
	bool pair_kernel_enabled()
	{
		static const bool enabled = []()
		{
			const char *env = std::getenv("AVOCADO_B200_CONV");
			return not (env != nullptr and std::strcmp(env, "single") == 0);
		}();
		return enabled;
	}

	/* AVOCADO_B200_FILTERS=stream keeps the filters in the ring of stages for every layer (for A/B timing) */
	bool resident_filters_enabled()
	{
		static const bool enabled = []()
		{
			const char *env = std::getenv("AVOCADO_B200_FILTERS");
			return not (env != nullptr and std::strcmp(env, "stream") == 0);
		}();
		return enabled;
	}

	template<typename T>
	avStatus_t launch_typed(ContextObject &ctx, const ConvArgs &args, avDataType_t yType, const void *alpha1, const void *alpha2, const void *beta)
	{
		const int elem = static_cast<int>(sizeof(T));
		const int block_channels = kBlockKBytes / elem;
		/* Shapes the kernel covers; everything else goes to the direct kernel.  The channel count need not fill whole
		 * 128-byte blocks: both copies (im2col pixels, and filters through a map whose innermost dimension is the channels
		 * of ONE tap) fill the channels past the end with zeros.  What TMA needs is 16-byte pitches: C times the element
		 * size. */
		if ((args.channels * elem) % 16 != 0)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const int out_align = Element<T>::kInteger ? 16 : 8;
		if (args.filters % out_align != 0 or args.filters < 16)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (args.kernel_h > 16 or args.kernel_w > 16 or args.kernel_h * args.kernel_w > 64)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const long long pixels = static_cast<long long>(args.batch) * args.out_height * args.out_width;
		if (pixels == 0)
			return AVOCADO_STATUS_SUCCESS;
		if (pixels > 0x7FFFFF00ll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		/* bounding box of the im2col map: base pixels run from pad to pad + out - 1 */
		const int lower[2] = { args.pad_w, args.pad_h };
		const int upper[2] = { args.out_width - args.width + args.pad_w, args.out_height - args.height + args.pad_h };
		for (int i = 0; i < 2; i++)
			if (lower[i] < -128 or lower[i] > 127 or upper[i] < -128 or upper[i] > 127)
				return AVOCADO_STATUS_NOT_SUPPORTED;
		/* less than one block of output pixels: the direct kernel is the better fit */
		if (pixels < kBlockM)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (reinterpret_cast<uintptr_t>(args.x) % 16 != 0 or reinterpret_cast<uintptr_t>(args.w) % 16 != 0 or reinterpret_cast<uintptr_t>(args.y) % 16 != 0
				or (args.z != nullptr and reinterpret_cast<uintptr_t>(args.z) % 16 != 0))
			return AVOCADO_STATUS_NOT_SUPPORTED;

		CUtensorMap mapX, mapW;
		{
			const uint64_t dims[4] = { static_cast<uint64_t>(args.channels), static_cast<uint64_t>(args.width), static_cast<uint64_t>(args.height),
					static_cast<uint64_t>(args.batch) };
			const uint64_t strides[3] = { static_cast<uint64_t>(args.channels) * elem, static_cast<uint64_t>(args.width) * args.channels * elem,
					static_cast<uint64_t>(args.height) * args.width * args.channels * elem };
			if (not umma::make_im2col_map(&mapX, Element<T>::kTma, const_cast<void*>(args.x), dims, strides, lower, upper, block_channels, kBlockM,
					CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		const int taps = args.kernel_h * args.kernel_w;
		const int block_n = (args.filters <= 64) ? 64 : (args.filters <= 128) ? 128 : 256;
		const bool use_pair = pair_kernel_enabled() and pixels > kBlockM;
		{
			const uint64_t dims[3] = { static_cast<uint64_t>(args.channels), static_cast<uint64_t>(taps), static_cast<uint64_t>(args.filters) };
			const uint64_t strides[2] = { static_cast<uint64_t>(args.channels) * elem, static_cast<uint64_t>(taps) * args.channels * elem };
			/* the pair kernel copies the filter block in two halves, one per CTA */
			const uint32_t box_rows = use_pair ? static_cast<uint32_t>(block_n / 2) : static_cast<uint32_t>(block_n);
			const uint32_t box[3] = { static_cast<uint32_t>(block_channels), 1u, box_rows };
			if (not umma::make_tensor_map(&mapW, Element<T>::kTma, 3, const_cast<void*>(args.w), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}

		IgParams p;
		p.pixels = static_cast<int>(pixels);
		p.filters = args.filters;
		p.channels = args.channels;
		p.out_h = args.out_height;
		p.out_w = args.out_width;
		p.pad_h = args.pad_h;
		p.pad_w = args.pad_w;
		p.kernel_h = args.kernel_h;
		p.kernel_w = args.kernel_w;
		p.rotate = args.rotate_kernel ? 1 : 0;
		p.m_blocks = static_cast<int>((pixels + kBlockM - 1) / kBlockM);
		p.c_blocks = (args.channels + block_channels - 1) / block_channels;
		p.k_blocks = taps * p.c_blocks;
		p.bias = args.bias;
		p.scales = reinterpret_cast<const float*>(args.scales);
		p.z = args.z;
		p.y = args.y;
		p.alpha1 = getAlphaValue<float>(alpha1);
		p.alpha2 = getAlphaValue<float>(alpha2);
		p.beta = getBetaValue<float>(beta);
		p.activation = static_cast<int>(args.activation);
		p.int8_output = (yType == AVOCADO_DTYPE_INT8) ? 1 : 0;
		/* contraction blocks per stage x stages, measured per tile width: three blocks three deep for 64 filters (20 KB per
		 * block and CTA; 5-11 % faster than two blocks four deep on the 64-channel layers), two blocks four deep for 128
		 * (three were 2 % faster on 128 x 28 x 28 x 128 and 6 % slower on 32 x 112 x 112 x 64), two blocks three deep for 256 */
		/* with at most nine contraction blocks (3x3 filters over at most 128 bytes of channels) and one block of filters the
		 * filters stay in shared memory (36 or 72 KB per CTA) */
		const bool resident = use_pair and resident_filters_enabled() and p.k_blocks <= 9 and args.filters <= block_n;
		switch (block_n)
		{
			case 64:
				if (resident)
					return launch_pair<T, 64, 3, 3, 9>(ctx, mapX, mapW, p);
				return use_pair ? launch_pair<T, 64, 3, 3>(ctx, mapX, mapW, p) : launch_config<T, 64, 6>(ctx, mapX, mapW, p);
			case 128:
				if (resident)
					return launch_pair<T, 128, 2, 4, 9>(ctx, mapX, mapW, p);
				return use_pair ? launch_pair<T, 128, 2, 4>(ctx, mapX, mapW, p) : launch_config<T, 128, 5>(ctx, mapX, mapW, p);
			default:
				return use_pair ? launch_pair<T, 256, 2, 3>(ctx, mapX, mapW, p) : launch_config<T, 256, 4>(ctx, mapX, mapW, p);
		}
	}
}

namespace bk
{
	__device__ __noinline__ float activation_forward_call(avocado::backend::avActivationType_t activation, float x)
	{
		return activation_forward(activation, x);
	}

	avStatus_t launch_implicit_gemm_tc(ContextObject &ctx, const ConvArgs &args, avDataType_t xType, avDataType_t yType, const void *alpha1,
			const void *alpha2, const void *beta)
	{
		if (not tensor_cores_enabled() or cuda_sm_version(ctx.device) != 100)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		switch (xType)
		{
			case AVOCADO_DTYPE_INT8:
				return launch_typed<int8_t>(ctx, args, yType, alpha1, alpha2, beta);
			case AVOCADO_DTYPE_FLOAT16:
				return launch_typed<half>(ctx, args, yType, alpha1, alpha2, beta);
			case AVOCADO_DTYPE_BFLOAT16:
				return launch_typed<__nv_bfloat16>(ctx, args, yType, alpha1, alpha2, beta);
			default:
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
	}
} /* namespace bk */
