/*
 * device_utils.cuh -- storage <-> compute type conversion, aligned vector access and the activation
 * functions shared by every epilogue.
 *
 * All arithmetic on 16-bit storage types is done in float and rounded once, to nearest even, on store.  The
 * reference computes in the storage type (half2 arithmetic, src/numbers/fp16_number.cuh:284-323) and
 * truncates float -> bfloat16 (src/numbers/bf16_number.cuh:40-43); the activation formulas are those of
 * src/activations.cuh:202-425.
 */
#ifndef B200_DEVICE_UTILS_CUH_
#define B200_DEVICE_UTILS_CUH_

#include <Avocado/backend_defs.h>

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <utility>
#include <cuda_runtime.h>

namespace bk
{
	template<typename T> struct ComputeType
	{
			using type = float;
	};
	template<> struct ComputeType<double>
	{
			using type = double;
	};

	__host__ __device__ __forceinline__ float to_compute(half x)
	{
		return __half2float(x);
	}
	__host__ __device__ __forceinline__ float to_compute(__nv_bfloat16 x)
	{
		return __bfloat162float(x);
	}
	__host__ __device__ __forceinline__ float to_compute(float x)
	{
		return x;
	}
	__host__ __device__ __forceinline__ double to_compute(double x)
	{
		return x;
	}

	template<typename T> __device__ __forceinline__ T from_compute(float x);
	template<> __device__ __forceinline__ half from_compute<half>(float x)
	{
		return __float2half_rn(x);
	}
	template<> __device__ __forceinline__ __nv_bfloat16 from_compute<__nv_bfloat16>(float x)
	{
		return __float2bfloat16_rn(x);
	}
	template<> __device__ __forceinline__ float from_compute<float>(float x)
	{
		return x;
	}
	template<typename T> __device__ __forceinline__ T from_compute(double x);
	template<> __device__ __forceinline__ double from_compute<double>(double x)
	{
		return x;
	}

	/* N elements of T moved with one memory instruction of N * sizeof(T) bytes */
	template<typename T, int N>
	struct alignas(sizeof(T) * N) Vec
	{
			T v[N];
	};

	template<typename T, int N>
	__device__ __forceinline__ Vec<T, N> load_vec(const T *ptr)
	{
		return *reinterpret_cast<const Vec<T, N>*>(ptr);
	}
	template<typename T, int N>
	__device__ __forceinline__ void store_vec(T *ptr, const Vec<T, N> &value)
	{
		*reinterpret_cast<Vec<T, N>*>(ptr) = value;
	}

	/* Integer <-> float conversions built from FP32 adds and one FMA.  The hardware conversion instructions have a
	 * small fraction of the FP32 rate, and the requantisation epilogues convert every output element twice.
	 * Both functions round to nearest even, exactly like cvt.rn.f32.s32 and cvt.rni.sat.s8.f32.
	 * 12582912 = 1.5 * 2^23: adding it to an integer |i| < 2^22 places i in the low mantissa bits. */
	__device__ __forceinline__ float small_int_to_float(int32_t i) /* exact for |i| < 2^22 */
	{
		return __int_as_float(0x4B400000 + i) - 12582912.0f;
	}
	__device__ __forceinline__ float int_to_float_rn(int32_t t)
	{
		/* t = hi * 4096 + lo with both parts exact in float; the FMA rounds the exact sum once */
		return fmaf(small_int_to_float(t >> 12), 4096.0f, small_int_to_float(t & 0xFFF));
	}
	__device__ __forceinline__ int32_t float_to_int8_rn_sat(float v) /* NaN gives -128 */
	{
		v = fminf(fmaxf(v, -128.0f), 127.0f);
		return __float_as_int(v + 12582912.0f) - 0x4B400000;
	}

	/* Programmatic dependent launch: a kernel launched with launch_chained() may begin while the kernel before it on the
	 * stream is still draining.  Everything it does before chain_wait() must touch only shared memory, TMEM and barriers;
	 * chain_wait() returns once the previous kernel has completed and its writes are visible.  chain_release() lets the
	 * next kernel on the stream start its own prologue.  Both are no-ops in a kernel launched the ordinary way. */
	__device__ __forceinline__ void chain_wait()
	{
		asm volatile("griddepcontrol.wait;" ::: "memory");
	}
	__device__ __forceinline__ void chain_release()
	{
		asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
	}

	template<typename CT>
	__device__ __forceinline__ CT activation_forward(avocado::backend::avActivationType_t activation, CT x)
	{
		using namespace avocado::backend;
		switch (activation)
		{
			default:
			case AVOCADO_ACTIVATION_LINEAR:
				return x;
			case AVOCADO_ACTIVATION_SIGMOID:
				return static_cast<CT>(1) / (static_cast<CT>(1) + exp(-x));
			case AVOCADO_ACTIVATION_TANH:
				return tanh(x);
			case AVOCADO_ACTIVATION_RELU:
				return max(static_cast<CT>(0), x);
			case AVOCADO_ACTIVATION_SELU:
				return (x >= static_cast<CT>(0)) ? static_cast<CT>(1.05070098f) * x :
						static_cast<CT>(1.05070098f) * static_cast<CT>(1.67326324f) * expm1(x);
			case AVOCADO_ACTIVATION_ELU:
				return (x >= static_cast<CT>(0)) ? x : expm1(x);
			case AVOCADO_ACTIVATION_EXPONENTIAL:
				return exp(x);
			case AVOCADO_ACTIVATION_SOFTPLUS:
				return log1p(exp(x));
			case AVOCADO_ACTIVATION_SOFTSIGN:
				return x / (fabs(x) + static_cast<CT>(1));
		}
	}
	/* The same switch behind a call, for epilogues that are unrolled many times: inlining the transcendental cases into
	 * every copy makes the loop body larger than the instruction cache even when only linear / relu ever run. */
	__device__ __noinline__ float activation_forward_call(avocado::backend::avActivationType_t activation, float x);
} /* namespace bk */

namespace bk
{
	/* AVOCADO_B200_CHAIN=0 launches every kernel the ordinary way (for A/B timing) */
	inline bool chained_launches_enabled()
	{
		static const bool enabled = []()
		{
			const char *env = std::getenv("AVOCADO_B200_CHAIN");
			return not (env != nullptr and std::strcmp(env, "0") == 0);
		}();
		return enabled;
	}
	/* Launches a kernel that calls chain_wait() before its first global access, allowing it to overlap the tail of the
	 * previous kernel on the stream. */
	template<typename ... KernelArgs, typename ... Args>
	cudaError_t launch_chained(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t sharedBytes, cudaStream_t stream, Args &&... args)
	{
		cudaLaunchConfig_t config = { };
		config.gridDim = grid;
		config.blockDim = block;
		config.dynamicSmemBytes = sharedBytes;
		config.stream = stream;
		cudaLaunchAttribute attribute[1];
		attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
		attribute[0].val.programmaticStreamSerializationAllowed = chained_launches_enabled() ? 1 : 0;
		config.attrs = attribute;
		config.numAttrs = 1;
		return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
	}
} /* namespace bk */

#endif /* B200_DEVICE_UTILS_CUH_ */
