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
} /* namespace bk */

#endif /* B200_DEVICE_UTILS_CUH_ */
