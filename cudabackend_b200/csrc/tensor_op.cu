/*
 * tensor_op.cu -- the two element-wise steps that sit right behind a convolution when it is not fused into one:
 *
 *   cudaAddBias            y = alpha1 * activation(alpha2 * x + b + beta1 * z) + beta2 * z + beta3 * y
 *                          (reference src/tensor_op.cu:199-228 kernel, :493-551 entry point); b is broadcast along
 *                          every dimension but the trailing ones it covers, float32 for 16-bit and float32 tensors,
 *                          float64 for float64 tensors
 *   cudaActivationForward  y = alpha * activation(x) + beta * y   (reference src/activations.cu, header :490-491)
 *
 * Both are bound by HBM: one thread moves 16 bytes of every operand per step when the row length and the pointers
 * allow it, single elements otherwise; arithmetic is float32 (float64 for float64 tensors) with one rounding on store.
 * The activation is a template parameter for linear and relu so that the common cases carry no switch.
 */
#include <Avocado/cuda_backend.h>

#include "objects.hpp"
#include "device_utils.cuh"

#include <algorithm>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;
	using namespace bk;

	/* ACT: 0 linear, 1 relu, 2 any (switch) */
	template<int ACT, typename CT>
	__device__ __forceinline__ CT apply_activation(avActivationType_t activation, CT x)
	{
		if (ACT == 0)
			return x;
		if (ACT == 1)
			return x > static_cast<CT>(0) ? x : static_cast<CT>(0);
		return activation_forward(activation, x);
	}

	template<typename T, typename BT, int VEC, int ACT>
	__global__ void __launch_bounds__(256) kernel_add_bias(T *y, const T *__restrict__ x, const BT *__restrict__ bias, const T *z, long long rows, int row_length,
			typename ComputeType<T>::type alpha1, typename ComputeType<T>::type alpha2, typename ComputeType<T>::type beta1,
			typename ComputeType<T>::type beta2, typename ComputeType<T>::type beta3, avActivationType_t activation)
	{
		using CT = typename ComputeType<T>::type;
		const int vectors_per_row = row_length / VEC;
		const long long total = rows * vectors_per_row;
		const bool use_z = (z != nullptr) and (beta1 != static_cast<CT>(0) or beta2 != static_cast<CT>(0));
		for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			const int column = static_cast<int>(i % vectors_per_row) * VEC;
			const long long offset = i * VEC;
			const Vec<T, VEC> xv = load_vec<T, VEC>(x + offset);
			Vec<T, VEC> zv, yv, out;
			if (use_z)
				zv = load_vec<T, VEC>(z + offset);
			if (beta3 != static_cast<CT>(0))
				yv = load_vec<T, VEC>(y + offset);
#pragma unroll
			for (int k = 0; k < VEC; k++)
			{
				CT t = alpha2 * static_cast<CT>(to_compute(xv.v[k])) + static_cast<CT>(bias[column + k]);
				if (use_z)
				{
					const CT e = static_cast<CT>(to_compute(zv.v[k]));
					t = alpha1 * apply_activation<ACT>(activation, t + beta1 * e) + beta2 * e;
				}
				else
					t = alpha1 * apply_activation<ACT>(activation, t);
				if (beta3 != static_cast<CT>(0))
					t += beta3 * static_cast<CT>(to_compute(yv.v[k]));
				out.v[k] = from_compute<T>(t);
			}
			store_vec<T, VEC>(y + offset, out);
		}
	}

	template<typename T, int VEC, int ACT>
	__global__ void __launch_bounds__(256) kernel_activation(T *y, const T *__restrict__ x, long long vectors, typename ComputeType<T>::type alpha,
			typename ComputeType<T>::type beta, avActivationType_t activation)
	{
		using CT = typename ComputeType<T>::type;
		for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < vectors; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			const long long offset = i * VEC;
			const Vec<T, VEC> xv = load_vec<T, VEC>(x + offset);
			Vec<T, VEC> yv, out;
			if (beta != static_cast<CT>(0))
				yv = load_vec<T, VEC>(y + offset);
#pragma unroll
			for (int k = 0; k < VEC; k++)
			{
				CT t = alpha * apply_activation<ACT>(activation, static_cast<CT>(to_compute(xv.v[k])));
				if (beta != static_cast<CT>(0))
					t += beta * static_cast<CT>(to_compute(yv.v[k]));
				out.v[k] = from_compute<T>(t);
			}
			store_vec<T, VEC>(y + offset, out);
		}
	}

	int grid_for(const ContextObject &ctx, long long work_items)
	{
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		return static_cast<int>(std::max<long long>(1, std::min<long long>((work_items + 255) / 256, static_cast<long long>(sms) * 8)));
	}
	int activation_class(avActivationType_t activation)
	{
		return activation == AVOCADO_ACTIVATION_LINEAR ? 0 : activation == AVOCADO_ACTIVATION_RELU ? 1 : 2;
	}
	bool aligned16(const void *p)
	{
		return p == nullptr or reinterpret_cast<uintptr_t>(p) % 16 == 0;
	}

	template<typename T, typename BT, int VEC>
	avStatus_t launch_add_bias_vec(ContextObject &ctx, void *y, const void *x, const void *bias, const void *z, long long rows, int row_length, const void *alpha1,
			const void *alpha2, const void *beta1, const void *beta2, const void *beta3, avActivationType_t activation)
	{
		using CT = typename ComputeType<T>::type;
		const CT a1 = getAlphaValue<CT>(alpha1), a2 = getAlphaValue<CT>(alpha2);
		const CT b1 = getBetaValue<CT>(beta1), b2 = getBetaValue<CT>(beta2), b3 = getBetaValue<CT>(beta3);
		const int grid = grid_for(ctx, rows * (row_length / VEC));
		T *yp = reinterpret_cast<T*>(y);
		const T *xp = reinterpret_cast<const T*>(x), *zp = reinterpret_cast<const T*>(z);
		const BT *bp = reinterpret_cast<const BT*>(bias);
		switch (activation_class(activation))
		{
			case 0:
				kernel_add_bias<T, BT, VEC, 0> <<<grid, 256, 0, ctx.getStream()>>>(yp, xp, bp, zp, rows, row_length, a1, a2, b1, b2, b3, activation);
				break;
			case 1:
				kernel_add_bias<T, BT, VEC, 1> <<<grid, 256, 0, ctx.getStream()>>>(yp, xp, bp, zp, rows, row_length, a1, a2, b1, b2, b3, activation);
				break;
			default:
				kernel_add_bias<T, BT, VEC, 2> <<<grid, 256, 0, ctx.getStream()>>>(yp, xp, bp, zp, rows, row_length, a1, a2, b1, b2, b3, activation);
				break;
		}
		return checkForErrors();
	}
	template<typename T, typename BT>
	avStatus_t launch_add_bias(ContextObject &ctx, void *y, const void *x, const void *bias, const void *z, long long rows, int row_length, const void *alpha1,
			const void *alpha2, const void *beta1, const void *beta2, const void *beta3, avActivationType_t activation)
	{
		constexpr int kVec = 16 / static_cast<int>(sizeof(T));
		if (row_length % kVec == 0 and aligned16(y) and aligned16(x) and aligned16(z))
			return launch_add_bias_vec<T, BT, kVec>(ctx, y, x, bias, z, rows, row_length, alpha1, alpha2, beta1, beta2, beta3, activation);
		return launch_add_bias_vec<T, BT, 1>(ctx, y, x, bias, z, rows, row_length, alpha1, alpha2, beta1, beta2, beta3, activation);
	}

	template<typename T, int VEC>
	avStatus_t launch_activation_vec(ContextObject &ctx, void *y, const void *x, long long elements, const void *alpha, const void *beta,
			avActivationType_t activation)
	{
		using CT = typename ComputeType<T>::type;
		const CT a = getAlphaValue<CT>(alpha), b = getBetaValue<CT>(beta);
		const long long vectors = elements / VEC;
		const int grid = grid_for(ctx, vectors);
		T *yp = reinterpret_cast<T*>(y);
		const T *xp = reinterpret_cast<const T*>(x);
		switch (activation_class(activation))
		{
			case 0:
				kernel_activation<T, VEC, 0> <<<grid, 256, 0, ctx.getStream()>>>(yp, xp, vectors, a, b, activation);
				break;
			case 1:
				kernel_activation<T, VEC, 1> <<<grid, 256, 0, ctx.getStream()>>>(yp, xp, vectors, a, b, activation);
				break;
			default:
				kernel_activation<T, VEC, 2> <<<grid, 256, 0, ctx.getStream()>>>(yp, xp, vectors, a, b, activation);
				break;
		}
		return checkForErrors();
	}
	template<typename T>
	avStatus_t launch_activation(ContextObject &ctx, void *y, const void *x, long long elements, const void *alpha, const void *beta,
			avActivationType_t activation)
	{
		constexpr int kVec = 16 / static_cast<int>(sizeof(T));
		if (elements % kVec == 0 and aligned16(y) and aligned16(x))
			return launch_activation_vec<T, kVec>(ctx, y, x, elements, alpha, beta, activation);
		return launch_activation_vec<T, 1>(ctx, y, x, elements, alpha, beta, activation);
	}
}

namespace avocado
{
	namespace backend
	{
		avStatus_t cudaAddBias(avContextDescriptor_t context, const void *alpha1, const void *alpha2, const avTensorDescriptor_t xDesc,
				const avMemoryDescriptor_t xMem, const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const avTensorDescriptor_t yDesc,
				avMemoryDescriptor_t yMem, const void *beta1, const void *beta2, const void *beta3, const avMemoryDescriptor_t zMem, avActivationType_t activation)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				const TensorObject &x = getTensor(xDesc);
				const TensorObject &b = getTensor(bDesc);
				const TensorObject &y = getTensor(yDesc);
				const void *x_ptr = getPointer(xMem);
				const void *b_ptr = getPointer(bMem);
				const void *z_ptr = getPointer(zMem);
				void *y_ptr = getPointer(yMem);
				if (x_ptr == nullptr or b_ptr == nullptr or y_ptr == nullptr or x.dtype != y.dtype or x.volume() != y.volume())
					return AVOCADO_STATUS_BAD_PARAM;
				/* the bias covers the trailing dimensions of x */
				if (b.nb_dims > x.nb_dims)
					return AVOCADO_STATUS_BAD_PARAM;
				for (int i = 0; i < b.nb_dims; i++)
					if (b.dims[b.nb_dims - 1 - i] != x.dims[x.nb_dims - 1 - i])
						return AVOCADO_STATUS_BAD_PARAM;
				const long long row_length = b.volume();
				if (x.volume() == 0)
					return AVOCADO_STATUS_SUCCESS;
				if (row_length == 0 or row_length > 0x7FFFFFFFll)
					return AVOCADO_STATUS_BAD_PARAM;
				const long long rows = x.volume() / row_length;
				const avDataType_t bias_type = (x.dtype == AVOCADO_DTYPE_FLOAT64) ? AVOCADO_DTYPE_FLOAT64 : AVOCADO_DTYPE_FLOAT32;
				if (b.dtype != bias_type)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				ctx.setDevice();
				const int n = static_cast<int>(row_length);
				switch (x.dtype)
				{
					case AVOCADO_DTYPE_FLOAT16:
						return launch_add_bias<half, float>(ctx, y_ptr, x_ptr, b_ptr, z_ptr, rows, n, alpha1, alpha2, beta1, beta2, beta3, activation);
					case AVOCADO_DTYPE_BFLOAT16:
						return launch_add_bias<__nv_bfloat16, float>(ctx, y_ptr, x_ptr, b_ptr, z_ptr, rows, n, alpha1, alpha2, beta1, beta2, beta3, activation);
					case AVOCADO_DTYPE_FLOAT32:
						return launch_add_bias<float, float>(ctx, y_ptr, x_ptr, b_ptr, z_ptr, rows, n, alpha1, alpha2, beta1, beta2, beta3, activation);
					case AVOCADO_DTYPE_FLOAT64:
						return launch_add_bias<double, double>(ctx, y_ptr, x_ptr, b_ptr, z_ptr, rows, n, alpha1, alpha2, beta1, beta2, beta3, activation);
					default:
						return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				}
			AVOCADO_API_END
		}

		avStatus_t cudaActivationForward(avContextDescriptor_t context, avActivationType_t activation, const void *alpha, const avTensorDescriptor_t xDesc,
				const avMemoryDescriptor_t xMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				const TensorObject &x = getTensor(xDesc);
				const TensorObject &y = getTensor(yDesc);
				const void *x_ptr = getPointer(xMem);
				void *y_ptr = getPointer(yMem);
				if (x_ptr == nullptr or y_ptr == nullptr or x.dtype != y.dtype or x.volume() != y.volume())
					return AVOCADO_STATUS_BAD_PARAM;
				if (x.volume() == 0)
					return AVOCADO_STATUS_SUCCESS;
				ctx.setDevice();
				switch (x.dtype)
				{
					case AVOCADO_DTYPE_FLOAT16:
						return launch_activation<half>(ctx, y_ptr, x_ptr, x.volume(), alpha, beta, activation);
					case AVOCADO_DTYPE_BFLOAT16:
						return launch_activation<__nv_bfloat16>(ctx, y_ptr, x_ptr, x.volume(), alpha, beta, activation);
					case AVOCADO_DTYPE_FLOAT32:
						return launch_activation<float>(ctx, y_ptr, x_ptr, x.volume(), alpha, beta, activation);
					case AVOCADO_DTYPE_FLOAT64:
						return launch_activation<double>(ctx, y_ptr, x_ptr, x.volume(), alpha, beta, activation);
					default:
						return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				}
			AVOCADO_API_END
		}
	} /* namespace backend */
} /* namespace avocado */
