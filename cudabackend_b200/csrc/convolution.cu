/*
 * convolution.cu -- the one-call convolution entry points and their CUDA-core kernel.
 *
 *   cudaConvolutionImplicitGemmForward   (reference include/Avocado/cuda_backend.h:814-818; the reference body,
 *                                         src/conv2d_implicit_gemm.cu:303-352, is an unfinished kernel)
 *   cudaConvolutionWinogradFusedForward  (reference :840-844; body src/winograd_fused.cu:789-826, unfinished)
 *
 * Each entry point validates its arguments on the host, then picks a kernel: the tensor-core kernels of
 * conv_implicit_gemm_tc.cu / winograd_fused_tc.cu when the shape is one they cover, otherwise the direct
 * CUDA-core kernel below, which handles every dtype, kernel size, padding and channel count of the API.
 * Nothing runs on the CPU.
 */
#include <Avocado/cuda_backend.h>

#include "objects.hpp"
#include "conv_common.cuh"
#include "conv_kernels.hpp"

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;
	using namespace ::bk;

	/* One thread per (pixel, KPT adjacent output channels); the input pixel is read once for the KPT filters.
	 * Threads of a warp share the pixel (broadcast loads of x) and differ in the filter. */
	template<typename T, typename BT>
	__global__ void __launch_bounds__(256) kernel_conv_direct_float(ConvArgs args, typename ComputeType<T>::type alpha1,
			typename ComputeType<T>::type alpha2, typename ComputeType<T>::type beta)
	{
		using CT = typename ComputeType<T>::type;
		const long long total = static_cast<long long>(args.batch) * args.out_height * args.out_width * args.filters;
		const long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
		if (g >= total)
			return;
		const int k = static_cast<int>(g % args.filters);
		const long long pixel = g / args.filters;
		const int ow = static_cast<int>(pixel % args.out_width);
		const int oh = static_cast<int>((pixel / args.out_width) % args.out_height);
		const int n = static_cast<int>(pixel / (static_cast<long long>(args.out_width) * args.out_height));
		const T *x = reinterpret_cast<const T*>(args.x);
		const T *w = reinterpret_cast<const T*>(args.w);

		CT acc = static_cast<CT>(0);
		for (int i = 0; i < args.kernel_h; i++)
			for (int j = 0; j < args.kernel_w; j++)
			{
				const int h = args.pad_h + i + oh;
				const int v = args.pad_w + j + ow;
				if (h < 0 or h >= args.height or v < 0 or v >= args.width)
					continue;
				const int wi = args.rotate_kernel ? args.kernel_h - 1 - i : i;
				const int wj = args.rotate_kernel ? args.kernel_w - 1 - j : j;
				const T *xp = x + ((static_cast<size_t>(n) * args.height + h) * args.width + v) * args.channels;
				const T *wp = w + ((static_cast<size_t>(k) * args.kernel_h + wi) * args.kernel_w + wj) * args.channels;
				for (int c = 0; c < args.channels; c++)
					acc += static_cast<CT>(to_compute(xp[c])) * static_cast<CT>(to_compute(wp[c]));
			}
		const size_t index = static_cast<size_t>(pixel) * args.filters + k;
		CT t = alpha1 * acc;
		if (args.bias != nullptr)
			t += static_cast<CT>(reinterpret_cast<const BT*>(args.bias)[k]);
		if (args.z != nullptr)
			t += alpha2 * static_cast<CT>(to_compute(reinterpret_cast<const T*>(args.z)[index]));
		t = activation_forward(args.activation, t);
		T *y = reinterpret_cast<T*>(args.y);
		if (beta != static_cast<CT>(0))
			t += beta * static_cast<CT>(to_compute(y[index]));
		y[index] = from_compute<T>(t);
	}

	template<bool INT8_OUTPUT>
	__global__ void __launch_bounds__(256) kernel_conv_direct_int8(ConvArgs args, float alpha1, float alpha2)
	{
		const long long total = static_cast<long long>(args.batch) * args.out_height * args.out_width * args.filters;
		const long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
		if (g >= total)
			return;
		const int k = static_cast<int>(g % args.filters);
		const long long pixel = g / args.filters;
		const int ow = static_cast<int>(pixel % args.out_width);
		const int oh = static_cast<int>((pixel / args.out_width) % args.out_height);
		const int n = static_cast<int>(pixel / (static_cast<long long>(args.out_width) * args.out_height));
		const int8_t *x = reinterpret_cast<const int8_t*>(args.x);
		const int8_t *w = reinterpret_cast<const int8_t*>(args.w);

		int32_t acc = 0;
		for (int i = 0; i < args.kernel_h; i++)
			for (int j = 0; j < args.kernel_w; j++)
			{
				const int h = args.pad_h + i + oh;
				const int v = args.pad_w + j + ow;
				if (h < 0 or h >= args.height or v < 0 or v >= args.width)
					continue;
				const int wi = args.rotate_kernel ? args.kernel_h - 1 - i : i;
				const int wj = args.rotate_kernel ? args.kernel_w - 1 - j : j;
				const int8_t *xp = x + ((static_cast<size_t>(n) * args.height + h) * args.width + v) * args.channels;
				const int8_t *wp = w + ((static_cast<size_t>(k) * args.kernel_h + wi) * args.kernel_w + wj) * args.channels;
				for (int c = 0; c < args.channels; c++)
					acc += static_cast<int32_t>(xp[c]) * static_cast<int32_t>(wp[c]);
			}
		const size_t index = static_cast<size_t>(pixel) * args.filters + k;
		const int32_t t = acc + (args.bias != nullptr ? reinterpret_cast<const int32_t*>(args.bias)[k] : 0);
		if (INT8_OUTPUT)
			reinterpret_cast<int8_t*>(args.y)[index] = requantize(t, alpha1, alpha1 != 1.0f, reinterpret_cast<const float*>(args.scales), k,
					reinterpret_cast<const int8_t*>(args.z), index, alpha2, args.activation);
		else
			reinterpret_cast<int32_t*>(args.y)[index] = t;
	}

	avStatus_t launch_direct(ContextObject &ctx, const ConvArgs &args, avDataType_t xType, avDataType_t yType, const void *alpha1, const void *alpha2,
			const void *beta)
	{
		const long long total = static_cast<long long>(args.batch) * args.out_height * args.out_width * args.filters;
		if (total == 0)
			return AVOCADO_STATUS_SUCCESS;
		const unsigned int grid = static_cast<unsigned int>((total + 255) / 256);
		cudaStream_t stream = ctx.getStream();
		switch (xType)
		{
			case AVOCADO_DTYPE_INT8:
				if (yType == AVOCADO_DTYPE_INT8)
					kernel_conv_direct_int8<true> <<<grid, 256, 0, stream>>>(args, getAlphaValue<float>(alpha1), getAlphaValue<float>(alpha2));
				else
					kernel_conv_direct_int8<false> <<<grid, 256, 0, stream>>>(args, 1.0f, 1.0f);
				break;
			case AVOCADO_DTYPE_FLOAT16:
				kernel_conv_direct_float<half, float> <<<grid, 256, 0, stream>>>(args, getAlphaValue<float>(alpha1), getAlphaValue<float>(alpha2),
						getBetaValue<float>(beta));
				break;
			case AVOCADO_DTYPE_BFLOAT16:
				kernel_conv_direct_float<__nv_bfloat16, float> <<<grid, 256, 0, stream>>>(args, getAlphaValue<float>(alpha1), getAlphaValue<float>(alpha2),
						getBetaValue<float>(beta));
				break;
			case AVOCADO_DTYPE_FLOAT32:
				kernel_conv_direct_float<float, float> <<<grid, 256, 0, stream>>>(args, getAlphaValue<float>(alpha1), getAlphaValue<float>(alpha2),
						getBetaValue<float>(beta));
				break;
			case AVOCADO_DTYPE_FLOAT64:
				kernel_conv_direct_float<double, double> <<<grid, 256, 0, stream>>>(args, getAlphaValue<double>(alpha1), getAlphaValue<double>(alpha2),
						getBetaValue<double>(beta));
				break;
			default:
				return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
		}
		return checkForErrors();
	}

	/* AVOCADO_B200_CONV=direct keeps every convolution on the CUDA-core kernel (A/B comparison) */
	bool lowering_enabled()
	{
		static const bool enabled = []()
		{
			const char *env = std::getenv("AVOCADO_B200_CONV");
			return not (env != nullptr and std::strcmp(env, "direct") == 0);
		}();
		return enabled;
	}

	enum class Algorithm
	{
		ImplicitGemm, WinogradFused
	};

	avStatus_t convolution_forward(Algorithm algorithm, avContextDescriptor_t context, const avConvolutionDescriptor_t config, const void *alpha1,
			const avTensorDescriptor_t xDesc, const avMemoryDescriptor_t xMem, const avTensorDescriptor_t wDesc, const avMemoryDescriptor_t wMem,
			const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const void *alpha2, const avTensorDescriptor_t zDesc,
			const avMemoryDescriptor_t zMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem, avActivationType_t activation)
	{
		AVOCADO_API_BEGIN
			ContextObject &ctx = getContext(context);
			const ConvolutionObject &conv = getConvolution(config);
			const TensorObject &x = getTensor(xDesc);
			const TensorObject &w = getTensor(wDesc);
			const TensorObject &y = getTensor(yDesc);
			if (x.nb_dims != 4 or w.nb_dims != 4 or y.nb_dims != 4)
				return AVOCADO_STATUS_BAD_PARAM;
			if (x.dims[3] != w.dims[3] or y.dims[3] != w.dims[0] or y.dims[0] != x.dims[0])
				return AVOCADO_STATUS_BAD_PARAM;
			/* unit stride and dilation, one group, zero padding value: what the reference kernels assume
			 * (src/conv2d_implicit_gemm.cu:326, src/winograd_fused.cu:810) */
			for (int i = 0; i < 2; i++)
				if (conv.strides[i] != 1 or conv.dilation[i] != 1)
					return AVOCADO_STATUS_NOT_SUPPORTED;
			if (conv.groups != 1 or not conv.paddingValueIsZero())
				return AVOCADO_STATUS_NOT_SUPPORTED;
			if (w.dtype != x.dtype)
				return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;

			ConvArgs args;
			args.batch = x.dims[0];
			args.height = x.dims[1];
			args.width = x.dims[2];
			args.channels = x.dims[3];
			args.filters = w.dims[0];
			args.kernel_h = w.dims[1];
			args.kernel_w = w.dims[2];
			args.out_height = y.dims[1];
			args.out_width = y.dims[2];
			args.pad_h = conv.padding[0];
			args.pad_w = conv.padding[1];
			args.rotate_kernel = (conv.mode == AVOCADO_CROSS_CORRELATION_MODE);
			args.x = getPointer(xMem);
			args.w = getPointer(wMem);
			args.y = getPointer(yMem);
			args.bias = getPointer(bMem);
			args.z = getPointer(zMem);
			args.scales = nullptr;
			args.activation = activation;
			if (args.x == nullptr or args.w == nullptr or args.y == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			if (x.dtype == AVOCADO_DTYPE_INT8)
			{
				if (y.dtype != AVOCADO_DTYPE_INT8 and y.dtype != AVOCADO_DTYPE_INT32)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				if (args.bias != nullptr and getTensor(bDesc).dtype != AVOCADO_DTYPE_INT32)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				if (getBetaValue<float>(beta) != 0.0f)
					return AVOCADO_STATUS_NOT_SUPPORTED;
				if (y.dtype == AVOCADO_DTYPE_INT32 and (args.z != nullptr or getAlphaValue<float>(alpha1) != 1.0f or activation != AVOCADO_ACTIVATION_LINEAR))
					return AVOCADO_STATUS_NOT_SUPPORTED;
				if (args.z != nullptr and getTensor(zDesc).dtype != AVOCADO_DTYPE_INT8)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				if (conv.quant_scales != AVOCADO_INVALID_DESCRIPTOR)
				{
					const MemoryObject &scales = getMemory(conv.quant_scales);
					if (scales.size < static_cast<int64_t>(sizeof(float)) * args.filters)
						return AVOCADO_STATUS_BAD_PARAM;
					args.scales = scales.ptr;
				}
			}
			else
			{
				if (y.dtype != x.dtype)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				if (args.z != nullptr and getTensor(zDesc).dtype != x.dtype)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				if (args.bias != nullptr)
				{
					const avDataType_t expected = (x.dtype == AVOCADO_DTYPE_FLOAT64) ? AVOCADO_DTYPE_FLOAT64 : AVOCADO_DTYPE_FLOAT32;
					if (getTensor(bDesc).dtype != expected)
						return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				}
			}
			ctx.setDevice();

			avStatus_t status = AVOCADO_STATUS_NOT_SUPPORTED;
			if (algorithm == Algorithm::ImplicitGemm)
				status = launch_implicit_gemm_tc(ctx, args, x.dtype, y.dtype, alpha1, alpha2, beta);
			else
				status = launch_winograd_fused_tc(ctx, args, x.dtype, y.dtype, alpha1, alpha2, beta);
			if (status != AVOCADO_STATUS_NOT_SUPPORTED)
				return status;
			/* float32 has no implicit tensor-core kernel: lowering + 3xTF32 GEMM, before the CUDA-core kernel of last resort */
			if (algorithm == Algorithm::ImplicitGemm and x.dtype == AVOCADO_DTYPE_FLOAT32 and lowering_enabled())
			{
				status = launch_conv_lowered_tf32(ctx, args, alpha1, alpha2, beta);
				if (status != AVOCADO_STATUS_NOT_SUPPORTED)
					return status;
			}
			return launch_direct(ctx, args, x.dtype, y.dtype, alpha1, alpha2, beta);
		AVOCADO_API_END
	}
}

namespace avocado
{
	namespace backend
	{
		avStatus_t cudaConvolutionImplicitGemmForward(avContextDescriptor_t context, const avConvolutionDescriptor_t config, const void *alpha1,
				const avTensorDescriptor_t xDesc, const avMemoryDescriptor_t xMem, const avTensorDescriptor_t wDesc, const avMemoryDescriptor_t wMem,
				const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const void *alpha2, const avTensorDescriptor_t zDesc,
				const avMemoryDescriptor_t zMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem, avActivationType_t activation)
		{
			return convolution_forward(Algorithm::ImplicitGemm, context, config, alpha1, xDesc, xMem, wDesc, wMem, bDesc, bMem, alpha2, zDesc, zMem, beta,
					yDesc, yMem, activation);
		}
		avStatus_t cudaConvolutionWinogradFusedForward(avContextDescriptor_t context, const avConvolutionDescriptor_t config, const void *alpha1,
				const avTensorDescriptor_t xDesc, const avMemoryDescriptor_t xMem, const avTensorDescriptor_t wDesc, const avMemoryDescriptor_t wMem,
				const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const void *alpha2, const avTensorDescriptor_t zDesc,
				const avMemoryDescriptor_t zMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem, avActivationType_t activation)
		{
			return convolution_forward(Algorithm::WinogradFused, context, config, alpha1, xDesc, xMem, wDesc, wMem, bDesc, bMem, alpha2, zDesc, zMem, beta,
					yDesc, yMem, activation);
		}
	} /* namespace backend */
} /* namespace avocado */
