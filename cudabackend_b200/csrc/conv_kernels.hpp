/*
 * conv_kernels.hpp -- launchers of the tensor-core convolution kernels.
 *
 * Each returns AVOCADO_STATUS_NOT_SUPPORTED, without launching anything, when the shape, dtype or alignment is
 * outside what the kernel covers; the caller then uses the direct CUDA-core kernel.
 */
#ifndef B200_CONV_KERNELS_HPP_
#define B200_CONV_KERNELS_HPP_

#include "objects.hpp"
#include "conv_common.cuh"

namespace bk
{
	/* implicit-GEMM convolution on tcgen05 (int8 with int32 accumulation; float16 / bfloat16 with float32 accumulation) */
	avocado::backend::avStatus_t launch_implicit_gemm_tc(avocado::backend::b200::ContextObject &ctx, const ConvArgs &args,
			avocado::backend::avDataType_t xType, avocado::backend::avDataType_t yType, const void *alpha1, const void *alpha2, const void *beta);

	/* fused Winograd F(2x2,3x3) forward on tcgen05 */
	avocado::backend::avStatus_t launch_winograd_fused_tc(avocado::backend::b200::ContextObject &ctx, const ConvArgs &args,
			avocado::backend::avDataType_t xType, avocado::backend::avDataType_t yType, const void *alpha1, const void *alpha2, const void *beta);

	/* Contraction + output transform of the F(2x2,3x3) convolution in one kernel: reads V[16][tiles][C] and U[16][K][C]
	 * (float16), writes y (float16 / bfloat16) with the bias / z / activation / beta epilogue of args.  deviceStatus is
	 * the word that receives the bit of a wait that ran out. */
	/* whether the kernel below takes this problem (device, dtype, extents and the alignment of y, z and bias), given
	 * transform-domain tensors that are 128-byte aligned */
	bool winograd_f23_contract_output_covers(const avocado::backend::b200::ContextObject &ctx, const ConvArgs &args,
			avocado::backend::avDataType_t yType, long long tiles);
	avocado::backend::avStatus_t winograd_f23_contract_output(avocado::backend::b200::ContextObject &ctx, const ConvArgs &args,
			avocado::backend::avDataType_t yType, long long tiles, const void *vPtr, const void *uPtr, const void *alpha1, const void *alpha2, const void *beta,
			int *deviceStatus);

	/* Contraction + output transform of the non-fused F(4x4,3x3) pipeline in one kernel: reads V[36][tiles][C] and
	 * U[36][K][C] (both float16 or both bfloat16), writes y[N][H][W][K] (float16 / bfloat16) with the bias / z / activation /
	 * beta epilogue of cudaWinogradOutputTransform.  Returns NOT_SUPPORTED, launching nothing, outside what it covers. */
	avocado::backend::avStatus_t winograd_f43_contract_output(avocado::backend::b200::ContextObject &ctx, const avocado::backend::b200::TensorObject &v,
			const void *vPtr, const avocado::backend::b200::TensorObject &u, const void *uPtr, const avocado::backend::b200::TensorObject &y, void *yPtr,
			const void *biasPtr, const void *zPtr, const void *alpha1, const void *alpha2, const void *beta,
			avocado::backend::avActivationType_t activation, int *deviceStatus);

	/* float32 convolution by explicit lowering onto the 3xTF32 tensor-core GEMM (conv_lowered.cu) */
	avocado::backend::avStatus_t launch_conv_lowered_tf32(avocado::backend::b200::ContextObject &ctx, const ConvArgs &args, const void *alpha1,
			const void *alpha2, const void *beta);

	/* rows[N*Ho*Wo, kh*kw*pixelBytes] of the explicit lowering for raw device pointers (im2row.cu); pixelBytes = C * element size,
	 * zero padding value */
	avocado::backend::avStatus_t im2row_words(avocado::backend::b200::ContextObject &ctx, const void *input, void *rows, int batch, int height, int width,
			int outHeight, int outWidth, int kernelH, int kernelW, int padH, int padW, bool rotate, long long pixelBytes);
} /* namespace bk */

#endif /* B200_CONV_KERNELS_HPP_ */
