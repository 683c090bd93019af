/*
 * Avocado/cuda_backend.h  --  C ABI of the B200 convolution backend.
 *
 * Every prototype below keeps the name, argument order and argument meaning of the entry point with the same
 * name in the reference's include/Avocado/cuda_backend.h (cited per group as "ref :line"), so a caller built
 * against that header can be rebuilt against this one without source changes.  Only the convolution path
 * (Winograd transforms, batched GEMM, fused Winograd, implicit GEMM) and the descriptor plumbing it needs are
 * implemented; the remaining entry points exist for link compatibility and return
 * AVOCADO_STATUS_NOT_SUPPORTED, as the reference itself does for its unfinished operators
 * (src/dropout.cu:24-36, src/pooling.cu:29-43).
 *
 * Conventions (ref :21-52):
 *  - descriptors are integer handles passed by value; `const` on a handle says the object is not modified;
 *  - every pointer argument points to HOST memory and is read before the call returns;
 *  - alpha-like scalars default to 1 and beta-like scalars to 0 when the pointer is null; their type is
 *    float for float16 / bfloat16 / integer tensors and double for float64 tensors;
 *  - an optional tensor (bias, z) is absent when its memory handle resolves to a null device pointer
 *    (pass AVOCADO_INVALID_DESCRIPTOR);
 *  - work is enqueued on the stream of `context` and the call returns without waiting for it.
 *
 * Tensor layouts on the convolution path: activations NHWC, filters [K, kh, kw, C], transform-domain
 * matrices [tile*tile, nbTiles, channels] where tile = transformSize + kernelSize - 1 and
 * nbTiles = N * ceil(H/transformSize) * ceil(W/transformSize), tile index = (n*tilesH + th)*tilesW + tw.
 * Convolution padding is the (normally negative) coordinate of the first input element that the first output
 * element reads: "pad 1" is padding = {-1, -1}  (ref src/winograd_nonfused.cu:333-334).
 */
#ifndef AVOCADO_CUDA_BACKEND_H_
#define AVOCADO_CUDA_BACKEND_H_

#include <Avocado/backend_defs.h>

#ifdef __cplusplus
namespace avocado
{
	namespace backend
	{
		extern "C"
		{
#endif

/* ------------------------------------------------------------------------------------------------------------
 * Convolution hot path
 * ------------------------------------------------------------------------------------------------------------ */

/* U = G w G^T for every (output, input) filter pair: w[K,kh,kw,C] -> matrices[tile^2, K, C].
 * AVOCADO_CROSS_CORRELATION_MODE rotates the kernel by 180 degrees first.  Replaces ref :856-858
 * (src/winograd_nonfused.cu:881-903).  float16, bfloat16, float32, float64; 3x3 with transformSize 2 or 4,
 * 5x5 with transformSize 2; anything else returns NOT_SUPPORTED. */
DLL_PUBLIC avStatus_t cudaWinogradWeightTransform(avContextDescriptor_t context, const avConvolutionDescriptor_t config, int transformSize,
		const avTensorDescriptor_t wDesc, const avMemoryDescriptor_t wMem, const avTensorDescriptor_t matricesDesc, avMemoryDescriptor_t matricesMem);

/* V = B^T d B for every input tile and channel: x[N,H,W,C] -> matrices[tile^2, nbTiles, C]; elements outside
 * the image read the descriptor's padding value.  Replaces ref :871-873 (src/winograd_nonfused.cu:906-929).
 * The dtype switch is on wDesc, as in the reference. */
DLL_PUBLIC avStatus_t cudaWinogradInputTransform(avContextDescriptor_t context, const avConvolutionDescriptor_t config, int transformSize,
		const avTensorDescriptor_t wDesc, const avTensorDescriptor_t xDesc, const avMemoryDescriptor_t xMem, const avTensorDescriptor_t matricesDesc,
		avMemoryDescriptor_t matricesMem);

/* y = activation(alpha1 * A^T M A + b + alpha2 * z) + beta * y, clipped at the image edge:
 * matrices[tile^2, nbTiles, K] -> y[N,H,W,K].  Bias is float32 when the tensors are 16-bit.
 * Replaces ref :895-898 (src/winograd_nonfused.cu:932-959, epilogue order :407-417). */
DLL_PUBLIC avStatus_t cudaWinogradOutputTransform(avContextDescriptor_t context, const avConvolutionDescriptor_t config, int transformSize,
		const avTensorDescriptor_t wDesc, const void *alpha1, const avTensorDescriptor_t matricesDesc, const avMemoryDescriptor_t matricesMem,
		const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem, const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem,
		const void *alpha2, const avTensorDescriptor_t zDesc, const avMemoryDescriptor_t zMem, const void *beta, avActivationType_t activation);

/* dy-side transform of the weight-gradient computation: dy[N,H,W,K] -> matrices[tile^2, nbTiles, K], zero
 * past the image edge.  float32 / float64.  Replaces ref :911-913 (src/winograd_nonfused.cu:963-980). */
DLL_PUBLIC avStatus_t cudaWinogradGradientTransform(avContextDescriptor_t context, const avConvolutionDescriptor_t config, int transformSize,
		const avTensorDescriptor_t wDesc, const avTensorDescriptor_t dyDesc, const avMemoryDescriptor_t dyMem, const avTensorDescriptor_t matricesDesc,
		avMemoryDescriptor_t matricesMem);

/* dw = alpha * (transform of matrices[tile^2, K, C]) + beta * dw, dw[K,kh,kw,C].  float32 / float64.
 * Replaces ref :927-929 (src/winograd_nonfused.cu:983-1000). */
DLL_PUBLIC avStatus_t cudaWinogradUpdateTransform(avContextDescriptor_t context, const avConvolutionDescriptor_t config, int transformSize,
		const void *alpha, const avTensorDescriptor_t matricesDesc, const avMemoryDescriptor_t matricesMem, const void *beta,
		const avTensorDescriptor_t dwDesc, avMemoryDescriptor_t dwMem);

/* C[i] = alpha * op(A[i]) * op(B[i]) + beta * C[i] for row-major 3-D tensors [batch, rows, cols]; the
 * transform-domain contraction of the non-fused Winograd pipeline.  Replaces ref :460-462
 * (src/gemm.cpp:126-209). */
DLL_PUBLIC avStatus_t cudaGemmBatched(avContextDescriptor_t context, avGemmOperation_t aOp, avGemmOperation_t bOp, const void *alpha,
		const avTensorDescriptor_t aDesc, const avMemoryDescriptor_t aMem, const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem,
		const void *beta, const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem);

/* Same for row-major 2-D tensors.  Replaces ref :442-444 (src/gemm.cpp:25-124). */
DLL_PUBLIC avStatus_t cudaGemm(avContextDescriptor_t context, avGemmOperation_t aOp, avGemmOperation_t bOp, const void *alpha,
		const avTensorDescriptor_t aDesc, const avMemoryDescriptor_t aMem, const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem,
		const void *beta, const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem);

/* y = activation(alpha1 * conv(x, w) + alpha2 * z + b) + beta * y computed in one kernel with Winograd
 * F(2x2,3x3) on the tensor cores.  Replaces ref :840-844; the reference declares this entry point but ships
 * only an unfinished body under another name (src/winograd_fused.cu:789). */
DLL_PUBLIC avStatus_t cudaConvolutionWinogradFusedForward(avContextDescriptor_t context, const avConvolutionDescriptor_t config, const void *alpha1,
		const avTensorDescriptor_t xDesc, const avMemoryDescriptor_t xMem, const avTensorDescriptor_t wDesc, const avMemoryDescriptor_t wMem,
		const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const void *alpha2, const avTensorDescriptor_t zDesc,
		const avMemoryDescriptor_t zMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem,
		avActivationType_t activation);

/* Same formula computed as an implicit GEMM (im2col on the fly).  int8 x and w accumulate in int32; the
 * result is requantised to int8 when yDesc is INT8 (see cuda_backend_ext.h for the per-channel scales) or
 * stored as int32 when yDesc is INT32.  Replaces ref :814-818; the reference body is an unfinished kernel
 * under another name (src/conv2d_implicit_gemm.cu:303). */
DLL_PUBLIC avStatus_t cudaConvolutionImplicitGemmForward(avContextDescriptor_t context, const avConvolutionDescriptor_t config, const void *alpha1,
		const avTensorDescriptor_t xDesc, const avMemoryDescriptor_t xMem, const avTensorDescriptor_t wDesc, const avMemoryDescriptor_t wMem,
		const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const void *alpha2, const avTensorDescriptor_t zDesc,
		const avMemoryDescriptor_t zMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem,
		avActivationType_t activation);

/* Explicit lowering: src[N,H,W,C] -> rows[N*Ho*Wo, kh*kw*C], so that rows x w[K, kh*kw*C]^T (cudaGemm with op(B) = T)
 * is the convolution.  Tap (i, j) of output pixel (oh, ow) holds input pixel (oh + i + padding_h, ow + j + padding_w),
 * or the descriptor's padding value outside the image; AVOCADO_CROSS_CORRELATION_MODE stores the taps in the opposite
 * order.  Ho = H - 2*padding_h - (kh - 1).  Any dtype (elements are only moved); stride 1, no dilation.
 * Replaces ref :791-792 (src/im2row.cu:29-66, :85-125), with which it coincides for the "same" padding
 * (padding = -kernel/2) the reference's kernel was written for. */
DLL_PUBLIC avStatus_t cudaIm2Row(avContextDescriptor_t context, const avConvolutionDescriptor_t config, const avTensorDescriptor_t filterDesc,
		const avTensorDescriptor_t srcDesc, const avMemoryDescriptor_t srcMem, const avTensorDescriptor_t rowDesc, avMemoryDescriptor_t rowMem);

/* y = alpha1 * activation(alpha2 * x + b + beta1 * z) + beta2 * z + beta3 * y, b broadcast over the leading dimensions of
 * x; b is float32 for float16 / bfloat16 / float32 tensors and float64 for float64 ones; z is optional.  The step that
 * follows a convolution whose epilogue was not fused.  Replaces ref :380-383 (src/tensor_op.cu:199-228, :493-551). */
DLL_PUBLIC avStatus_t cudaAddBias(avContextDescriptor_t context, const void *alpha1, const void *alpha2, const avTensorDescriptor_t xDesc,
		const avMemoryDescriptor_t xMem, const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const avTensorDescriptor_t yDesc,
		avMemoryDescriptor_t yMem, const void *beta1, const void *beta2, const void *beta3, const avMemoryDescriptor_t zMem, avActivationType_t activation);

/* y = alpha * activation(x) + beta * y, in place allowed.  float16, bfloat16, float32, float64.  Replaces ref :490-491. */
DLL_PUBLIC avStatus_t cudaActivationForward(avContextDescriptor_t context, avActivationType_t activation, const void *alpha, const avTensorDescriptor_t xDesc,
		const avMemoryDescriptor_t xMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem);

/* The weight update after the gradient all-reduce of a training step: w = alpha * step(dw) + beta * w with SGD (optional
 * momentum / Nesterov; one buffer of w's size in `workspace`) or Adam (two buffers).  float32 / float64.  `dwMem` is a
 * memory handle (the reference's prototype types it as a tensor handle; both are the same integer type).  Adam's bias
 * correction uses t = steps + 1 and increments the descriptor's step count.  Replaces ref :1049-1051
 * (src/optimizers.cu:34-70, :71-160, :168-186). */
DLL_PUBLIC avStatus_t cudaOptimizerLearn(avContextDescriptor_t context, const avOptimizerDescriptor_t config, const void *alpha,
		const avTensorDescriptor_t dwDesc, const avTensorDescriptor_t dwMem, const void *beta, const avTensorDescriptor_t wDesc, avMemoryDescriptor_t wMem,
		avMemoryDescriptor_t workspace);

/* ------------------------------------------------------------------------------------------------------------
 * Descriptor and context plumbing  (ref :58-262, :743-780, :992-1034; src/descriptors.cu, src/cuda_properties.cpp)
 * ------------------------------------------------------------------------------------------------------------ */

/* Number of visible CUDA devices, 0 on any error (ref :58). */
DLL_PUBLIC int cudaGetNumberOfDevices();
/* Writes one property of device `index` into `result` (at least 256 bytes) (ref :67). */
DLL_PUBLIC avStatus_t cudaGetDeviceProperty(avDeviceIndex_t index, avDeviceProperty_t propertyName, void *result);
/* Whether memory of device `from` can be copied straight to device `to` (ref :76). */
DLL_PUBLIC avStatus_t cudaIsCopyPossible(avDeviceIndex_t from, avDeviceIndex_t to, bool *result);

/* A context owns one stream on one device (ref :93-133).  The default context of a device uses the legacy
 * stream and synchronous copies, needs no creation and cannot be destroyed. */
DLL_PUBLIC avStatus_t cudaCreateContextDescriptor(avContextDescriptor_t *result, avDeviceIndex_t deviceIndex);
DLL_PUBLIC avStatus_t cudaDestroyContextDescriptor(avContextDescriptor_t desc);
DLL_PUBLIC avContextDescriptor_t cudaGetDefaultContext(avDeviceIndex_t deviceIndex);
DLL_PUBLIC avStatus_t cudaSynchronizeWithContext(avContextDescriptor_t context);
DLL_PUBLIC avStatus_t cudaIsContextReady(avContextDescriptor_t context, bool *result);

/* Device memory blocks and non-owning views into them (ref :151-222). */
DLL_PUBLIC avStatus_t cudaCreateMemoryDescriptor(avMemoryDescriptor_t *result, avDeviceIndex_t deviceIndex, av_int64 sizeInBytes);
DLL_PUBLIC avStatus_t cudaCreateMemoryView(avMemoryDescriptor_t *result, const avMemoryDescriptor_t desc, av_int64 sizeInBytes, av_int64 offsetInBytes);
DLL_PUBLIC avStatus_t cudaDestroyMemoryDescriptor(avMemoryDescriptor_t desc);
DLL_PUBLIC avStatus_t cudaSetMemory(avContextDescriptor_t context, avMemoryDescriptor_t dst, av_int64 dstOffset, av_int64 dstSize, const void *pattern,
		av_int64 patternSize);
DLL_PUBLIC avStatus_t cudaCopyMemory(avContextDescriptor_t context, avMemoryDescriptor_t dst, av_int64 dstOffset, const avMemoryDescriptor_t src,
		av_int64 srcOffset, av_int64 count);
DLL_PUBLIC avStatus_t cudaCopyMemoryToHost(avContextDescriptor_t context, void *dst, const avMemoryDescriptor_t src, av_int64 srcOffset, av_int64 bytes);
DLL_PUBLIC avStatus_t cudaCopyMemoryFromHost(avContextDescriptor_t context, avMemoryDescriptor_t dst, av_int64 dstOffset, const void *src, av_int64 bytes);
DLL_PUBLIC avStatus_t cudaPageLock(void *ptr, av_int64 count);
DLL_PUBLIC avStatus_t cudaPageUnlock(void *ptr);

/* Tensor descriptors: dtype + up to AVOCADO_MAX_TENSOR_DIMENSIONS extents (ref :235-262). */
DLL_PUBLIC avStatus_t cudaCreateTensorDescriptor(avTensorDescriptor_t *result);
DLL_PUBLIC avStatus_t cudaDestroyTensorDescriptor(avTensorDescriptor_t desc);
DLL_PUBLIC avStatus_t cudaSetTensorDescriptor(avTensorDescriptor_t desc, avDataType_t dtype, int nbDims, const int dimensions[]);
DLL_PUBLIC avStatus_t cudaGetTensorDescriptor(avTensorDescriptor_t desc, avDataType_t *dtype, int *nbDims, int dimensions[]);

/* Convolution descriptors (ref :743-780).  `paddingValue` points to 16 bytes holding the value in the tensor dtype. */
DLL_PUBLIC avStatus_t cudaCreateConvolutionDescriptor(avConvolutionDescriptor_t *result);
DLL_PUBLIC avStatus_t cudaDestroyConvolutionDescriptor(avConvolutionDescriptor_t desc);
DLL_PUBLIC avStatus_t cudaSetConvolutionDescriptor(avConvolutionDescriptor_t desc, avConvolutionMode_t mode, int nbDims, const int padding[],
		const int strides[], const int dilation[], int groups, const void *paddingValue);
DLL_PUBLIC avStatus_t cudaGetConvolutionDescriptor(avConvolutionDescriptor_t desc, avConvolutionMode_t *mode, int *nbDims, int padding[], int strides[],
		int dilation[], int *groups, void *paddingValue);

/* Optimizer descriptors (ref :992-1034); the update itself is cudaOptimizerLearn above. */
DLL_PUBLIC avStatus_t cudaCreateOptimizerDescriptor(avOptimizerDescriptor_t *result);
DLL_PUBLIC avStatus_t cudaDestroyOptimizerDescriptor(avOptimizerDescriptor_t desc);
DLL_PUBLIC avStatus_t cudaSetOptimizerDescriptor(avOptimizerDescriptor_t desc, avOptimizerType_t type, av_int64 steps, double learningRate,
		const double coefficients[], const bool flags[]);
DLL_PUBLIC avStatus_t cudaGetOptimizerDescriptor(avOptimizerDescriptor_t desc, avOptimizerType_t *type, av_int64 *steps, double *learningRate,
		double coefficients[], bool flags[]);
DLL_PUBLIC avStatus_t cudaGetOptimizerWorkspaceSize(avOptimizerDescriptor_t desc, const avTensorDescriptor_t wDesc, av_int64 *result);

/* ------------------------------------------------------------------------------------------------------------
 * Entry points outside the convolution path: exported, return AVOCADO_STATUS_NOT_SUPPORTED
 * (ref :278-441, :470-736, :791-792, :940-1064)
 * ------------------------------------------------------------------------------------------------------------ */
DLL_PUBLIC avStatus_t cudaChangeType(avContextDescriptor_t context, avMemoryDescriptor_t dst, avDataType_t dstType, const avMemoryDescriptor_t src,
		avDataType_t srcType, av_int64 elements);
DLL_PUBLIC avStatus_t cudaConcatTensors(avContextDescriptor_t context, const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem,
		const avTensorDescriptor_t aDesc[], const avMemoryDescriptor_t aMem[], int nbTensors);
DLL_PUBLIC avStatus_t cudaSplitTensors(avContextDescriptor_t context, const avTensorDescriptor_t cDesc[], avMemoryDescriptor_t cMem[],
		const avTensorDescriptor_t aDesc, const avMemoryDescriptor_t aMem, int nbTensors);
DLL_PUBLIC avStatus_t cudaTranspose(avContextDescriptor_t context, const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem,
		const avTensorDescriptor_t aDesc, const avMemoryDescriptor_t aMem, const int newDimOrder[]);
DLL_PUBLIC avStatus_t cudaScaleTensor(avContextDescriptor_t context, const avTensorDescriptor_t aDesc, const avMemoryDescriptor_t aMem, const void *alpha,
		const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem);
DLL_PUBLIC avStatus_t cudaAddScalarToTensor(avContextDescriptor_t context, const avTensorDescriptor_t aDesc, const avMemoryDescriptor_t aMem,
		const void *scalar, const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem);
DLL_PUBLIC avStatus_t cudaAddTensors(avContextDescriptor_t context, const void *alpha, const avTensorDescriptor_t aDesc, const avMemoryDescriptor_t aMem,
		const void *beta, const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem);
DLL_PUBLIC avStatus_t cudaBinaryOp(avContextDescriptor_t context, avBinaryOp_t operation, const void *alpha1, const avTensorDescriptor_t aDesc,
		const avMemoryDescriptor_t aMem, const void *alpha2, const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const void *beta,
		const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem);
DLL_PUBLIC avStatus_t cudaUnaryOp(avContextDescriptor_t context, avUnaryOp_t operation, const void *alpha, const avTensorDescriptor_t aDesc,
		const avMemoryDescriptor_t aMem, const void *beta, const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem);
DLL_PUBLIC avStatus_t cudaReduceTensor(avContextDescriptor_t context, avReduceOp_t operation, const void *alpha, const avTensorDescriptor_t aDesc,
		const avMemoryDescriptor_t aMem, const void *beta, const avTensorDescriptor_t cDesc, avMemoryDescriptor_t cMem);
DLL_PUBLIC avStatus_t cudaActivationBackward(avContextDescriptor_t context, avActivationType_t activation, const void *alpha, const avTensorDescriptor_t yDesc,
		const avMemoryDescriptor_t yMem, const avTensorDescriptor_t dyDesc, const avMemoryDescriptor_t dyMem, const void *beta,
		const avTensorDescriptor_t dxDesc, avMemoryDescriptor_t dxMem);
DLL_PUBLIC avStatus_t cudaSoftmaxForward(avContextDescriptor_t context, avSoftmaxMode_t mode, const void *alpha, const avTensorDescriptor_t xDesc,
		const avMemoryDescriptor_t xMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem);
DLL_PUBLIC avStatus_t cudaSoftmaxBackward(avContextDescriptor_t context, avSoftmaxMode_t mode, const void *alpha, const avTensorDescriptor_t yDesc,
		const avMemoryDescriptor_t yMem, const avTensorDescriptor_t dyDesc, const avMemoryDescriptor_t dyMem, const void *beta,
		const avTensorDescriptor_t dxDesc, avMemoryDescriptor_t dxMem);
DLL_PUBLIC avStatus_t cudaAffineForward(avContextDescriptor_t context, avActivationType_t activation, const avTensorDescriptor_t wDesc,
		const avMemoryDescriptor_t wMem, const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const void *alpha,
		const avTensorDescriptor_t xDesc, const avMemoryDescriptor_t xMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem);
DLL_PUBLIC avStatus_t cudaBatchNormInference(avContextDescriptor_t context, avActivationType_t activation, const void *alpha, const avTensorDescriptor_t xDesc,
		const avMemoryDescriptor_t xMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem,
		const avTensorDescriptor_t scaleBiasMeanVarDesc, const avMemoryDescriptor_t scaleMem, const avMemoryDescriptor_t biasMem,
		const avMemoryDescriptor_t meanMem, const avMemoryDescriptor_t varianceMem, double epsilon);
DLL_PUBLIC avStatus_t cudaBatchNormForward(avContextDescriptor_t context, avActivationType_t activation, const void *alpha, const avTensorDescriptor_t xDesc,
		const avMemoryDescriptor_t xMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem,
		const avTensorDescriptor_t scaleBiasMeanVarDesc, const avMemoryDescriptor_t scaleMem, const avMemoryDescriptor_t biasMem,
		avMemoryDescriptor_t meanMem, avMemoryDescriptor_t varianceMem, double epsilon);
DLL_PUBLIC avStatus_t cudaBatchNormBackward(avContextDescriptor_t context, avActivationType_t activation, const void *alpha, const avTensorDescriptor_t xDesc,
		const avMemoryDescriptor_t xMem, const avTensorDescriptor_t yDesc, const avMemoryDescriptor_t yMem, const void *beta,
		const avTensorDescriptor_t dxDesc, avMemoryDescriptor_t dxMem, const avTensorDescriptor_t dyDesc, avMemoryDescriptor_t dyMem,
		const avTensorDescriptor_t scaleMeanVarDesc, const avMemoryDescriptor_t scaleMem, const avMemoryDescriptor_t meanMem,
		const avMemoryDescriptor_t varianceMem, const void *alpha2, const void *beta2, avMemoryDescriptor_t scaleUpdateMem,
		avMemoryDescriptor_t biasUpdateMem, double epsilon);
DLL_PUBLIC avStatus_t cudaDropoutForward(avContextDescriptor_t context, const avDropoutDescriptor_t config, const avTensorDescriptor_t xDesc,
		const avMemoryDescriptor_t xMem, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem, avMemoryDescriptor_t states);
DLL_PUBLIC avStatus_t cudaDropoutBackward(avContextDescriptor_t context, const avDropoutDescriptor_t config, const avTensorDescriptor_t dyDesc,
		const avMemoryDescriptor_t dyMem, const avTensorDescriptor_t dxDesc, avMemoryDescriptor_t dxMem, const avTensorDescriptor_t states);
DLL_PUBLIC avStatus_t cudaPoolingForward(avContextDescriptor_t context, const avPoolingDescriptor_t config, const void *alpha, const avTensorDescriptor_t xDesc,
		const avMemoryDescriptor_t xMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem);
DLL_PUBLIC avStatus_t cudaPoolingBackward(avContextDescriptor_t context, const avPoolingDescriptor_t config, const void *alpha, const avTensorDescriptor_t xDesc,
		const avMemoryDescriptor_t xMem, const avTensorDescriptor_t dyDesc, const avMemoryDescriptor_t dyMem, const void *beta,
		const avTensorDescriptor_t dxDesc, avMemoryDescriptor_t dxMem);
DLL_PUBLIC avStatus_t cudaMetricFunction(avContextDescriptor_t context, avMetricType_t metricType, const avTensorDescriptor_t outputDesc,
		const avMemoryDescriptor_t outputMem, const avTensorDescriptor_t targetDesc, const avMemoryDescriptor_t targetMem, void *result);
DLL_PUBLIC avStatus_t cudaLossFunction(avContextDescriptor_t context, avLossType_t lossType, const avTensorDescriptor_t outputDesc,
		const avMemoryDescriptor_t outputMem, const avTensorDescriptor_t targetDesc, const avMemoryDescriptor_t targetMem, void *result);
DLL_PUBLIC avStatus_t cudaLossGradient(avContextDescriptor_t context, avLossType_t lossType, const void *alpha, const avTensorDescriptor_t outputDesc,
		const avMemoryDescriptor_t outputMem, const avTensorDescriptor_t targetDesc, const avMemoryDescriptor_t targetMem, const void *beta,
		const avTensorDescriptor_t gradientDesc, avMemoryDescriptor_t gradientMem, bool isFused);
DLL_PUBLIC avStatus_t cudaRegularizerL2(avContextDescriptor_t context, const avTensorDescriptor_t gradientDesc, avMemoryDescriptor_t dwMem,
		const avTensorDescriptor_t wDesc, const avMemoryDescriptor_t wMem, const void *scale, const void *offset, void *loss);

#ifdef __cplusplus
		} /* extern "C" */
	} /* namespace backend */
} /* namespace avocado */
#endif

#endif /* AVOCADO_CUDA_BACKEND_H_ */
