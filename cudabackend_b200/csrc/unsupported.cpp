/*
 * unsupported.cpp -- entry points of the C API that lie outside the convolution path.
 *
 * They are exported so that a caller linked against the whole header resolves, and they do no work: each
 * returns AVOCADO_STATUS_NOT_SUPPORTED, which is what the reference returns from its own unfinished operators
 * (src/dropout.cu:24-36, src/pooling.cu:29-43, src/metrics.cu:30-35).
 */
#include <Avocado/cuda_backend.h>

namespace avocado
{
	namespace backend
	{
		avStatus_t cudaChangeType(avContextDescriptor_t, avMemoryDescriptor_t, avDataType_t, const avMemoryDescriptor_t, avDataType_t, av_int64)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaConcatTensors(avContextDescriptor_t, const avTensorDescriptor_t, avMemoryDescriptor_t, const avTensorDescriptor_t *, const avMemoryDescriptor_t *, int)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaSplitTensors(avContextDescriptor_t, const avTensorDescriptor_t *, avMemoryDescriptor_t *, const avTensorDescriptor_t, const avMemoryDescriptor_t, int)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaTranspose(avContextDescriptor_t, const avTensorDescriptor_t, avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const int *)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaScaleTensor(avContextDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaAddScalarToTensor(avContextDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaAddTensors(avContextDescriptor_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaBinaryOp(avContextDescriptor_t, avBinaryOp_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaUnaryOp(avContextDescriptor_t, avUnaryOp_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaReduceTensor(avContextDescriptor_t, avReduceOp_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaActivationBackward(avContextDescriptor_t, avActivationType_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaSoftmaxForward(avContextDescriptor_t, avSoftmaxMode_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaSoftmaxBackward(avContextDescriptor_t, avSoftmaxMode_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaAffineForward(avContextDescriptor_t, avActivationType_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaBatchNormInference(avContextDescriptor_t, avActivationType_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avMemoryDescriptor_t, const avMemoryDescriptor_t, const avMemoryDescriptor_t, double)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaBatchNormForward(avContextDescriptor_t, avActivationType_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avMemoryDescriptor_t, avMemoryDescriptor_t, avMemoryDescriptor_t, double)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaBatchNormBackward(avContextDescriptor_t, avActivationType_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t, const avTensorDescriptor_t, avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avMemoryDescriptor_t, const avMemoryDescriptor_t, const void *, const void *, avMemoryDescriptor_t, avMemoryDescriptor_t, double)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaDropoutForward(avContextDescriptor_t, const avDropoutDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avTensorDescriptor_t, avMemoryDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaDropoutBackward(avContextDescriptor_t, const avDropoutDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avTensorDescriptor_t, avMemoryDescriptor_t, const avTensorDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaPoolingForward(avContextDescriptor_t, const avPoolingDescriptor_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaPoolingBackward(avContextDescriptor_t, const avPoolingDescriptor_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaMetricFunction(avContextDescriptor_t, avMetricType_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, void *)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaLossFunction(avContextDescriptor_t, avLossType_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, void *)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaLossGradient(avContextDescriptor_t, avLossType_t, const void *, const avTensorDescriptor_t, const avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const avTensorDescriptor_t, avMemoryDescriptor_t, bool)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		avStatus_t cudaRegularizerL2(avContextDescriptor_t, const avTensorDescriptor_t, avMemoryDescriptor_t, const avTensorDescriptor_t, const avMemoryDescriptor_t, const void *, const void *, void *)
		{
			return AVOCADO_STATUS_NOT_SUPPORTED;
		}
	} /* namespace backend */
} /* namespace avocado */
