/*
 * Avocado/backend_defs.h  --  shared type vocabulary of the Avocado backend C API.
 *
 * The reference tree includes this header (include/Avocado/cuda_backend.h:11) but does not ship it: it
 * belongs to a separate support library that is absent from the reference mount.  This file is therefore
 * written from the identifiers the reference uses (every AVOCADO_* name, av*_t type and DLL_PUBLIC that
 * appears in src/, test/ and include/).  Numeric values of the enumerators and the width of the handle
 * types are this library's own choice; a caller must be compiled against this header.
 */
#ifndef AVOCADO_BACKEND_DEFS_H_
#define AVOCADO_BACKEND_DEFS_H_

#include <stdint.h>
#ifndef __cplusplus
#include <stdbool.h>
#endif

#if defined(_WIN32)
#  define DLL_PUBLIC __declspec(dllexport)
#else
#  define DLL_PUBLIC __attribute__((visibility("default")))
#endif

#define AVOCADO_MAX_TENSOR_DIMENSIONS 8
#define AVOCADO_INVALID_DESCRIPTOR (-1)

#ifdef __cplusplus
namespace avocado
{
	namespace backend
	{
#endif
		typedef int64_t av_int64;
		typedef int32_t avDeviceIndex_t;

		/* Opaque integer handles, passed by value.  -1 is never a valid handle. */
		typedef int64_t avContextDescriptor_t;
		typedef int64_t avMemoryDescriptor_t;
		typedef int64_t avTensorDescriptor_t;
		typedef int64_t avConvolutionDescriptor_t;
		typedef int64_t avOptimizerDescriptor_t;
		typedef int64_t avDropoutDescriptor_t;
		typedef int64_t avPoolingDescriptor_t;

		typedef enum
		{
			AVOCADO_STATUS_SUCCESS = 0,
			AVOCADO_STATUS_ALLOC_FAILED,
			AVOCADO_STATUS_BAD_ALLOC,
			AVOCADO_STATUS_FREE_FAILED,
			AVOCADO_STATUS_BAD_PARAM,
			AVOCADO_STATUS_ARCH_MISMATCH,
			AVOCADO_STATUS_INTERNAL_ERROR,
			AVOCADO_STATUS_NOT_SUPPORTED,
			AVOCADO_STATUS_UNSUPPORTED_DATATYPE,
			AVOCADO_STATUS_EXECUTION_FAILED,
			AVOCADO_STATUS_INSUFFICIENT_DRIVER,
			AVOCADO_STATUS_DEVICE_TYPE_MISMATCH
		} avStatus_t;

		typedef enum
		{
			AVOCADO_DTYPE_UNKNOWN = 0,
			AVOCADO_DTYPE_UINT8,
			AVOCADO_DTYPE_INT8,
			AVOCADO_DTYPE_INT16,
			AVOCADO_DTYPE_INT32,
			AVOCADO_DTYPE_INT64,
			AVOCADO_DTYPE_FLOAT16,
			AVOCADO_DTYPE_BFLOAT16,
			AVOCADO_DTYPE_FLOAT32,
			AVOCADO_DTYPE_FLOAT64,
			AVOCADO_DTYPE_COMPLEX32,
			AVOCADO_DTYPE_COMPLEX64
		} avDataType_t;

		typedef enum
		{
			AVOCADO_ACTIVATION_LINEAR = 0,
			AVOCADO_ACTIVATION_SIGMOID,
			AVOCADO_ACTIVATION_TANH,
			AVOCADO_ACTIVATION_RELU,
			AVOCADO_ACTIVATION_SELU,
			AVOCADO_ACTIVATION_ELU,
			AVOCADO_ACTIVATION_EXPONENTIAL,
			AVOCADO_ACTIVATION_SOFTPLUS,
			AVOCADO_ACTIVATION_SOFTSIGN
		} avActivationType_t;

		typedef enum
		{
			AVOCADO_CONVOLUTION_MODE = 0, /* kernel applied as stored (deep-learning "convolution") */
			AVOCADO_CROSS_CORRELATION_MODE /* kernel rotated by 180 degrees before it is applied */
		} avConvolutionMode_t;

		typedef enum
		{
			AVOCADO_GEMM_OPERATION_N = 0,
			AVOCADO_GEMM_OPERATION_T
		} avGemmOperation_t;

		typedef enum
		{
			AVOCADO_DEVICE_NAME = 0,
			AVOCADO_DEVICE_PROCESSOR_COUNT,
			AVOCADO_DEVICE_MEMORY,
			AVOCADO_DEVICE_SUPPORTS_HALF_PRECISION,
			AVOCADO_DEVICE_SUPPORTS_BFLOAT16,
			AVOCADO_DEVICE_SUPPORTS_SINGLE_PRECISION,
			AVOCADO_DEVICE_SUPPORTS_DOUBLE_PRECISION,
			AVOCADO_DEVICE_SUPPORTS_SSE,
			AVOCADO_DEVICE_SUPPORTS_SSE2,
			AVOCADO_DEVICE_SUPPORTS_SSE3,
			AVOCADO_DEVICE_SUPPORTS_SSSE3,
			AVOCADO_DEVICE_SUPPORTS_SSE41,
			AVOCADO_DEVICE_SUPPORTS_SSE42,
			AVOCADO_DEVICE_SUPPORTS_AVX,
			AVOCADO_DEVICE_SUPPORTS_AVX2,
			AVOCADO_DEVICE_SUPPORTS_AVX512_F,
			AVOCADO_DEVICE_SUPPORTS_AVX512_VL_BW_DQ,
			AVOCADO_DEVICE_SUPPORTS_DP4A,
			AVOCADO_DEVICE_ARCH_MAJOR,
			AVOCADO_DEVICE_ARCH_MINOR,
			AVOCADO_DEVICE_SUPPORTS_TENSOR_CORES
		} avDeviceProperty_t;

		/* The enumerations below are only consumed by entry points outside the convolution path. */
		typedef enum
		{
			AVOCADO_BINARY_OP_ADD = 0,
			AVOCADO_BINARY_OP_ADD_SQUARE,
			AVOCADO_BINARY_OP_SUB,
			AVOCADO_BINARY_OP_MUL,
			AVOCADO_BINARY_OP_DIV,
			AVOCADO_BINARY_OP_MOD,
			AVOCADO_BINARY_OP_POW,
			AVOCADO_BINARY_OP_MIN,
			AVOCADO_BINARY_OP_MAX,
			AVOCADO_BINARY_OP_COMPARE_EQ,
			AVOCADO_BINARY_OP_COMPARE_NEQ,
			AVOCADO_BINARY_OP_COMPARE_GT,
			AVOCADO_BINARY_OP_COMPARE_GE,
			AVOCADO_BINARY_OP_COMPARE_LT,
			AVOCADO_BINARY_OP_COMPARE_LE,
			AVOCADO_BINARY_OP_LOGICAL_AND,
			AVOCADO_BINARY_OP_LOGICAL_OR,
			AVOCADO_BINARY_OP_LOGICAL_XOR
		} avBinaryOp_t;

		typedef enum
		{
			AVOCADO_UNARY_OP_ABS = 0,
			AVOCADO_UNARY_OP_CEIL,
			AVOCADO_UNARY_OP_COS,
			AVOCADO_UNARY_OP_EXP,
			AVOCADO_UNARY_OP_FLOOR,
			AVOCADO_UNARY_OP_LN,
			AVOCADO_UNARY_OP_NEG,
			AVOCADO_UNARY_OP_RCP,
			AVOCADO_UNARY_OP_RSQRT,
			AVOCADO_UNARY_OP_SIN,
			AVOCADO_UNARY_OP_SQUARE,
			AVOCADO_UNARY_OP_SQRT,
			AVOCADO_UNARY_OP_TAN,
			AVOCADO_UNARY_OP_LOGICAL_NOT
		} avUnaryOp_t;

		typedef enum
		{
			AVOCADO_REDUCE_ADD = 0,
			AVOCADO_REDUCE_MUL,
			AVOCADO_REDUCE_MIN,
			AVOCADO_REDUCE_MAX,
			AVOCADO_REDUCE_AMAX,
			AVOCADO_REDUCE_AVG,
			AVOCADO_REDUCE_NORM1,
			AVOCADO_REDUCE_NORM2,
			AVOCADO_REDUCE_MUL_NO_ZEROS
		} avReduceOp_t;

		typedef enum
		{
			AVOCADO_SOFTMAX_MODE_INSTANCE = 0,
			AVOCADO_SOFTMAX_MODE_CHANNEL
		} avSoftmaxMode_t;

		typedef enum
		{
			AVOCADO_MEAN_SQUARE_LOSS = 0,
			AVOCADO_CROSS_ENTROPY_LOSS,
			AVOCADO_KL_DIVERGENCE_LOSS
		} avLossType_t;

		typedef enum
		{
			AVOCADO_METRIC_CATEGORICAL_ACCURACY = 0
		} avMetricType_t;

		typedef enum
		{
			AVOCADO_OPTIMIZER_SGD = 0,
			AVOCADO_OPTIMIZER_ADAM
		} avOptimizerType_t;

#ifdef __cplusplus
	} /* namespace backend */
} /* namespace avocado */
#endif

#endif /* AVOCADO_BACKEND_DEFS_H_ */
