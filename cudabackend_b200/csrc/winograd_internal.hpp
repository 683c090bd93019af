/*
 * winograd_internal.hpp -- the transform and contraction launchers behind the C entry points, callable with objects
 * and raw device pointers instead of handles.  The one-call fused convolution chains them on the context's scratch
 * buffer; the entry points of winograd_nonfused.cu and gemm.cu are thin wrappers over the same functions.
 */
#ifndef B200_WINOGRAD_INTERNAL_HPP_
#define B200_WINOGRAD_INTERNAL_HPP_

#include "objects.hpp"

namespace bk
{
	avocado::backend::avStatus_t winograd_weight_transform(avocado::backend::b200::ContextObject &ctx, const avocado::backend::b200::ConvolutionObject &conv,
			int transformSize, const avocado::backend::b200::TensorObject &w, const void *wPtr, const avocado::backend::b200::TensorObject &m, void *mPtr);

	/* A weight transform (3x3 kernel) that may ride along with the launch of an input transform instead of being a
	 * kernel of its own: the first blocks of that launch compute it.  See f43::WeightJob. */
	struct WeightRide
	{
			const void *weights; /* [K, 3, 3, C] */
			void *matrices; /* [(transformSize + 2)^2, K, C] */
			int filters, channels, transformSize;
			bool invert;
			avocado::backend::avDataType_t weightType, matrixType;
	};

	/* deviceStatus: where the TMA-staged kernel reports a wait that ran out; null = the context's own status word.
	 * ride / rideTaken: a weight transform offered to this launch, and whether the launch took it (only the TMA-staged
	 * kernel can; when it did not, the caller launches the weight transform itself). */
	avocado::backend::avStatus_t winograd_input_transform(avocado::backend::b200::ContextObject &ctx, const avocado::backend::b200::ConvolutionObject &conv,
			int transformSize, const avocado::backend::b200::TensorObject &w, const avocado::backend::b200::TensorObject &x, const void *xPtr,
			const avocado::backend::b200::TensorObject &m, void *mPtr, int *deviceStatus = nullptr, const WeightRide *ride = nullptr,
			bool *rideTaken = nullptr);

	avocado::backend::avStatus_t winograd_output_transform(avocado::backend::b200::ContextObject &ctx, const avocado::backend::b200::ConvolutionObject &conv,
			int transformSize, const avocado::backend::b200::TensorObject &w, const void *alpha1, const avocado::backend::b200::TensorObject &m,
			const void *mPtr, const avocado::backend::b200::TensorObject &y, void *yPtr, const void *bPtr, const void *alpha2, const void *zPtr,
			const void *beta, avocado::backend::avActivationType_t activation);

	/* C[i] = alpha * op(A[i]) * op(B[i]) + beta * C[i] on row-major 3-D tensors */
	avocado::backend::avStatus_t gemm_batched(avocado::backend::b200::ContextObject &ctx, bool transA, bool transB, const void *alpha,
			const avocado::backend::b200::TensorObject &a, const void *aPtr, const avocado::backend::b200::TensorObject &b, const void *bPtr, const void *beta,
			const avocado::backend::b200::TensorObject &c, void *cPtr);

	/* C[i] = A[i] * B[i]^T on the tensor-core kernel only, with the kernel's error word at a caller-chosen address;
	 * returns NOT_SUPPORTED instead of falling back when the shape is outside what that kernel covers */
	avocado::backend::avStatus_t gemm_batched_nt_tensor_core(avocado::backend::b200::ContextObject &ctx, const avocado::backend::b200::TensorObject &a,
			const void *aPtr, const avocado::backend::b200::TensorObject &b, const void *bPtr, const avocado::backend::b200::TensorObject &c, void *cPtr,
			int *deviceStatus);

	/* Holds the call back instead of launching it when the context has fusion switched on and the call is the contraction
	 * of an F(4x4,3x3) pipeline that the fused contraction + output transform kernel could take over; returns whether it did. */
	bool defer_gemm_batched(avocado::backend::b200::ContextObject &ctx, bool transA, bool transB, const void *alpha,
			const avocado::backend::b200::TensorObject &a, const void *aPtr, const avocado::backend::b200::TensorObject &b, const void *bPtr, const void *beta,
			const avocado::backend::b200::TensorObject &c, void *cPtr);

	/* Launches the weight transform the context is holding back, if any (see DeferredWeightTransform in objects.hpp). */
	avocado::backend::avStatus_t flush_deferred_weights(avocado::backend::b200::ContextObject &ctx);

	/* Launches the batched GEMM the context is holding back, if any (see DeferredGemm in objects.hpp). */
	avocado::backend::avStatus_t flush_deferred_gemm(avocado::backend::b200::ContextObject &ctx);

	/* Device address of the error word inside the fixed scratch array of cudaConvolutionWinogradFusedForwardNoAlloc on
	 * this device, or null while no call of that entry point has resolved the array's address there yet. */
	int* no_alloc_status_word(int device) noexcept;
} /* namespace bk */

#endif /* B200_WINOGRAD_INTERNAL_HPP_ */
