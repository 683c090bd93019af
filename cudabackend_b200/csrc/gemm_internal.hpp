/*
 * gemm_internal.hpp -- the problem description shared by the contraction kernels of gemm.cu and gemm_tf32.cu.
 */
#ifndef B200_GEMM_INTERNAL_HPP_
#define B200_GEMM_INTERNAL_HPP_

#include "objects.hpp"

namespace bk
{
	/* C[i] (M x N, row-major, pitch ldc) = alpha * op(A[i]) * op(B[i]) + beta * C[i]; op(A) is M x Kc, op(B) is Kc x N;
	 * lda / ldb are the row pitches of A and B as stored, the strides separate consecutive matrices of the batch */
	struct GemmShape
	{
			int batch, M, N, Kc;
			int lda, ldb, ldc;
			long long strideA, strideB, strideC;
			bool transA, transB;
	};

	/* float32 contraction on the tensor cores (three TF32 passes over a hi/lo split of both operands).  Returns
	 * NOT_SUPPORTED, launching nothing, for shapes it does not cover. */
	avocado::backend::avStatus_t launch_gemm_tf32(avocado::backend::b200::ContextObject &ctx, const GemmShape &s, const void *A, const void *B, void *C,
			float alpha, float beta);

	/* int8 x int8^T -> int32 on the tensor cores (one matrix, op(A) = A, op(B) = B^T).  Returns NOT_SUPPORTED, launching
	 * nothing, for shapes it does not cover. */
	avocado::backend::avStatus_t launch_gemm_i8(avocado::backend::b200::ContextObject &ctx, const GemmShape &s, const void *A, const void *B, void *C);
} /* namespace bk */

#endif /* B200_GEMM_INTERNAL_HPP_ */
