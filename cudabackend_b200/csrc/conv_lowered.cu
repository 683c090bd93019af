/*
 * conv_lowered.cu -- float32 convolution on the tensor cores by explicit lowering, behind
 * cudaConvolutionImplicitGemmForward.
 *
 * The reference dispatches its implicit-GEMM entry point for INT8 and FLOAT32 (src/conv2d_implicit_gemm.cu:330-347).
 * The tcgen05 implicit-GEMM kernel of this library covers int8 / float16 / bfloat16, whose operands the tensor core
 * takes as they lie in memory; float32 operands need the hi / lo split of the 3xTF32 scheme, which the batched GEMM
 * kernel (gemm_tf32.cu) already does on operands it has staged in shared memory.  So float32 goes the way the
 * reference's scratch driver went for its own test of this entry point (app/CudaBackend.cu:233-240): lower, multiply,
 * finish --
 *
 *   rows[N*Ho*Wo, kh*kw*C] = im2row(x)                      kernel_im2row (im2row.cu), chunked over the batch
 *   acc[N*Ho*Wo, K]        = rows x w[K, kh*kw*C]^T         kernel_gemm_nt_tf32x3 (tcgen05, float32-level accuracy)
 *   y = activation(alpha1 * acc + b + alpha2 * z) + beta * y kernel_conv_epilogue below (skipped when it would be the identity)
 *
 * in the context's scratch buffer, one chunk of images at a time so that the row matrix stays within kChunkBytes.
 * It moves (1 + 2 * kh*kw) times the input instead of once, which is why the 16-bit and int8 types have the implicit
 * kernel; against the one-thread-per-output CUDA-core kernel it replaces for float32 it is one to two orders faster.
 */
#include "conv_kernels.hpp"
#include "gemm_internal.hpp"

#include <algorithm>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;
	using namespace bk;

	constexpr long long kChunkBytes = 1ll << 30; /* row matrix per chunk of images */

	__device__ __noinline__ float activation_slow(avActivationType_t activation, float x)
	{
		return activation_forward(activation, x);
	}

	/* y = activation(alpha1 * acc + bias[k] + alpha2 * z) + beta * y, four filters per thread; acc may alias y when beta == 0 */
	__global__ void __launch_bounds__(256) kernel_conv_epilogue(float *y, const float *acc, const float *__restrict__ bias, const float *__restrict__ z,
			long long vectors, int filters, float alpha1, float alpha2, float beta, avActivationType_t activation)
	{
		const int vectors_per_row = filters / 4;
		for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < vectors; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			const int k = static_cast<int>(i % vectors_per_row) * 4;
			const float4 a = reinterpret_cast<const float4*>(acc)[i];
			float t[4] = { alpha1 * a.x, alpha1 * a.y, alpha1 * a.z, alpha1 * a.w };
			if (bias != nullptr)
			{
				const float4 b = *reinterpret_cast<const float4*>(bias + k);
				t[0] += b.x, t[1] += b.y, t[2] += b.z, t[3] += b.w;
			}
			if (z != nullptr)
			{
				const float4 e = reinterpret_cast<const float4*>(z)[i];
				t[0] = fmaf(alpha2, e.x, t[0]), t[1] = fmaf(alpha2, e.y, t[1]), t[2] = fmaf(alpha2, e.z, t[2]), t[3] = fmaf(alpha2, e.w, t[3]);
			}
			if (activation == AVOCADO_ACTIVATION_RELU)
			{
#pragma unroll
				for (int q = 0; q < 4; q++)
					t[q] = fmaxf(t[q], 0.0f);
			}
			else if (activation != AVOCADO_ACTIVATION_LINEAR)
			{
#pragma unroll
				for (int q = 0; q < 4; q++)
					t[q] = activation_slow(activation, t[q]);
			}
			if (beta != 0.0f)
			{
				const float4 old = reinterpret_cast<const float4*>(y)[i];
				t[0] = fmaf(beta, old.x, t[0]), t[1] = fmaf(beta, old.y, t[1]), t[2] = fmaf(beta, old.z, t[2]), t[3] = fmaf(beta, old.w, t[3]);
			}
			reinterpret_cast<float4*>(y)[i] = make_float4(t[0], t[1], t[2], t[3]);
		}
	}
}

namespace bk
{
	avStatus_t launch_conv_lowered_tf32(ContextObject &ctx, const ConvArgs &args, const void *alpha1, const void *alpha2, const void *beta)
	{
		if (cuda_sm_version(ctx.device) != 100)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const long long taps = static_cast<long long>(args.kernel_h) * args.kernel_w;
		const long long depth = taps * args.channels; /* contraction length */
		const long long pixels_per_image = static_cast<long long>(args.out_height) * args.out_width;
		if (args.batch == 0 or pixels_per_image == 0 or args.filters == 0)
			return AVOCADO_STATUS_SUCCESS;
		/* what the lowering and the TF32 GEMM need: whole 16-byte pixels, filter counts in fours, aligned tensors */
		if (args.channels % 4 != 0 or args.filters % 4 != 0 or args.filters < 8 or depth < 8 or depth > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (args.out_height != args.height - 2 * args.pad_h - (args.kernel_h - 1) or args.out_width != args.width - 2 * args.pad_w - (args.kernel_w - 1))
			return AVOCADO_STATUS_NOT_SUPPORTED;
		for (const void *ptr : { args.x, args.w, static_cast<const void*>(args.y), args.z, args.bias })
			if (ptr != nullptr and reinterpret_cast<uintptr_t>(ptr) % 16 != 0)
				return AVOCADO_STATUS_NOT_SUPPORTED;
		const float a1 = getAlphaValue<float>(alpha1), a2 = getAlphaValue<float>(alpha2), b = getBetaValue<float>(beta);
		const bool identity = (a1 == 1.0f and args.bias == nullptr and args.z == nullptr and b == 0.0f and args.activation == AVOCADO_ACTIVATION_LINEAR);

		const long long row_bytes_per_image = pixels_per_image * depth * 4;
		const long long acc_bytes_per_image = pixels_per_image * args.filters * 4;
		if (row_bytes_per_image > (8ll << 30))
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const int images = static_cast<int>(std::max<long long>(1, std::min<long long>(args.batch, kChunkBytes / row_bytes_per_image)));
		if (static_cast<long long>(images) * pixels_per_image > 0x7FFFFF00ll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const bool separate_acc = (b != 0.0f); /* the old y is still needed: the products go to scratch first */
		const size_t rows_bytes = static_cast<size_t>(images) * row_bytes_per_image;
		const size_t acc_bytes = separate_acc ? static_cast<size_t>(images) * acc_bytes_per_image : 0;
		uint8_t *scratch = reinterpret_cast<uint8_t*>(ctx.getWorkspace(rows_bytes + acc_bytes + 256));
		float *rows = reinterpret_cast<float*>(scratch);
		float *acc_scratch = reinterpret_cast<float*>(scratch + ((rows_bytes + 255) / 256) * 256);
		ctx.setDevice();
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);

		for (int first = 0; first < args.batch; first += images)
		{
			const int count = std::min(images, args.batch - first);
			const float *x = reinterpret_cast<const float*>(args.x) + static_cast<size_t>(first) * args.height * args.width * args.channels;
			float *y = reinterpret_cast<float*>(args.y) + static_cast<size_t>(first) * pixels_per_image * args.filters;
			const float *z = (args.z == nullptr) ? nullptr : reinterpret_cast<const float*>(args.z) + static_cast<size_t>(first) * pixels_per_image * args.filters;
			avStatus_t status = im2row_words(ctx, x, rows, count, args.height, args.width, args.out_height, args.out_width, args.kernel_h, args.kernel_w,
					args.pad_h, args.pad_w, args.rotate_kernel, args.channels * 4);
			if (status != AVOCADO_STATUS_SUCCESS)
				return status;
			GemmShape s;
			s.batch = 1;
			s.transA = false;
			s.transB = true;
			s.M = static_cast<int>(count * pixels_per_image);
			s.N = args.filters;
			s.Kc = static_cast<int>(depth);
			s.lda = s.Kc;
			s.ldb = s.Kc;
			s.ldc = s.N;
			s.strideA = static_cast<long long>(s.M) * s.Kc;
			s.strideB = static_cast<long long>(s.N) * s.Kc;
			s.strideC = static_cast<long long>(s.M) * s.N;
			float *acc = separate_acc ? acc_scratch : y;
			status = launch_gemm_tf32(ctx, s, rows, args.w, acc, 1.0f, 0.0f);
			if (status != AVOCADO_STATUS_SUCCESS)
				return status; /* NOT_SUPPORTED can only come before the first launch: the shape test does not depend on the chunk */
			if (not identity)
			{
				const long long vectors = static_cast<long long>(s.M) * (args.filters / 4);
				const int grid = static_cast<int>(std::min<long long>((vectors + 255) / 256, static_cast<long long>(sms) * 8));
				kernel_conv_epilogue<<<grid, 256, 0, ctx.getStream()>>>(y, acc, reinterpret_cast<const float*>(args.bias), z, vectors, args.filters, a1, a2, b,
						args.activation);
				status = checkForErrors();
				if (status != AVOCADO_STATUS_SUCCESS)
					return status;
			}
		}
		return AVOCADO_STATUS_SUCCESS;
	}
} /* namespace bk */
