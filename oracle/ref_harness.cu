/*
 * ref_harness.cu -- drives the reference's own non-fused Winograd kernels.  TEST INFRASTRUCTURE ONLY.
 *
 * Linked with the reference's src/winograd_nonfused.cu, src/gemm.cpp and src/im2row.cu (compiled unmodified, see
 * build_ref.py).  It supplies the helper those files take from a translation unit that is not compiled here
 * (cuda_sm_version, src/cuda_properties.cpp:121-140) and two C entry points:
 *   ref_winograd_chain     the chain of ref app/CudaBackend.cu:401-420 (weight transform, input transform, batched GEMM,
 *                          output transform) plus the dW chain (gradient transform, GEMM(T,N), update transform) on host
 *                          buffers, returning every intermediate;
 *   ref_im2row_gemm_int8   the explicit lowering the reference's scratch test used for its int8 convolution
 *                          (ref app/CudaBackend.cu:233-240): cudaIm2Row (src/im2row.cu:83-121) followed by the
 *                          int8 -> int32 cudaGemm (src/gemm.cpp:42-57), i.e. the reference's own int32 accumulators.
 */
#include <Avocado/cuda_backend.h>
#include <Avocado/backend_descriptors.hpp>

#include <cuda_runtime_api.h>
#include <cublas_v2.h>

#include <vector>

namespace avocado
{
	namespace backend
	{
		using namespace cuda;
		int cuda_sm_version(int device) noexcept
		{
			int major = 0, minor = 0;
			cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
			cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
			return major * 10 + minor;
		}
	}
}

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::cuda;

	struct Tensor
	{
			TensorDescriptor desc;
			MemoryDescriptor mem;
			size_t bytes = 0;
			Tensor(avDataType_t dtype, std::initializer_list<int> dims, size_t elementSize)
			{
				desc.type = dtype;
				desc.rank = static_cast<int>(dims.size());
				int i = 0;
				size_t volume = 1;
				for (int d : dims)
				{
					desc.dims[i++] = d;
					volume *= static_cast<size_t>(d);
				}
				bytes = volume * elementSize;
				cudaMalloc(&mem.ptr, bytes > 0 ? bytes : 1);
				cudaMemset(mem.ptr, 0, bytes);
			}
			~Tensor()
			{
				cudaFree(mem.ptr);
			}
			avTensorDescriptor_t d()
			{
				return static_cast<avTensorDescriptor_t>(reinterpret_cast<intptr_t>(&desc));
			}
			avMemoryDescriptor_t m()
			{
				return static_cast<avMemoryDescriptor_t>(reinterpret_cast<intptr_t>(&mem));
			}
			void upload(const void *src)
			{
				if (src != nullptr)
					cudaMemcpy(mem.ptr, src, bytes, cudaMemcpyHostToDevice);
			}
			void download(void *dst)
			{
				if (dst != nullptr)
					cudaMemcpy(dst, mem.ptr, bytes, cudaMemcpyDeviceToHost);
			}
	};
}

/* dtype: an avDataType_t value (FLOAT16 or FLOAT32).  All pointers are host buffers in the tensors' dtype; outputs may
 * be null.  Returns 0 on success, otherwise 100*stage + avStatus_t of the failing call, or -1 for a CUDA error. */
extern "C" int ref_winograd_chain(int dtype, int transformSize, int kernelSize, int N, int H, int W, int C, int K, const void *x, const void *w,
		const void *bias, const void *dy, void *u, void *v, void *m, void *y, void *g, void *mw, void *dw, int relu)
{
	const avDataType_t type = static_cast<avDataType_t>(dtype);
	const size_t es = (type == AVOCADO_DTYPE_FLOAT16) ? 2 : 4;
	const int tile = transformSize + kernelSize - 1;
	const int planes = tile * tile;
	const int tiles = N * ((H + transformSize - 1) / transformSize) * ((W + transformSize - 1) / transformSize);

	cudaSetDevice(0);
	ContextDescriptor context;
	cudaStreamCreate(&context.stream);
	cublasCreate(&context.handle);
	cublasSetStream(context.handle, context.stream);
	ConvolutionDescriptor conv;
	conv.padding[0] = -(kernelSize / 2);
	conv.padding[1] = -(kernelSize / 2);
	const avContextDescriptor_t ctx = static_cast<avContextDescriptor_t>(reinterpret_cast<intptr_t>(&context));
	const avConvolutionDescriptor_t cfg = static_cast<avConvolutionDescriptor_t>(reinterpret_cast<intptr_t>(&conv));
	int result = 0;
	{
		Tensor tx(type, { N, H, W, C }, es), tw(type, { K, kernelSize, kernelSize, C }, es), ty(type, { N, H, W, K }, es);
		Tensor tb(AVOCADO_DTYPE_FLOAT32, { K }, 4), tdy(type, { N, H, W, K }, es), tdw(type, { K, kernelSize, kernelSize, C }, es);
		Tensor tu(type, { planes, K, C }, es), tv(type, { planes, tiles, C }, es), tm(type, { planes, tiles, K }, es);
		Tensor tg(type, { planes, tiles, K }, es), tmw(type, { planes, K, C }, es);
		tx.upload(x);
		tw.upload(w);
		tb.upload(bias);
		tdy.upload(dy);

		avStatus_t s = cudaWinogradWeightTransform(ctx, cfg, transformSize, tw.d(), tw.m(), tu.d(), tu.m());
		if (s != AVOCADO_STATUS_SUCCESS)
			result = 100 + s;
		if (result == 0 and (s = cudaWinogradInputTransform(ctx, cfg, transformSize, tw.d(), tx.d(), tx.m(), tv.d(), tv.m())) != AVOCADO_STATUS_SUCCESS)
			result = 200 + s;
		if (result == 0 and (s = cudaGemmBatched(ctx, AVOCADO_GEMM_OPERATION_N, AVOCADO_GEMM_OPERATION_T, nullptr, tv.d(), tv.m(), tu.d(), tu.m(), nullptr,
				tm.d(), tm.m())) != AVOCADO_STATUS_SUCCESS)
			result = 300 + s;
		Tensor none(AVOCADO_DTYPE_UNKNOWN, { }, 0);
		if (result == 0 and (s = cudaWinogradOutputTransform(ctx, cfg, transformSize, tw.d(), nullptr, tm.d(), tm.m(), ty.d(), ty.m(), tb.d(),
				bias != nullptr ? tb.m() : static_cast<avMemoryDescriptor_t>(-1), nullptr, static_cast<avTensorDescriptor_t>(-1),
				static_cast<avMemoryDescriptor_t>(-1), nullptr, relu ? AVOCADO_ACTIVATION_RELU : AVOCADO_ACTIVATION_LINEAR)) != AVOCADO_STATUS_SUCCESS)
			result = 400 + s;
		if (result == 0 and dy != nullptr and type == AVOCADO_DTYPE_FLOAT32)
		{
			if ((s = cudaWinogradGradientTransform(ctx, cfg, transformSize, tw.d(), tdy.d(), tdy.m(), tg.d(), tg.m())) != AVOCADO_STATUS_SUCCESS)
				result = 500 + s;
			if (result == 0 and (s = cudaGemmBatched(ctx, AVOCADO_GEMM_OPERATION_T, AVOCADO_GEMM_OPERATION_N, nullptr, tg.d(), tg.m(), tv.d(), tv.m(), nullptr,
					tmw.d(), tmw.m())) != AVOCADO_STATUS_SUCCESS)
				result = 600 + s;
			if (result == 0 and (s = cudaWinogradUpdateTransform(ctx, cfg, transformSize, nullptr, tmw.d(), tmw.m(), nullptr, tdw.d(), tdw.m()))
					!= AVOCADO_STATUS_SUCCESS)
				result = 700 + s;
		}
		if (cudaStreamSynchronize(context.stream) != cudaSuccess or cudaGetLastError() != cudaSuccess)
			result = (result == 0) ? -1 : result;
		if (result == 0)
		{
			tu.download(u);
			tv.download(v);
			tm.download(m);
			ty.download(y);
			tg.download(g);
			tmw.download(mw);
			tdw.download(dw);
		}
	}
	cublasDestroy(context.handle);
	cudaStreamDestroy(context.stream);
	return result;
}

/* x: int8 [N,H,W,C], w: int8 [K,3,3,C] (host).  rows (optional): int8 [N*H*W, 9*C]; acc: int32 [N*H*W, K].
 * Returns 0 on success, otherwise 100*stage + avStatus_t of the failing call, or -1 for a CUDA error. */
extern "C" int ref_im2row_gemm_int8(int N, int H, int W, int C, int K, const void *x, const void *w, void *rows, void *acc)
{
	cudaSetDevice(0);
	ContextDescriptor context;
	cudaStreamCreate(&context.stream);
	cublasCreate(&context.handle);
	cublasSetStream(context.handle, context.stream);
	ConvolutionDescriptor conv;
	conv.padding[0] = -1;
	conv.padding[1] = -1;
	const avContextDescriptor_t ctx = static_cast<avContextDescriptor_t>(reinterpret_cast<intptr_t>(&context));
	const avConvolutionDescriptor_t cfg = static_cast<avConvolutionDescriptor_t>(reinterpret_cast<intptr_t>(&conv));
	int result = 0;
	{
		Tensor tx(AVOCADO_DTYPE_INT8, { N, H, W, C }, 1), tw(AVOCADO_DTYPE_INT8, { K, 3, 3, C }, 1);
		Tensor trows(AVOCADO_DTYPE_INT8, { N * H * W, 9 * C }, 1), tw2d(AVOCADO_DTYPE_INT8, { K, 9 * C }, 1), tacc(AVOCADO_DTYPE_INT32, { N * H * W, K }, 4);
		tx.upload(x);
		tw.upload(w);
		tw2d.upload(w);
		avStatus_t s = cudaIm2Row(ctx, cfg, tw.d(), tx.d(), tx.m(), trows.d(), trows.m());
		if (s != AVOCADO_STATUS_SUCCESS)
			result = 100 + s;
		if (result == 0 and (s = cudaGemm(ctx, AVOCADO_GEMM_OPERATION_N, AVOCADO_GEMM_OPERATION_T, nullptr, trows.d(), trows.m(), tw2d.d(), tw2d.m(), nullptr,
				tacc.d(), tacc.m())) != AVOCADO_STATUS_SUCCESS)
			result = 200 + s;
		if (cudaStreamSynchronize(context.stream) != cudaSuccess or cudaGetLastError() != cudaSuccess)
			result = (result == 0) ? -1 : result;
		if (result == 0)
		{
			trows.download(rows);
			tacc.download(acc);
		}
	}
	cublasDestroy(context.handle);
	cudaStreamDestroy(context.stream);
	return result;
}
