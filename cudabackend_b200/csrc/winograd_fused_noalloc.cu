/*
 * winograd_fused_noalloc.cu -- cudaConvolutionWinogradFusedForwardNoAlloc: the one-call Winograd convolution for
 * callers that must not trigger a device allocation.
 *
 * Who needs this.  cudaConvolutionWinogradFusedForward keeps its transform-domain tensors in a scratch buffer that
 * the context allocates with cudaMalloc the first time (and every time a larger layer arrives).  Some hosts cannot
 * tolerate that: an inference server that has handed the whole GPU to its own memory pool has nothing left for
 * cudaMalloc to return; a latency-bound control loop cannot absorb the device-wide synchronisation an allocation
 * implies; a process running under a "no allocation after start-up" policy is simply not allowed to.  For them the
 * scratch lives in the library image itself: a file-scope __device__ array, part of the library's device code on
 * every GPU that uses it for as long as the process lives, and limited to AVOCADO_NO_ALLOC_SCRATCH_BYTES.
 *
 * What it computes: exactly what cudaConvolutionWinogradFusedForward computes for float16 and bfloat16 tensors with a
 * 3x3 kernel (same kernels, same order, bit-identical result), as long as the transform-domain tensors fit:
 *     32 * (K*C + tiles*C) bytes <= AVOCADO_NO_ALLOC_SCRATCH_BYTES,   tiles = N * ceil(H/2) * ceil(W/2)
 * (each term rounded up to 256 bytes).  When y, z or the bias is not aligned to 16 / 16 / 4 bytes the single-kernel
 * contraction + output transform does not apply and the products M are written out as well, which adds 32 * tiles*K
 * bytes to the sum.  A problem that does not fit is refused with AVOCADO_STATUS_BAD_PARAM before anything is
 * launched.  Where the allocating entry point would fall back to CUDA-core kernels (C or K not a multiple of 8) this
 * one returns AVOCADO_STATUS_NOT_SUPPORTED: those kernels are outside the no-allocation guarantee.
 *
 * Rules for the caller:
 *  - The first call on each device looks up the device address of the array (cudaGetSymbolAddress with that device
 *    current) and sets the kernels' shared-memory attributes.  The CUDA runtime loads device code lazily, so this
 *    first call is also the moment the driver places the array (and the kernels) in device memory, and it
 *    synchronises.  Make it during start-up: before the host's own pool takes the remaining memory and before any
 *    stream capture.  (CUDA_MODULE_LOADING=EAGER moves the loading to library load time instead.)
 *  - All calls on a device share the one array, whatever context they use.  Two calls whose work overlaps on the
 *    GPU (different streams, no ordering between them) race on it; order them or use the allocating entry point.
 *  - The array keeps the previous call's contents.  Nothing needs to start from zero except the 256-byte word in
 *    which the tensor-core kernels report a wait that ran out.  That word starts as zero (static initialisation),
 *    is only ever OR-ed into by kernels, and is read and cleared by cudaGetLastDeviceStatus of any context on the
 *    device -- a report is therefore kept until somebody reads it.
 *  - No cudaMalloc, cudaFree or allocating library routine is called on this path.
 */
#include <Avocado/cuda_backend.h>
#include <Avocado/cuda_backend_ext.h>

#include "objects.hpp"
#include "winograd_internal.hpp"
#include "conv_kernels.hpp"

#include <mutex>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;

	constexpr size_t kStatusBytes = 256;
	constexpr size_t kScratchBytes = AVOCADO_NO_ALLOC_SCRATCH_BYTES;

	/* [0, 256): error word of the tensor-core kernel; [256, 256 + kScratchBytes): U, V and M.
	 * In host code this name is only a stand-in for the symbol, never a device address. */
	static __device__ __align__(256) unsigned char no_alloc_scratch[kStatusBytes + kScratchBytes];

	std::mutex address_mutex;
	unsigned char *address[kMaxDevices] = { };

	/* device address of the array, looked up once per device with that device current */
	avStatus_t scratch_address(int device, unsigned char **result)
	{
		if (device < 0 or device >= kMaxDevices)
			return AVOCADO_STATUS_BAD_PARAM;
		std::lock_guard<std::mutex> lock(address_mutex);
		if (address[device] == nullptr)
		{
			if (cudaSetDevice(device) != cudaSuccess)
				return AVOCADO_STATUS_EXECUTION_FAILED;
			unsigned char *ptr = nullptr;
			const cudaError_t status = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), no_alloc_scratch);
			if (status != cudaSuccess or ptr == nullptr)
			{
				cudaGetLastError();
				return AVOCADO_STATUS_EXECUTION_FAILED;
			}
			address[device] = ptr;
		}
		result[0] = address[device];
		return AVOCADO_STATUS_SUCCESS;
	}

	size_t align_up(size_t value, size_t alignment)
	{
		return (value + alignment - 1) / alignment * alignment;
	}
	TensorObject make_tensor(avDataType_t dtype, std::initializer_list<int> dims)
	{
		TensorObject t;
		t.dtype = dtype;
		t.nb_dims = static_cast<int>(dims.size());
		int i = 0;
		for (int d : dims)
			t.dims[i++] = d;
		return t;
	}
}

namespace bk
{
	int* no_alloc_status_word(int device) noexcept
	{
		if (device < 0 or device >= kMaxDevices)
			return nullptr;
		std::lock_guard<std::mutex> lock(address_mutex);
		return reinterpret_cast<int*>(address[device]);
	}
} /* namespace bk */

namespace avocado
{
	namespace backend
	{
		avStatus_t cudaConvolutionWinogradFusedForwardNoAlloc(avContextDescriptor_t context, const avConvolutionDescriptor_t config, const void *alpha1,
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
				const void *xPtr = getPointer(xMem);
				const void *wPtr = getPointer(wMem);
				void *yPtr = getPointer(yMem);
				const void *bPtr = getPointer(bMem);
				const void *zPtr = getPointer(zMem);
				if (x.nb_dims != 4 or w.nb_dims != 4 or y.nb_dims != 4 or xPtr == nullptr or wPtr == nullptr or yPtr == nullptr)
					return AVOCADO_STATUS_BAD_PARAM;
				if (x.dims[3] != w.dims[3] or y.dims[3] != w.dims[0] or y.dims[0] != x.dims[0] or y.dims[1] != x.dims[1] or y.dims[2] != x.dims[2])
					return AVOCADO_STATUS_BAD_PARAM;
				if (x.dtype != AVOCADO_DTYPE_FLOAT16 and x.dtype != AVOCADO_DTYPE_BFLOAT16)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				if (w.dtype != x.dtype or y.dtype != x.dtype or (zPtr != nullptr and getTensor(zDesc).dtype != x.dtype)
						or (bPtr != nullptr and getTensor(bDesc).dtype != AVOCADO_DTYPE_FLOAT32))
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				if (w.dims[1] != 3 or w.dims[2] != 3 or conv.strides[0] != 1 or conv.strides[1] != 1 or conv.dilation[0] != 1 or conv.dilation[1] != 1
						or conv.groups != 1 or not conv.paddingValueIsZero())
					return AVOCADO_STATUS_NOT_SUPPORTED;

				const int batch = x.dims[0], height = x.dims[1], width = x.dims[2], channels = x.dims[3], filters = w.dims[0];
				const long long tiles = static_cast<long long>(batch) * ((height + 1) / 2) * ((width + 1) / 2);
				if (tiles == 0 or channels == 0 or filters == 0)
					return AVOCADO_STATUS_SUCCESS;
				constexpr int planes = 16;
				bk::ConvArgs args = { };
				args.batch = batch, args.height = height, args.width = width, args.channels = channels, args.filters = filters;
				args.out_height = height, args.out_width = width;
				args.y = yPtr, args.bias = bPtr, args.z = zPtr, args.activation = activation;
				/* the single-kernel contraction + output transform keeps M in TMEM; only the two-kernel form needs room for it */
				const bool single_kernel = bk::winograd_f23_contract_output_covers(ctx, args, y.dtype, tiles);
				if (not single_kernel and (channels % 8 != 0 or filters % 8 != 0))
					return AVOCADO_STATUS_NOT_SUPPORTED;
				const size_t u_bytes = align_up(static_cast<size_t>(planes) * filters * channels * 2, 256);
				const size_t v_bytes = align_up(static_cast<size_t>(planes) * tiles * channels * 2, 256);
				const size_t m_bytes = single_kernel ? 0 : align_up(static_cast<size_t>(planes) * tiles * filters * 2, 256);
				/* the fixed array is all there is: a problem that does not fit is refused, never trimmed */
				if (tiles > 0x7FFFFF00ll or u_bytes + v_bytes + m_bytes > kScratchBytes)
					return AVOCADO_STATUS_BAD_PARAM;

				unsigned char *base = nullptr;
				const avStatus_t lookup = scratch_address(ctx.device, &base);
				if (lookup != AVOCADO_STATUS_SUCCESS)
					return lookup;
				ctx.setDevice();
				int *status_word = reinterpret_cast<int*>(base);
				void *u_ptr = base + kStatusBytes;
				void *v_ptr = base + kStatusBytes + u_bytes;
				void *m_ptr = base + kStatusBytes + u_bytes + v_bytes;

				const avDataType_t domain = AVOCADO_DTYPE_FLOAT16;
				const TensorObject u = make_tensor(domain, { planes, filters, channels });
				const TensorObject v = make_tensor(domain, { planes, static_cast<int>(tiles), channels });
				const TensorObject m = make_tensor(domain, { planes, static_cast<int>(tiles), filters });

				bk::WeightRide ride = { wPtr, u_ptr, filters, channels, 2, conv.mode == AVOCADO_CROSS_CORRELATION_MODE, w.dtype, domain };
				bool ride_taken = false;
				avStatus_t status = bk::winograd_input_transform(ctx, conv, 2, w, x, xPtr, v, v_ptr, status_word, &ride, &ride_taken);
				if (status != AVOCADO_STATUS_SUCCESS)
					return status;
				if (not ride_taken)
				{
					status = bk::winograd_weight_transform(ctx, conv, 2, w, wPtr, u, u_ptr);
					if (status != AVOCADO_STATUS_SUCCESS)
						return status;
				}
				if (single_kernel)
					/* the same single-kernel contraction + output transform the allocating entry point uses */
					return bk::winograd_f23_contract_output(ctx, args, y.dtype, tiles, v_ptr, u_ptr, alpha1, alpha2, beta, status_word);
				status = bk::gemm_batched_nt_tensor_core(ctx, v, v_ptr, u, u_ptr, m, m_ptr, status_word);
				if (status != AVOCADO_STATUS_SUCCESS)
					return status;
				return bk::winograd_output_transform(ctx, conv, 2, w, alpha1, m, m_ptr, y, yPtr, bPtr, alpha2, zPtr, beta, activation);
			AVOCADO_API_END
		}
	} /* namespace backend */
} /* namespace avocado */
