/*
 * descriptors.cu -- handle pools, contexts, device memory and the descriptor entry points of the C API.
 *
 * Behavioural counterpart of the reference's src/descriptors.cu (memory :48-192, devices :194, contexts
 * :199-253, tensor :255-289, convolution :291-322, optimizer :324-368) and src/cuda_properties.cpp
 * (:40-140), plus the object model the reference takes from a support library outside its tree.
 */
#include <Avocado/cuda_backend.h>
#include <Avocado/cuda_backend_ext.h>

#include "objects.hpp"
#include "winograd_internal.hpp"

#include <algorithm>
#include <atomic>
#include <cstdio>

namespace avocado
{
	namespace backend
	{
		namespace b200
		{
			size_t dtype_size(avDataType_t dtype) noexcept
			{
				switch (dtype)
				{
					case AVOCADO_DTYPE_UINT8:
					case AVOCADO_DTYPE_INT8:
						return 1;
					case AVOCADO_DTYPE_INT16:
					case AVOCADO_DTYPE_FLOAT16:
					case AVOCADO_DTYPE_BFLOAT16:
						return 2;
					case AVOCADO_DTYPE_INT32:
					case AVOCADO_DTYPE_FLOAT32:
						return 4;
					case AVOCADO_DTYPE_INT64:
					case AVOCADO_DTYPE_FLOAT64:
					case AVOCADO_DTYPE_COMPLEX32:
						return 8;
					case AVOCADO_DTYPE_COMPLEX64:
						return 16;
					default:
						return 0;
				}
			}

			avStatus_t convertStatus(cudaError_t err) noexcept
			{
				switch (err)
				{
					case cudaSuccess:
						return AVOCADO_STATUS_SUCCESS;
					case cudaErrorMemoryAllocation:
						return AVOCADO_STATUS_ALLOC_FAILED;
					case cudaErrorInsufficientDriver:
						return AVOCADO_STATUS_INSUFFICIENT_DRIVER;
					default:
						return AVOCADO_STATUS_EXECUTION_FAILED;
				}
			}
			avStatus_t checkForErrors() noexcept
			{
				return convertStatus(cudaGetLastError());
			}

			int getNumberOfDevices() noexcept
			{
				static const int count = []()
				{
					int n = 0;
					if (cudaGetDeviceCount(&n) != cudaSuccess)
					{
						cudaGetLastError();
						n = 0;
					}
					return std::min(n, kMaxDevices);
				}();
				return count;
			}
			int cuda_sm_version(int device) noexcept
			{
				static const std::vector<int> versions = []()
				{
					std::vector<int> result;
					for (int i = 0; i < getNumberOfDevices(); i++)
					{
						int major = 0, minor = 0;
						if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) != cudaSuccess
								or cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, i) != cudaSuccess)
							result.push_back(0);
						else
							result.push_back(major * 10 + minor);
					}
					return result;
				}();
				if (device < 0 or device >= static_cast<int>(versions.size()))
					return 0;
				return versions[device];
			}

			MemoryObject::~MemoryObject()
			{
				if (owning and ptr != nullptr)
				{
					int previous = 0;
					cudaGetDevice(&previous);
					cudaSetDevice(device);
					cudaFree(ptr);
					cudaSetDevice(previous);
				}
			}

			ContextObject::ContextObject(int deviceIndex, bool isDefault) :
					device(deviceIndex), is_default(isDefault)
			{
				if (not isDefault)
				{
					if (cudaSetDevice(device) != cudaSuccess)
						throw std::runtime_error("cudaSetDevice failed");
					if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess)
						throw std::runtime_error("cudaStreamCreate failed");
				}
			}
			ContextObject::~ContextObject()
			{
				int previous = 0;
				cudaGetDevice(&previous);
				cudaSetDevice(device);
				if (stream != nullptr)
				{
					cudaStreamSynchronize(stream);
					cudaStreamDestroy(stream);
				}
				if (workspace != nullptr)
					cudaFree(workspace);
				if (device_status != nullptr)
					cudaFree(device_status);
				if (order_event != nullptr)
					cudaEventDestroy(order_event);
				cudaSetDevice(previous);
			}
			void ContextObject::setDevice() const
			{
				if (cudaSetDevice(device) != cudaSuccess)
					throw std::runtime_error("cudaSetDevice failed");
			}
			void* ContextObject::getWorkspace(size_t bytes)
			{
				std::lock_guard<std::mutex> lock(lazy_mutex);
				if (bytes > workspace_size)
				{
					setDevice();
					cudaStreamSynchronize(stream);
					if (workspace != nullptr)
						cudaFree(workspace);
					workspace = nullptr;
					workspace_size = 0;
					const size_t rounded = (bytes + 0xFFFFFu) & ~static_cast<size_t>(0xFFFFFu);
					if (cudaMalloc(&workspace, rounded) != cudaSuccess)
					{
						cudaGetLastError();
						throw std::bad_alloc();
					}
					workspace_size = rounded;
				}
				return workspace;
			}
			int* ContextObject::getDeviceStatus()
			{
				std::lock_guard<std::mutex> lock(lazy_mutex);
				if (device_status == nullptr)
				{
					setDevice();
					if (cudaMalloc(reinterpret_cast<void**>(&device_status), 256) != cudaSuccess)
					{
						cudaGetLastError();
						throw std::bad_alloc();
					}
					cudaMemset(device_status, 0, 256);
				}
				return device_status;
			}

			Pool<ContextObject>& contextPool()
			{
				static Pool<ContextObject> pool(Kind::Context);
				return pool;
			}
			Pool<MemoryObject>& memoryPool()
			{
				static Pool<MemoryObject> pool(Kind::Memory);
				return pool;
			}
			Pool<TensorObject>& tensorPool()
			{
				static Pool<TensorObject> pool(Kind::Tensor);
				return pool;
			}
			Pool<ConvolutionObject>& convolutionPool()
			{
				static Pool<ConvolutionObject> pool(Kind::Convolution);
				return pool;
			}
			Pool<OptimizerObject>& optimizerPool()
			{
				static Pool<OptimizerObject> pool(Kind::Optimizer);
				return pool;
			}

			/* default contexts live for the whole process, one per device, created on first use */
			static ContextObject& default_context(int device)
			{
				{
					static std::mutex mutex;
					static std::unique_ptr<ContextObject> contexts[kMaxDevices];
					if (device < 0 or device >= getNumberOfDevices())
						throw std::invalid_argument("invalid device of a default context");
					std::lock_guard<std::mutex> lock(mutex);
					if (contexts[device] == nullptr)
						contexts[device] = std::make_unique<ContextObject>(device, true);
					return *contexts[device];
				}
			}

			bool isDefault(avContextDescriptor_t handle) noexcept
			{
				return handle >= 0 and handle_kind(handle) == Kind::Context and handle_is_default(handle);
			}
			ContextObject& getContextKeepDeferred(avContextDescriptor_t handle)
			{
				if (isDefault(handle))
					return default_context(static_cast<int>(handle_slot(handle)));
				return contextPool().get(handle);
			}
			ContextObject& getContext(avContextDescriptor_t handle)
			{
				ContextObject &ctx = getContextKeepDeferred(handle);
				/* in the order the calls were made: a weight transform can only have been held back before a GEMM */
				if (ctx.deferred_weights.valid and bk::flush_deferred_weights(ctx) != AVOCADO_STATUS_SUCCESS)
					throw std::runtime_error("the weight transform held back on this context failed to launch");
				if (ctx.deferred.valid and bk::flush_deferred_gemm(ctx) != AVOCADO_STATUS_SUCCESS)
					throw std::runtime_error("the batched GEMM held back on this context failed to launch");
				return ctx;
			}
			static std::atomic<int> deferred_contexts { 0 };
			int deferredCount() noexcept
			{
				return deferred_contexts.load();
			}
			void noteDeferred(int delta) noexcept
			{
				deferred_contexts.fetch_add(delta);
			}
			MemoryObject& getMemory(avMemoryDescriptor_t handle)
			{
				return memoryPool().get(handle);
			}
			TensorObject& getTensor(avTensorDescriptor_t handle)
			{
				return tensorPool().get(handle);
			}
			ConvolutionObject& getConvolution(avConvolutionDescriptor_t handle)
			{
				return convolutionPool().get(handle);
			}
			OptimizerObject& getOptimizer(avOptimizerDescriptor_t handle)
			{
				return optimizerPool().get(handle);
			}

			bool is_conv(int expectedSize, const TensorObject &wDesc) noexcept
			{
				for (int i = 1; i < wDesc.nb_dims - 1; i++)
					if (wDesc.dims[i] != expectedSize)
						return false;
				return true;
			}
		} /* namespace b200 */
	} /* namespace backend */
} /* namespace avocado */

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;

	template<typename T>
	__global__ void kernel_fill_pattern(T *ptr, long long length, T value)
	{
		const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
		for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < length; i += stride)
			ptr[i] = value;
	}
	template<typename T>
	avStatus_t fill_pattern(cudaStream_t stream, void *dst, av_int64 bytes, const void *pattern)
	{
		const long long length = bytes / static_cast<av_int64>(sizeof(T));
		if (length == 0)
			return AVOCADO_STATUS_SUCCESS;
		T value;
		std::memcpy(&value, pattern, sizeof(T));
		const int block = 256;
		const int grid = static_cast<int>(std::min<long long>(148 * 8, (length + block - 1) / block));
		kernel_fill_pattern<<<grid, block, 0, stream>>>(reinterpret_cast<T*>(dst), length, value);
		return checkForErrors();
	}
}

namespace avocado
{
	namespace backend
	{
		using namespace b200;

		int cudaGetNumberOfDevices()
		{
			return getNumberOfDevices();
		}

		avStatus_t cudaGetDeviceProperty(avDeviceIndex_t index, avDeviceProperty_t propertyName, void *result)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			cudaDeviceProp prop;
			if (cudaGetDeviceProperties(&prop, index) != cudaSuccess)
			{
				cudaGetLastError();
				return AVOCADO_STATUS_INTERNAL_ERROR;
			}
			const int cc = prop.major * 10 + prop.minor;
			switch (propertyName)
			{
				case AVOCADO_DEVICE_NAME:
					std::memset(result, 0, 256);
					std::memcpy(result, prop.name, std::min<size_t>(255, sizeof(prop.name)));
					break;
				case AVOCADO_DEVICE_PROCESSOR_COUNT:
					reinterpret_cast<int32_t*>(result)[0] = prop.multiProcessorCount;
					break;
				case AVOCADO_DEVICE_MEMORY:
					reinterpret_cast<int64_t*>(result)[0] = static_cast<int64_t>(prop.totalGlobalMem);
					break;
				case AVOCADO_DEVICE_SUPPORTS_HALF_PRECISION:
					reinterpret_cast<bool*>(result)[0] = cc >= 53;
					break;
				case AVOCADO_DEVICE_SUPPORTS_BFLOAT16:
				case AVOCADO_DEVICE_SUPPORTS_SINGLE_PRECISION:
					reinterpret_cast<bool*>(result)[0] = true;
					break;
				case AVOCADO_DEVICE_SUPPORTS_DOUBLE_PRECISION:
					reinterpret_cast<bool*>(result)[0] = cc >= 13;
					break;
				case AVOCADO_DEVICE_SUPPORTS_SSE:
				case AVOCADO_DEVICE_SUPPORTS_SSE2:
				case AVOCADO_DEVICE_SUPPORTS_SSE3:
				case AVOCADO_DEVICE_SUPPORTS_SSSE3:
				case AVOCADO_DEVICE_SUPPORTS_SSE41:
				case AVOCADO_DEVICE_SUPPORTS_SSE42:
				case AVOCADO_DEVICE_SUPPORTS_AVX:
				case AVOCADO_DEVICE_SUPPORTS_AVX2:
				case AVOCADO_DEVICE_SUPPORTS_AVX512_F:
				case AVOCADO_DEVICE_SUPPORTS_AVX512_VL_BW_DQ:
					reinterpret_cast<bool*>(result)[0] = false;
					break;
				case AVOCADO_DEVICE_SUPPORTS_DP4A:
					reinterpret_cast<bool*>(result)[0] = cc >= 61;
					break;
				case AVOCADO_DEVICE_ARCH_MAJOR:
					reinterpret_cast<int32_t*>(result)[0] = prop.major;
					break;
				case AVOCADO_DEVICE_ARCH_MINOR:
					reinterpret_cast<int32_t*>(result)[0] = prop.minor;
					break;
				case AVOCADO_DEVICE_SUPPORTS_TENSOR_CORES:
					/* the reference hard-wires false (src/cuda_properties.cpp:94-96); this library drives tcgen05 on sm_100 */
					reinterpret_cast<bool*>(result)[0] = cc >= 100;
					break;
				default:
					return AVOCADO_STATUS_BAD_PARAM;
			}
			return AVOCADO_STATUS_SUCCESS;
		}

		avStatus_t cudaIsCopyPossible(avDeviceIndex_t from, avDeviceIndex_t to, bool *result)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			if (from == to)
				result[0] = true;
			else
			{
				int tmp = 0;
				if (cudaDeviceCanAccessPeer(&tmp, to, from) == cudaSuccess)
					result[0] = (tmp != 0);
				else
				{
					cudaGetLastError();
					result[0] = false;
				}
			}
			return AVOCADO_STATUS_SUCCESS;
		}

		avStatus_t cudaCreateContextDescriptor(avContextDescriptor_t *result, avDeviceIndex_t deviceIndex)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			if (deviceIndex < 0 or deviceIndex >= getNumberOfDevices())
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				result[0] = contextPool().insert(std::make_unique<ContextObject>(deviceIndex, false));
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaDestroyContextDescriptor(avContextDescriptor_t desc)
		{
			if (isDefault(desc))
				return AVOCADO_STATUS_BAD_PARAM;
			std::unique_ptr<ContextObject> object = contextPool().remove(desc);
			if (object == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			if (object->deferred_weights.valid)
				bk::flush_deferred_weights(*object); /* the caller asked for these results: they are not dropped with the context */
			if (object->deferred.valid)
				bk::flush_deferred_gemm(*object);
			object.reset();
			return AVOCADO_STATUS_SUCCESS;
		}
		avContextDescriptor_t cudaGetDefaultContext(avDeviceIndex_t deviceIndex)
		{
			if (deviceIndex >= 0 and deviceIndex < getNumberOfDevices())
				return make_handle(Kind::Context, true, 0, static_cast<uint32_t>(deviceIndex));
			return static_cast<avContextDescriptor_t>(AVOCADO_INVALID_DESCRIPTOR);
		}
		avStatus_t cudaSynchronizeWithContext(avContextDescriptor_t context)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				ctx.setDevice();
				if (cudaStreamSynchronize(ctx.getStream()) != cudaSuccess)
					return AVOCADO_STATUS_INTERNAL_ERROR;
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaIsContextReady(avContextDescriptor_t context, bool *result)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				ctx.setDevice();
				const cudaError_t status = cudaStreamQuery(ctx.getStream());
				result[0] = (status == cudaSuccess);
				if (status != cudaSuccess and status != cudaErrorNotReady)
					return convertStatus(status);
				if (status == cudaErrorNotReady)
					cudaGetLastError();
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}

		avStatus_t cudaCreateMemoryDescriptor(avMemoryDescriptor_t *result, avDeviceIndex_t deviceIndex, av_int64 sizeInBytes)
		{
			if (result == nullptr or sizeInBytes < 0)
				return AVOCADO_STATUS_BAD_PARAM;
			if (deviceIndex < 0 or deviceIndex >= getNumberOfDevices())
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				std::unique_ptr<MemoryObject> object = std::make_unique<MemoryObject>();
				object->device = deviceIndex;
				object->size = sizeInBytes;
				object->owning = true;
				if (sizeInBytes > 0)
				{
					if (cudaSetDevice(deviceIndex) != cudaSuccess)
						return AVOCADO_STATUS_BAD_PARAM;
					if (cudaMalloc(&object->ptr, static_cast<size_t>(sizeInBytes)) != cudaSuccess)
					{
						cudaGetLastError();
						object->ptr = nullptr;
						return AVOCADO_STATUS_BAD_ALLOC;
					}
				}
				result[0] = memoryPool().insert(std::move(object));
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaCreateMemoryView(avMemoryDescriptor_t *result, const avMemoryDescriptor_t desc, av_int64 sizeInBytes, av_int64 offsetInBytes)
		{
			if (result == nullptr or sizeInBytes < 0 or offsetInBytes < 0)
				return AVOCADO_STATUS_BAD_PARAM;
			if (not memoryPool().valid(desc))
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				const MemoryObject &parent = getMemory(desc);
				if (not parent.owning or offsetInBytes + sizeInBytes > parent.size)
					return AVOCADO_STATUS_BAD_PARAM;
				std::unique_ptr<MemoryObject> object = std::make_unique<MemoryObject>();
				object->device = parent.device;
				object->size = sizeInBytes;
				object->owning = false;
				object->ptr = (parent.ptr == nullptr) ? nullptr : reinterpret_cast<uint8_t*>(parent.ptr) + offsetInBytes;
				result[0] = memoryPool().insert(std::move(object));
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaDestroyMemoryDescriptor(avMemoryDescriptor_t desc)
		{
			/* a batched GEMM that some context is holding back may read or write this memory: launch it before the memory
			 * goes (freeing waits for launched work, as it does for every other kernel) */
			if (deferredCount() > 0)
				contextPool().for_each([](ContextObject &ctx)
				{
					if (ctx.deferred_weights.valid)
						bk::flush_deferred_weights(ctx);
					if (ctx.deferred.valid)
						bk::flush_deferred_gemm(ctx);
				});
			std::unique_ptr<MemoryObject> object = memoryPool().remove(desc);
			if (object == nullptr)
				return AVOCADO_STATUS_FREE_FAILED;
			object.reset();
			return AVOCADO_STATUS_SUCCESS;
		}
		avStatus_t cudaSetMemory(avContextDescriptor_t context, avMemoryDescriptor_t dst, av_int64 dstOffset, av_int64 dstSize, const void *pattern,
				av_int64 patternSize)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				MemoryObject &mem = getMemory(dst);
				if (mem.ptr == nullptr)
					return (dstSize != 0) ? AVOCADO_STATUS_BAD_PARAM : AVOCADO_STATUS_SUCCESS;
				if (dstOffset < 0 or dstSize < 0 or dstOffset + dstSize > mem.size)
					return AVOCADO_STATUS_BAD_PARAM;
				ctx.setDevice();
				uint8_t *ptr = reinterpret_cast<uint8_t*>(mem.ptr) + dstOffset;
				if (pattern == nullptr)
				{
					cudaError_t status;
					if (ctx.is_default)
						status = cudaMemset(ptr, 0, dstSize);
					else
						status = cudaMemsetAsync(ptr, 0, dstSize, ctx.getStream());
					return convertStatus(status);
				}
				if (patternSize <= 0 or dstSize % patternSize != 0 or dstOffset % patternSize != 0)
					return AVOCADO_STATUS_BAD_PARAM;
				switch (patternSize)
				{
					case 1:
						return fill_pattern<uint8_t>(ctx.getStream(), ptr, dstSize, pattern);
					case 2:
						return fill_pattern<uint16_t>(ctx.getStream(), ptr, dstSize, pattern);
					case 4:
						return fill_pattern<uint32_t>(ctx.getStream(), ptr, dstSize, pattern);
					case 8:
						return fill_pattern<uint2>(ctx.getStream(), ptr, dstSize, pattern);
					case 16:
						return fill_pattern<uint4>(ctx.getStream(), ptr, dstSize, pattern);
					default:
						return AVOCADO_STATUS_BAD_PARAM;
				}
			AVOCADO_API_END
		}
		avStatus_t cudaCopyMemoryToHost(avContextDescriptor_t context, void *dst, const avMemoryDescriptor_t src, av_int64 srcOffset, av_int64 bytes)
		{
			if (dst == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				const MemoryObject &mem = getMemory(src);
				if (srcOffset < 0 or bytes < 0 or srcOffset + bytes > mem.size)
					return AVOCADO_STATUS_BAD_PARAM;
				ctx.setDevice();
				const uint8_t *ptr = reinterpret_cast<const uint8_t*>(mem.ptr) + srcOffset;
				cudaError_t status;
				if (ctx.is_default)
					status = cudaMemcpy(dst, ptr, bytes, cudaMemcpyDeviceToHost);
				else
					status = cudaMemcpyAsync(dst, ptr, bytes, cudaMemcpyDeviceToHost, ctx.getStream());
				return convertStatus(status);
			AVOCADO_API_END
		}
		avStatus_t cudaCopyMemoryFromHost(avContextDescriptor_t context, avMemoryDescriptor_t dst, av_int64 dstOffset, const void *src, av_int64 bytes)
		{
			if (src == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				MemoryObject &mem = getMemory(dst);
				if (dstOffset < 0 or bytes < 0 or dstOffset + bytes > mem.size)
					return AVOCADO_STATUS_BAD_PARAM;
				ctx.setDevice();
				uint8_t *ptr = reinterpret_cast<uint8_t*>(mem.ptr) + dstOffset;
				cudaError_t status;
				if (ctx.is_default)
					status = cudaMemcpy(ptr, src, bytes, cudaMemcpyHostToDevice);
				else
					status = cudaMemcpyAsync(ptr, src, bytes, cudaMemcpyHostToDevice, ctx.getStream());
				return convertStatus(status);
			AVOCADO_API_END
		}
		avStatus_t cudaCopyMemory(avContextDescriptor_t context, avMemoryDescriptor_t dst, av_int64 dstOffset, const avMemoryDescriptor_t src,
				av_int64 srcOffset, av_int64 count)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				MemoryObject &d = getMemory(dst);
				const MemoryObject &s = getMemory(src);
				if (dstOffset < 0 or srcOffset < 0 or count < 0 or dstOffset + count > d.size or srcOffset + count > s.size)
					return AVOCADO_STATUS_BAD_PARAM;
				ctx.setDevice();
				uint8_t *dptr = reinterpret_cast<uint8_t*>(d.ptr) + dstOffset;
				const uint8_t *sptr = reinterpret_cast<const uint8_t*>(s.ptr) + srcOffset;
				bool direct = false;
				cudaIsCopyPossible(s.device, d.device, &direct);
				if (direct)
				{
					cudaError_t status;
					if (s.device == d.device)
					{
						if (ctx.is_default)
							status = cudaMemcpy(dptr, sptr, count, cudaMemcpyDeviceToDevice);
						else
							status = cudaMemcpyAsync(dptr, sptr, count, cudaMemcpyDeviceToDevice, ctx.getStream());
					}
					else
					{
						if (ctx.is_default)
							status = cudaMemcpyPeer(dptr, d.device, sptr, s.device, count);
						else
							status = cudaMemcpyPeerAsync(dptr, d.device, sptr, s.device, count, ctx.getStream());
					}
					return convertStatus(status);
				}
				/* no peer access: bounce through host memory, as the reference does (src/descriptors.cu:126-135).  The
				 * context's stream does not synchronise with the legacy stream the blocking copies run on, so wait for
				 * the kernels that may still be producing the source first. */
				if (not ctx.is_default and cudaStreamSynchronize(ctx.getStream()) != cudaSuccess)
					return checkForErrors();
				std::unique_ptr<uint8_t[]> buffer(new uint8_t[count]);
				cudaError_t status = cudaMemcpy(buffer.get(), sptr, count, cudaMemcpyDeviceToHost);
				if (status != cudaSuccess)
					return convertStatus(status);
				status = cudaMemcpy(dptr, buffer.get(), count, cudaMemcpyHostToDevice);
				return convertStatus(status);
			AVOCADO_API_END
		}
		avStatus_t cudaPageLock(void *ptr, av_int64 count)
		{
			if (ptr == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			return convertStatus(cudaHostRegister(ptr, count, cudaHostRegisterDefault));
		}
		avStatus_t cudaPageUnlock(void *ptr)
		{
			if (ptr == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			return convertStatus(cudaHostUnregister(ptr));
		}

		avStatus_t cudaCreateTensorDescriptor(avTensorDescriptor_t *result)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				result[0] = tensorPool().insert(std::make_unique<TensorObject>());
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaDestroyTensorDescriptor(avTensorDescriptor_t desc)
		{
			return (tensorPool().remove(desc) != nullptr) ? AVOCADO_STATUS_SUCCESS : AVOCADO_STATUS_FREE_FAILED;
		}
		avStatus_t cudaSetTensorDescriptor(avTensorDescriptor_t desc, avDataType_t dtype, int nbDims, const int dimensions[])
		{
			if (nbDims < 0 or nbDims > AVOCADO_MAX_TENSOR_DIMENSIONS)
				return AVOCADO_STATUS_BAD_PARAM;
			if (dimensions == nullptr and nbDims != 0)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				TensorObject &t = getTensor(desc);
				t.dtype = dtype;
				t.nb_dims = nbDims;
				for (int i = 0; i < AVOCADO_MAX_TENSOR_DIMENSIONS; i++)
					t.dims[i] = (i < nbDims) ? dimensions[i] : 0;
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaGetTensorDescriptor(avTensorDescriptor_t desc, avDataType_t *dtype, int *nbDims, int dimensions[])
		{
			AVOCADO_API_BEGIN
				const TensorObject &t = getTensor(desc);
				if (dtype != nullptr)
					dtype[0] = t.dtype;
				if (nbDims != nullptr)
					nbDims[0] = t.nb_dims;
				if (dimensions != nullptr)
					for (int i = 0; i < t.nb_dims; i++)
						dimensions[i] = t.dims[i];
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}

		avStatus_t cudaCreateConvolutionDescriptor(avConvolutionDescriptor_t *result)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				result[0] = convolutionPool().insert(std::make_unique<ConvolutionObject>());
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaDestroyConvolutionDescriptor(avConvolutionDescriptor_t desc)
		{
			return (convolutionPool().remove(desc) != nullptr) ? AVOCADO_STATUS_SUCCESS : AVOCADO_STATUS_FREE_FAILED;
		}
		avStatus_t cudaSetConvolutionDescriptor(avConvolutionDescriptor_t desc, avConvolutionMode_t mode, int nbDims, const int padding[], const int strides[],
				const int dilation[], int groups, const void *paddingValue)
		{
			if (nbDims < 1 or nbDims > 3)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				ConvolutionObject &c = getConvolution(desc);
				c.mode = mode;
				c.nb_dims = nbDims;
				for (int i = 0; i < 3; i++)
				{
					c.padding[i] = (padding != nullptr and i < nbDims) ? padding[i] : 0;
					c.strides[i] = (strides != nullptr and i < nbDims) ? strides[i] : 1;
					c.dilation[i] = (dilation != nullptr and i < nbDims) ? dilation[i] : 1;
				}
				c.groups = groups;
				if (paddingValue != nullptr)
					std::memcpy(c.padding_value, paddingValue, 16);
				else
					std::memset(c.padding_value, 0, 16);
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaGetConvolutionDescriptor(avConvolutionDescriptor_t desc, avConvolutionMode_t *mode, int *nbDims, int padding[], int strides[],
				int dilation[], int *groups, void *paddingValue)
		{
			AVOCADO_API_BEGIN
				const ConvolutionObject &c = getConvolution(desc);
				if (mode != nullptr)
					mode[0] = c.mode;
				if (nbDims != nullptr)
					nbDims[0] = c.nb_dims;
				for (int i = 0; i < c.nb_dims; i++)
				{
					if (padding != nullptr)
						padding[i] = c.padding[i];
					if (strides != nullptr)
						strides[i] = c.strides[i];
					if (dilation != nullptr)
						dilation[i] = c.dilation[i];
				}
				if (groups != nullptr)
					groups[0] = c.groups;
				if (paddingValue != nullptr)
					std::memcpy(paddingValue, c.padding_value, 16);
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}

		avStatus_t cudaCreateOptimizerDescriptor(avOptimizerDescriptor_t *result)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				result[0] = optimizerPool().insert(std::make_unique<OptimizerObject>());
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaDestroyOptimizerDescriptor(avOptimizerDescriptor_t desc)
		{
			return (optimizerPool().remove(desc) != nullptr) ? AVOCADO_STATUS_SUCCESS : AVOCADO_STATUS_FREE_FAILED;
		}
		avStatus_t cudaSetOptimizerDescriptor(avOptimizerDescriptor_t desc, avOptimizerType_t type, av_int64 steps, double learningRate,
				const double coefficients[], const bool flags[])
		{
			AVOCADO_API_BEGIN
				OptimizerObject &o = getOptimizer(desc);
				o.type = type;
				o.steps = steps;
				o.learning_rate = learningRate;
				for (int i = 0; i < 4; i++)
				{
					o.coef[i] = (coefficients != nullptr) ? coefficients[i] : 0.0;
					o.flags[i] = (flags != nullptr) ? flags[i] : false;
				}
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaGetOptimizerDescriptor(avOptimizerDescriptor_t desc, avOptimizerType_t *type, av_int64 *steps, double *learningRate,
				double coefficients[], bool flags[])
		{
			AVOCADO_API_BEGIN
				const OptimizerObject &o = getOptimizer(desc);
				if (type != nullptr)
					type[0] = o.type;
				if (steps != nullptr)
					steps[0] = o.steps;
				if (learningRate != nullptr)
					learningRate[0] = o.learning_rate;
				for (int i = 0; i < 4; i++)
				{
					if (coefficients != nullptr)
						coefficients[i] = o.coef[i];
					if (flags != nullptr)
						flags[i] = o.flags[i];
				}
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaGetOptimizerWorkspaceSize(avOptimizerDescriptor_t desc, const avTensorDescriptor_t wDesc, av_int64 *result)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				const OptimizerObject &o = getOptimizer(desc);
				const TensorObject &w = getTensor(wDesc);
				/* SGD keeps one momentum buffer when flags[0] is set, Adam keeps two moment buffers
				 * (ref src/optimizers.cu:70-74, :116) */
				int64_t buffers = 0;
				if (o.type == AVOCADO_OPTIMIZER_SGD)
					buffers = o.flags[0] ? 1 : 0;
				else if (o.type == AVOCADO_OPTIMIZER_ADAM)
					buffers = 2;
				result[0] = buffers * w.sizeInBytes();
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}

		/* ---- additive extension entry points (cuda_backend_ext.h) ---- */

		avStatus_t cudaGetMemoryPointer(const avMemoryDescriptor_t desc, void **result)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				result[0] = getMemory(desc).ptr;
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaGetContextStream(avContextDescriptor_t context, void **result)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				result[0] = reinterpret_cast<void*>(getContext(context).getStream());
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaSetConvolutionQuantization(avConvolutionDescriptor_t desc, const avMemoryDescriptor_t scalesMem)
		{
			AVOCADO_API_BEGIN
				ConvolutionObject &c = getConvolution(desc);
				if (scalesMem != AVOCADO_INVALID_DESCRIPTOR and not memoryPool().valid(scalesMem))
					return AVOCADO_STATUS_BAD_PARAM;
				c.quant_scales = scalesMem;
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaGetLastDeviceStatus(avContextDescriptor_t context, int *result)
		{
			if (result == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				ctx.setDevice();
				/* two words can hold a report: the context's own, and the one inside the fixed scratch array of the
				 * entry point that allocates nothing (shared by every context of the device) */
				int *words[2] = { ctx.device_status, bk::no_alloc_status_word(ctx.device) };
				if (words[0] == nullptr and words[1] == nullptr)
				{
					result[0] = 0;
					return AVOCADO_STATUS_SUCCESS;
				}
				if (cudaStreamSynchronize(ctx.getStream()) != cudaSuccess)
					return AVOCADO_STATUS_EXECUTION_FAILED;
				int combined = 0;
				for (int *word : words)
				{
					if (word == nullptr)
						continue;
					int value = 0;
					if (cudaMemcpyAsync(&value, word, sizeof(int), cudaMemcpyDeviceToHost, ctx.getStream()) != cudaSuccess
							or cudaStreamSynchronize(ctx.getStream()) != cudaSuccess)
						return AVOCADO_STATUS_EXECUTION_FAILED;
					/* cleared on the context's own stream, so the clear is ordered before the next kernel of this context */
					if (value != 0 and cudaMemsetAsync(word, 0, sizeof(int), ctx.getStream()) != cudaSuccess)
						return AVOCADO_STATUS_EXECUTION_FAILED;
					combined |= value;
				}
				result[0] = combined;
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}

		avStatus_t cudaContextSetWinogradFusion(avContextDescriptor_t context, int flags)
		{
			AVOCADO_API_BEGIN
				if (isDefault(context) or (flags & ~(AVOCADO_WINOGRAD_FUSE_WEIGHTS | AVOCADO_WINOGRAD_FUSE_OUTPUT)) != 0)
					return AVOCADO_STATUS_BAD_PARAM;
				ContextObject &ctx = getContext(context); /* launches whatever was held back under the old setting */
				ctx.fuse_weights = (flags & AVOCADO_WINOGRAD_FUSE_WEIGHTS) != 0;
				ctx.fuse_winograd = (flags & AVOCADO_WINOGRAD_FUSE_OUTPUT) != 0;
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}

		avStatus_t cudaContextWaitForContext(avContextDescriptor_t waiting, avContextDescriptor_t signalling)
		{
			AVOCADO_API_BEGIN
				ContextObject &later = getContext(waiting);
				ContextObject &earlier = getContext(signalling);
				if (&later == &earlier)
					return AVOCADO_STATUS_SUCCESS; /* a stream is ordered with itself */
				earlier.setDevice();
				if (earlier.order_event == nullptr and cudaEventCreateWithFlags(&earlier.order_event, cudaEventDisableTiming) != cudaSuccess)
					return checkForErrors();
				if (cudaEventRecord(earlier.order_event, earlier.getStream()) != cudaSuccess)
					return checkForErrors();
				later.setDevice();
				if (cudaStreamWaitEvent(later.getStream(), earlier.order_event, 0) != cudaSuccess)
					return checkForErrors();
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}

		avStatus_t cudaContextBeginCapture(avContextDescriptor_t context)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				if (ctx.is_default)
					return AVOCADO_STATUS_BAD_PARAM;
				ctx.setDevice();
				return convertStatus(cudaStreamBeginCapture(ctx.getStream(), cudaStreamCaptureModeRelaxed));
			AVOCADO_API_END
		}
		avStatus_t cudaContextEndCapture(avContextDescriptor_t context, av_int64 *graph)
		{
			if (graph == nullptr)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				ctx.setDevice();
				cudaGraph_t captured = nullptr;
				cudaError_t status = cudaStreamEndCapture(ctx.getStream(), &captured);
				if (status != cudaSuccess or captured == nullptr)
				{
					cudaGetLastError();
					return AVOCADO_STATUS_EXECUTION_FAILED;
				}
				cudaGraphExec_t executable = nullptr;
				status = cudaGraphInstantiate(&executable, captured, 0);
				cudaGraphDestroy(captured);
				if (status != cudaSuccess)
				{
					cudaGetLastError();
					return AVOCADO_STATUS_EXECUTION_FAILED;
				}
				graph[0] = static_cast<av_int64>(reinterpret_cast<intptr_t>(executable));
				return AVOCADO_STATUS_SUCCESS;
			AVOCADO_API_END
		}
		avStatus_t cudaContextLaunchGraph(avContextDescriptor_t context, av_int64 graph)
		{
			if (graph == 0)
				return AVOCADO_STATUS_BAD_PARAM;
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				ctx.setDevice();
				return convertStatus(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(static_cast<intptr_t>(graph)), ctx.getStream()));
			AVOCADO_API_END
		}
		avStatus_t cudaDestroyCapturedGraph(av_int64 graph)
		{
			if (graph == 0)
				return AVOCADO_STATUS_BAD_PARAM;
			return convertStatus(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(static_cast<intptr_t>(graph))));
		}
	} /* namespace backend */
} /* namespace avocado */
