/*
 * objects.hpp -- the objects behind the integer handles of the C API and the pools that own them.
 *
 * The reference keeps these classes (ContextDescriptor, MemoryDescriptor, TensorDescriptor,
 * ConvolutionDescriptor, OptimizerDescriptor, create_descriptor/destroy_descriptor, getContext/getTensor/...)
 * in a support library that is not part of its tree; their behaviour is known only from the call sites in
 * src/descriptors.cu, src/gemm.cpp:131-144 and src/winograd_nonfused.cu:612-669.  This is an independent
 * implementation of that behaviour.
 *
 * Handle layout (64 bit): [63:56] object kind, [55] default-context flag, [54:32] generation, [31:0] slot.
 * A destroyed slot bumps its generation, so a stale handle is rejected instead of aliasing a new object.
 */
#ifndef B200_OBJECTS_HPP_
#define B200_OBJECTS_HPP_

#include <Avocado/backend_defs.h>

#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstring>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <vector>

namespace avocado
{
	namespace backend
	{
		namespace b200
		{
			enum class Kind : uint8_t
			{
				Context = 1, Memory = 2, Tensor = 3, Convolution = 4, Optimizer = 5
			};

			constexpr int kMaxDevices = 64;

			/* One-time set-up per device (kernel attributes and the like) that several host threads may reach at the
			 * same moment: the first caller on a device runs `configure`, the others wait for it and see its result. */
			class PerDeviceOnce
			{
					std::once_flag m_flags[kMaxDevices];
					cudaError_t m_results[kMaxDevices] = { };
				public:
					template<class F>
					cudaError_t run(int device, F &&configure)
					{
						if (device < 0 or device >= kMaxDevices)
							return cudaErrorInvalidDevice;
						std::call_once(m_flags[device], [&]()
						{	m_results[device] = configure();});
						return m_results[device];
					}
			};

			inline int64_t make_handle(Kind kind, bool isDefault, uint32_t generation, uint32_t slot) noexcept
			{
				return (static_cast<int64_t>(kind) << 56) | (static_cast<int64_t>(isDefault ? 1 : 0) << 55)
						| (static_cast<int64_t>(generation & 0x7FFFFFu) << 32) | static_cast<int64_t>(slot);
			}
			inline Kind handle_kind(int64_t h) noexcept
			{
				return static_cast<Kind>((static_cast<uint64_t>(h) >> 56) & 0xFFu);
			}
			inline bool handle_is_default(int64_t h) noexcept
			{
				return ((static_cast<uint64_t>(h) >> 55) & 1u) != 0;
			}
			inline uint32_t handle_generation(int64_t h) noexcept
			{
				return static_cast<uint32_t>((static_cast<uint64_t>(h) >> 32) & 0x7FFFFFu);
			}
			inline uint32_t handle_slot(int64_t h) noexcept
			{
				return static_cast<uint32_t>(static_cast<uint64_t>(h) & 0xFFFFFFFFu);
			}

			size_t dtype_size(avDataType_t dtype) noexcept;

			struct TensorObject
			{
				avDataType_t dtype = AVOCADO_DTYPE_UNKNOWN;
				int nb_dims = 0;
				int dims[AVOCADO_MAX_TENSOR_DIMENSIONS] = { };

				int dimension(int i) const
				{
					if (i < 0 or i >= nb_dims)
						throw std::out_of_range("tensor dimension index");
					return dims[i];
				}
				int firstDim() const
				{
					return nb_dims == 0 ? 0 : dims[0];
				}
				int lastDim() const
				{
					return nb_dims == 0 ? 0 : dims[nb_dims - 1];
				}
				int64_t volume() const noexcept
				{
					if (nb_dims == 0)
						return 0;
					int64_t v = 1;
					for (int i = 0; i < nb_dims; i++)
						v *= dims[i];
					return v;
				}
				int64_t volumeWithoutFirstDim() const noexcept
				{
					if (nb_dims == 0)
						return 0;
					int64_t v = 1;
					for (int i = 1; i < nb_dims; i++)
						v *= dims[i];
					return v;
				}
				int64_t sizeInBytes() const noexcept
				{
					return volume() * static_cast<int64_t>(dtype_size(dtype));
				}
			};

			struct MemoryObject
			{
				void *ptr = nullptr;
				int64_t size = 0;
				int device = 0;
				bool owning = false;
				~MemoryObject();
			};

			struct ConvolutionObject
			{
				avConvolutionMode_t mode = AVOCADO_CONVOLUTION_MODE;
				int nb_dims = 2;
				int padding[3] = { 0, 0, 0 };
				int strides[3] = { 1, 1, 1 };
				int dilation[3] = { 1, 1, 1 };
				int groups = 1;
				uint8_t padding_value[16] = { };
				/* additive extension: per-output-channel float32 requantisation scales (device memory handle, -1 = none) */
				int64_t quant_scales = -1;

				template<typename T>
				T getPaddingValue() const noexcept
				{
					T v;
					std::memcpy(&v, padding_value, sizeof(T));
					return v;
				}
				bool paddingValueIsZero() const noexcept
				{
					for (int i = 0; i < 16; i++)
						if (padding_value[i] != 0)
							return false;
					return true;
				}
			};

			struct OptimizerObject
			{
				avOptimizerType_t type = AVOCADO_OPTIMIZER_SGD;
				int64_t steps = 0;
				double learning_rate = 0.0;
				double coef[4] = { 0.0, 0.0, 0.0, 0.0 };
				bool flags[4] = { false, false, false, false };
			};

			/* A cudaGemmBatched call that a context with Winograd fusion switched on has accepted but not launched yet:
			 * M = V x U^T of the F(4x4,3x3) pipeline, waiting to see whether the next call on the context is the output
			 * transform of exactly that M (then one kernel does both and M is never written) or anything else (then the
			 * batched GEMM is launched first, as if it had never been held back). */
			struct DeferredGemm
			{
				bool valid = false;
				TensorObject a, b, c;
				const void *aPtr = nullptr;
				const void *bPtr = nullptr;
				void *cPtr = nullptr;
			};

			/* A cudaWinogradWeightTransform call (3x3 kernel) that a context with Winograd fusion switched on has accepted but
			 * not launched yet: if the next call on the context is an input transform that the TMA-staged kernel takes, the
			 * weight transform rides along in that launch; anything else launches it first as a kernel of its own. */
			struct DeferredWeightTransform
			{
				bool valid = false;
				ConvolutionObject conv;
				int transform_size = 0;
				TensorObject w, u;
				const void *wPtr = nullptr;
				void *uPtr = nullptr;
			};

			/* One stream on one device, a grow-only scratch buffer and a device-resident error word that kernels
			 * with bounded waits set when a wait runs out. */
			struct ContextObject
			{
				int device = 0;
				bool is_default = false;
				cudaStream_t stream = nullptr;
				void *workspace = nullptr;
				size_t workspace_size = 0;
				int *device_status = nullptr;
				cudaEvent_t order_event = nullptr; /* recorded on this stream when another context waits for this one */
				std::mutex lazy_mutex; /* guards the first allocation of workspace and device_status */
				bool fuse_winograd = false; /* cudaContextSetWinogradFusion, AVOCADO_WINOGRAD_FUSE_OUTPUT: hold cudaGemmBatched back */
				bool fuse_weights = false; /* AVOCADO_WINOGRAD_FUSE_WEIGHTS: hold cudaWinogradWeightTransform back */
				DeferredGemm deferred;
				DeferredWeightTransform deferred_weights;

				explicit ContextObject(int deviceIndex, bool isDefault);
				~ContextObject();
				ContextObject(const ContextObject&) = delete;
				ContextObject& operator=(const ContextObject&) = delete;

				void setDevice() const;
				cudaStream_t getStream() const noexcept
				{
					return stream;
				}
				/* Returns scratch of at least `bytes` bytes (256-byte aligned); grows the buffer when needed, which
				 * synchronises the stream first so earlier kernels are done with the old buffer. */
				void* getWorkspace(size_t bytes);
				int* getDeviceStatus();
			};

			template<class T>
			class Pool
			{
					std::mutex m_mutex;
					std::vector<std::unique_ptr<T>> m_slots;
					std::vector<uint32_t> m_generation;
					std::vector<uint32_t> m_free;
					Kind m_kind;
				public:
					explicit Pool(Kind kind) :
							m_kind(kind)
					{
					}
					int64_t insert(std::unique_ptr<T> object)
					{
						std::lock_guard<std::mutex> lock(m_mutex);
						uint32_t slot;
						if (m_free.empty())
						{
							slot = static_cast<uint32_t>(m_slots.size());
							m_slots.emplace_back();
							m_generation.push_back(1);
						}
						else
						{
							slot = m_free.back();
							m_free.pop_back();
						}
						m_slots[slot] = std::move(object);
						return make_handle(m_kind, false, m_generation[slot], slot);
					}
					T& get(int64_t handle)
					{
						std::lock_guard<std::mutex> lock(m_mutex);
						const uint32_t slot = handle_slot(handle);
						if (handle < 0 or handle_kind(handle) != m_kind or handle_is_default(handle) or slot >= m_slots.size() or m_slots[slot] == nullptr
								or m_generation[slot] != handle_generation(handle))
							throw std::invalid_argument("invalid descriptor");
						return *m_slots[slot];
					}
					bool valid(int64_t handle)
					{
						std::lock_guard<std::mutex> lock(m_mutex);
						const uint32_t slot = handle_slot(handle);
						return handle >= 0 and handle_kind(handle) == m_kind and not handle_is_default(handle) and slot < m_slots.size()
								and m_slots[slot] != nullptr and m_generation[slot] == handle_generation(handle);
					}
					/* Calls f(object) for every live object; f must not call back into this pool. */
					template<class F>
					void for_each(F &&f)
					{
						std::lock_guard<std::mutex> lock(m_mutex);
						for (auto &slot : m_slots)
							if (slot != nullptr)
								f(*slot);
					}
					/* Removes the object and returns it so that its destructor runs outside the pool lock. */
					std::unique_ptr<T> remove(int64_t handle)
					{
						std::lock_guard<std::mutex> lock(m_mutex);
						const uint32_t slot = handle_slot(handle);
						if (handle < 0 or handle_kind(handle) != m_kind or handle_is_default(handle) or slot >= m_slots.size() or m_slots[slot] == nullptr
								or m_generation[slot] != handle_generation(handle))
							return nullptr;
						std::unique_ptr<T> result = std::move(m_slots[slot]);
						m_generation[slot] = (m_generation[slot] + 1) & 0x7FFFFFu;
						if (m_generation[slot] == 0)
							m_generation[slot] = 1;
						m_free.push_back(slot);
						return result;
					}
			};

			Pool<ContextObject>& contextPool();
			Pool<MemoryObject>& memoryPool();
			Pool<TensorObject>& tensorPool();
			Pool<ConvolutionObject>& convolutionPool();
			Pool<OptimizerObject>& optimizerPool();

			int getNumberOfDevices() noexcept;

			/* Lookups used by the operators; each throws std::invalid_argument on a handle that is not live.
			 * getContext first launches a batched GEMM the context may be holding back (see DeferredGemm), so every
			 * entry point sees the context as if nothing had been deferred; getContextKeepDeferred is for the two
			 * entry points that look at the held-back call themselves. */
			ContextObject& getContext(avContextDescriptor_t handle);
			ContextObject& getContextKeepDeferred(avContextDescriptor_t handle);
			/* number of contexts currently holding a call back (lets the common path skip the search) */
			int deferredCount() noexcept;
			void noteDeferred(int delta) noexcept;
			bool isDefault(avContextDescriptor_t handle) noexcept;
			MemoryObject& getMemory(avMemoryDescriptor_t handle);
			TensorObject& getTensor(avTensorDescriptor_t handle);
			ConvolutionObject& getConvolution(avConvolutionDescriptor_t handle);
			OptimizerObject& getOptimizer(avOptimizerDescriptor_t handle);

			/* Device pointer behind a memory handle; null for AVOCADO_INVALID_DESCRIPTOR (how optional tensors are passed). */
			template<typename T = void>
			T* getPointer(avMemoryDescriptor_t handle)
			{
				if (handle == AVOCADO_INVALID_DESCRIPTOR)
					return nullptr;
				return reinterpret_cast<T*>(getMemory(handle).ptr);
			}

			/* Scalars arrive as host pointers: null means 1 for alpha-like and 0 for beta-like arguments. */
			template<typename T = float>
			T getAlphaValue(const void *alpha) noexcept
			{
				return alpha == nullptr ? static_cast<T>(1) : reinterpret_cast<const T*>(alpha)[0];
			}
			template<typename T = float>
			T getBetaValue(const void *beta) noexcept
			{
				return beta == nullptr ? static_cast<T>(0) : reinterpret_cast<const T*>(beta)[0];
			}
			inline bool is_transpose(avGemmOperation_t op) noexcept
			{
				return op == AVOCADO_GEMM_OPERATION_T;
			}

			/* true iff every spatial extent of w[K, kh, kw, C] equals expectedSize (ref src/im2row.cu:75-81) */
			bool is_conv(int expectedSize, const TensorObject &wDesc) noexcept;

			avStatus_t convertStatus(cudaError_t err) noexcept;
			/* Status of the launches issued since the last call (ref src/utilities.hpp:55-58). */
			avStatus_t checkForErrors() noexcept;
			int cuda_sm_version(int device) noexcept;
		} /* namespace b200 */
	} /* namespace backend */
} /* namespace avocado */

/* Wraps an entry-point body: handle-lookup failures become INTERNAL_ERROR as in ref src/descriptors.cu:270-276. */
#define AVOCADO_API_BEGIN try {
#define AVOCADO_API_END } catch (std::bad_alloc &e) { return AVOCADO_STATUS_BAD_ALLOC; } \
	catch (std::exception &e) { return AVOCADO_STATUS_INTERNAL_ERROR; }

#endif /* B200_OBJECTS_HPP_ */
