/*
 * Stand-in for the reference's missing support header Avocado/backend_descriptors.hpp.  TEST INFRASTRUCTURE ONLY.
 *
 * The reference's hot-path sources (src/winograd_nonfused.cu, src/gemm.cpp, src/im2row.cu, src/activations.cuh) include this header
 * from a support library that is not part of the reference tree.  This file supplies just the classes and lookup
 * functions those sources use, so that they can be compiled UNMODIFIED, where they lie, into oracle/_ref/ and run on
 * a GPU as the comparator for the parity tests.  Handles are pointers to the objects below, cast to the integer
 * handle type.  Nothing of the product includes this file.
 */
#ifndef REF_SHIM_BACKEND_DESCRIPTORS_HPP_
#define REF_SHIM_BACKEND_DESCRIPTORS_HPP_

#include <Avocado/backend_defs.h>

#include <cuda_runtime_api.h>
#include <cublas_v2.h>

#include <cassert>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>

#define BACKEND_NAMESPACE cuda

namespace avocado
{
	namespace backend
	{
		namespace cuda
		{
			struct ContextDescriptor
			{
					int device = 0;
					cudaStream_t stream = nullptr;
					cublasHandle_t handle = nullptr;
					void setDevice() const
					{
						cudaSetDevice(device);
					}
					cudaStream_t getStream() const
					{
						return stream;
					}
					cublasHandle_t getHandle() const
					{
						return handle;
					}
					int getDevice() const
					{
						return device;
					}
			};
			struct MemoryDescriptor
			{
					void *ptr = nullptr;
					template<typename T> T* data()
					{
						return reinterpret_cast<T*>(ptr);
					}
					template<typename T> const T* data() const
					{
						return reinterpret_cast<const T*>(ptr);
					}
			};
			struct TensorDescriptor
			{
					avDataType_t type = AVOCADO_DTYPE_UNKNOWN;
					int rank = 0;
					int dims[AVOCADO_MAX_TENSOR_DIMENSIONS] = { };
					int dimension(int i) const
					{
						return dims[i];
					}
					int firstDim() const
					{
						return rank == 0 ? 0 : dims[0];
					}
					int lastDim() const
					{
						return rank == 0 ? 0 : dims[rank - 1];
					}
					int nbDims() const
					{
						return rank;
					}
					avDataType_t dtype() const
					{
						return type;
					}
					int volume() const
					{
						int v = rank == 0 ? 0 : 1;
						for (int i = 0; i < rank; i++)
							v *= dims[i];
						return v;
					}
					int volumeWithoutFirstDim() const
					{
						int v = rank == 0 ? 0 : 1;
						for (int i = 1; i < rank; i++)
							v *= dims[i];
						return v;
					}
			};
			struct ConvolutionDescriptor
			{
					avConvolutionMode_t mode = AVOCADO_CONVOLUTION_MODE;
					int padding[3] = { 0, 0, 0 };
					unsigned char padding_value[16] = { };
					template<typename T> T getPaddingValue() const
					{
						T v;
						std::memcpy(&v, padding_value, sizeof(T));
						return v;
					}
					/* unit stride and dilation, one group: the only case the comparator drives (src/im2row.cu:89) */
					TensorDescriptor getOutputShape(const TensorDescriptor &x, const TensorDescriptor &w) const
					{
						TensorDescriptor y;
						y.type = x.type;
						y.rank = x.rank;
						y.dims[0] = x.dims[0];
						for (int i = 1; i < x.rank - 1; i++)
							y.dims[i] = x.dims[i] - 2 * padding[i - 1] - (w.dims[i] - 1);
						y.dims[x.rank - 1] = w.dims[0];
						return y;
					}
			};
			inline int dataTypeSize(avDataType_t dtype)
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

			inline ContextDescriptor& getContext(avContextDescriptor_t h)
			{
				return *reinterpret_cast<ContextDescriptor*>(static_cast<intptr_t>(h));
			}
			inline MemoryDescriptor& getMemory(avMemoryDescriptor_t h)
			{
				static MemoryDescriptor null_memory;
				if (h == -1)
					return null_memory;
				return *reinterpret_cast<MemoryDescriptor*>(static_cast<intptr_t>(h));
			}
			inline TensorDescriptor& getTensor(avTensorDescriptor_t h)
			{
				static TensorDescriptor null_tensor;
				if (h == -1)
					return null_tensor;
				return *reinterpret_cast<TensorDescriptor*>(static_cast<intptr_t>(h));
			}
			inline ConvolutionDescriptor& getConvolution(avConvolutionDescriptor_t h)
			{
				return *reinterpret_cast<ConvolutionDescriptor*>(static_cast<intptr_t>(h));
			}
			template<typename T = void>
			T* getPointer(avMemoryDescriptor_t h)
			{
				return reinterpret_cast<T*>(getMemory(h).ptr);
			}
			template<typename T> inline T scalar_constant(double value)
			{
				return static_cast<T>(value);
			}
			template<> inline float2 scalar_constant<float2>(double value) /* cuComplex */
			{
				return float2 { static_cast<float>(value), 0.0f };
			}
			template<> inline double2 scalar_constant<double2>(double value) /* cuDoubleComplex */
			{
				return double2 { value, 0.0 };
			}
			template<typename T = float>
			T getAlphaValue(const void *alpha)
			{
				return alpha == nullptr ? scalar_constant<T>(1.0) : reinterpret_cast<const T*>(alpha)[0];
			}
			template<typename T = float>
			T getBetaValue(const void *beta)
			{
				return beta == nullptr ? scalar_constant<T>(0.0) : reinterpret_cast<const T*>(beta)[0];
			}
			inline bool is_transpose(avGemmOperation_t op)
			{
				return op == AVOCADO_GEMM_OPERATION_T;
			}
		} /* namespace cuda */
	} /* namespace backend */
} /* namespace avocado */

#endif /* REF_SHIM_BACKEND_DESCRIPTORS_HPP_ */
