/*
 * optimizers.cu -- cudaOptimizerLearn: the weight update that follows the weight-gradient all-reduce of a training step.
 *
 * Counterpart of the reference's kernel_learn_sgd / kernel_learn_adam and their launchers (src/optimizers.cu:34-70,
 * :71-160, entry point :168-186).  Same formulas:
 *
 *   SGD        m = beta1 * m - lr * dw                      (only with the momentum flag; m lives in the workspace)
 *              step = m | beta1 * m - lr * dw (Nesterov) | -lr * dw (no momentum)
 *   ADAM       m = beta1 * m + (1 - beta1) * dw,   v = beta2 * v + (1 - beta2) * dw^2        (workspace: m then v)
 *              step = -lr_t * m / sqrt(v + eps),   lr_t = lr * sqrt(1 - beta2^t) / (1 - beta1^t) while t < 10000
 *   both       w = flush(alpha * step + beta * w),  flush(x) = 0 when |x| < eps
 *
 * Two deliberate differences:
 *   - the bias correction uses t = steps + 1.  The reference evaluates it with t = steps before incrementing, which is
 *     0 / 0 on the first update of a fresh descriptor;
 *   - eps is the machine epsilon of the tensor's type (the reference's scalar_eps<T>() is defined in a support header that
 *     is not part of its source tree).
 * Bound: HBM, 3 (SGD) to 7 (Adam) streams of the weight tensor's size; one thread per element, grid sized to the device.
 */
#include <Avocado/cuda_backend.h>

#include "objects.hpp"

#include <algorithm>
#include <cfloat>
#include <cmath>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;

	template<typename T> __host__ __device__ constexpr T type_eps();
	template<> __host__ __device__ constexpr float type_eps<float>()
	{
		return FLT_EPSILON;
	}
	template<> __host__ __device__ constexpr double type_eps<double>()
	{
		return DBL_EPSILON;
	}
	template<typename T>
	__device__ __forceinline__ T flush_small(T x)
	{
		return (x > -type_eps<T>() and x < type_eps<T>()) ? static_cast<T>(0) : x;
	}

	template<typename T>
	__global__ void __launch_bounds__(256) kernel_learn_sgd(T *__restrict__ weight, const T *__restrict__ update, T *__restrict__ momentum, long long elements,
			T learning_rate, T beta1, bool use_nesterov, T alpha, T beta)
	{
		for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < elements; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			const T g = update[i];
			T step;
			if (momentum != nullptr)
			{
				const T m = beta1 * momentum[i] - learning_rate * g;
				momentum[i] = m;
				step = use_nesterov ? beta1 * m - learning_rate * g : m;
			}
			else
				step = -learning_rate * g;
			weight[i] = flush_small(alpha * step + beta * weight[i]);
		}
	}
	template<typename T>
	__global__ void __launch_bounds__(256) kernel_learn_adam(T *__restrict__ weight, const T *__restrict__ update, T *__restrict__ momentum,
			T *__restrict__ variance, long long elements, T learning_rate, T beta1, T beta2, T alpha, T beta)
	{
		for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < elements; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			const T g = update[i];
			const T m = momentum[i] * beta1 + g * (static_cast<T>(1) - beta1);
			const T v = variance[i] * beta2 + g * g * (static_cast<T>(1) - beta2);
			momentum[i] = m;
			variance[i] = v;
			const T step = -m * learning_rate / sqrt(v + type_eps<T>());
			weight[i] = flush_small(alpha * step + beta * weight[i]);
		}
	}

	int grid_for(const ContextObject &ctx, long long elements)
	{
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		return static_cast<int>(std::max<long long>(1, std::min<long long>((elements + 255) / 256, static_cast<long long>(sms) * 8)));
	}

	template<typename T>
	avStatus_t learn(ContextObject &ctx, OptimizerObject &opt, const void *alpha, const void *beta, long long elements, void *w, const void *dw, void *workspace,
			size_t workspace_bytes)
	{
		const T a = getAlphaValue<T>(alpha);
		const T b = getBetaValue<T>(beta);
		const int grid = grid_for(ctx, elements);
		if (opt.type == AVOCADO_OPTIMIZER_SGD)
		{
			const bool use_momentum = opt.flags[0];
			if (use_momentum and (workspace == nullptr or workspace_bytes < static_cast<size_t>(elements) * sizeof(T)))
				return AVOCADO_STATUS_INTERNAL_ERROR; /* the status the reference gives for a workspace that is too small */
			kernel_learn_sgd<T> <<<grid, 256, 0, ctx.getStream()>>>(reinterpret_cast<T*>(w), reinterpret_cast<const T*>(dw),
					use_momentum ? reinterpret_cast<T*>(workspace) : nullptr, elements, static_cast<T>(opt.learning_rate), static_cast<T>(opt.coef[0]), opt.flags[1], a, b);
			return checkForErrors();
		}
		if (workspace == nullptr or workspace_bytes < 2 * static_cast<size_t>(elements) * sizeof(T))
			return AVOCADO_STATUS_INTERNAL_ERROR;
		const T beta1 = static_cast<T>(opt.coef[0]), beta2 = static_cast<T>(opt.coef[1]);
		T learning_rate = static_cast<T>(opt.learning_rate);
		const int64_t t = opt.steps + 1;
		if (t < 10000)
			learning_rate *= std::sqrt(static_cast<T>(1) - std::pow(beta2, static_cast<T>(t))) / (static_cast<T>(1) - std::pow(beta1, static_cast<T>(t)));
		kernel_learn_adam<T> <<<grid, 256, 0, ctx.getStream()>>>(reinterpret_cast<T*>(w), reinterpret_cast<const T*>(dw), reinterpret_cast<T*>(workspace),
				reinterpret_cast<T*>(workspace) + elements, elements, learning_rate, beta1, beta2, a, b);
		opt.steps++;
		return checkForErrors();
	}
}

namespace avocado
{
	namespace backend
	{
		avStatus_t cudaOptimizerLearn(avContextDescriptor_t context, const avOptimizerDescriptor_t config, const void *alpha, const avTensorDescriptor_t dwDesc,
				const avTensorDescriptor_t dwMem, const void *beta, const avTensorDescriptor_t wDesc, avMemoryDescriptor_t wMem, avMemoryDescriptor_t workspace)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				OptimizerObject &opt = getOptimizer(config);
				const TensorObject &w = getTensor(wDesc);
				const TensorObject &dw = getTensor(dwDesc);
				/* the reference's prototype types the gradient's memory handle as a tensor handle; it is a memory handle */
				const void *dw_ptr = getPointer(static_cast<avMemoryDescriptor_t>(dwMem));
				void *w_ptr = getPointer(wMem);
				if (w_ptr == nullptr or dw_ptr == nullptr or dw.dtype != w.dtype or dw.volume() != w.volume())
					return AVOCADO_STATUS_BAD_PARAM;
				if (opt.type != AVOCADO_OPTIMIZER_SGD and opt.type != AVOCADO_OPTIMIZER_ADAM)
					return AVOCADO_STATUS_BAD_PARAM;
				void *ws_ptr = getPointer(workspace);
				const size_t ws_bytes = (ws_ptr == nullptr) ? 0 : static_cast<size_t>(getMemory(workspace).size);
				ctx.setDevice();
				const long long elements = w.volume();
				if (elements == 0)
					return AVOCADO_STATUS_SUCCESS;
				switch (w.dtype)
				{
					case AVOCADO_DTYPE_FLOAT32:
						return learn<float>(ctx, opt, alpha, beta, elements, w_ptr, dw_ptr, ws_ptr, ws_bytes);
					case AVOCADO_DTYPE_FLOAT64:
						return learn<double>(ctx, opt, alpha, beta, elements, w_ptr, dw_ptr, ws_ptr, ws_bytes);
					default:
						return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				}
			AVOCADO_API_END
		}
	} /* namespace backend */
} /* namespace avocado */
