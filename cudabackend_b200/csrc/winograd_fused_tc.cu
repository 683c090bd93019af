/*
 * winograd_fused_tc.cu -- cudaConvolutionWinogradFusedForward: a whole Winograd convolution behind one call.
 *
 * The reference declares this entry point (include/Avocado/cuda_backend.h:840-844) and ships only an unfinished
 * F(2x2,3x3) kernel for it (src/winograd_fused.cu:587-775: weight tiles are constants, input tiles ignore the thread
 * index).  What the entry point promises -- y = activation(alpha1 * conv(x, w) + alpha2 * z + b) + beta * y with no
 * transform-domain tensor visible to the caller -- is delivered here by chaining, on the context's stream and in the
 * context's scratch buffer:
 *
 *   U = weight transform(w)        V = input transform(x)        M = V x U^T (tcgen05)        y = output transform(M)
 *
 * (the first two in one launch: the weight transform is a few blocks at the front of the input transform's grid)
 *
 * with the bias / z / activation / beta epilogue fused into the output transform.  For float16 / bfloat16 tensors the
 * last two steps are ONE kernel (winograd_fused_f23_tc.cu): M stays in TMEM and is never written to memory.  The transform-domain tensors are
 * internal, so their format is chosen for accuracy: float16 for float16 AND bfloat16 tensors with F(2x2,3x3) (a
 * bfloat16 domain would miss 1e-2, F(4x4,3x3) needs more than 10 mantissa bits), float32 with F(4x4,3x3) for float32.
 * The scratch buffer belongs to the context, grows on demand and is reused by the next call on that context, so
 * calls on one context are serialised by its stream and never see each other's scratch.
 */
#include "conv_kernels.hpp"
#include "winograd_internal.hpp"

#include <cstdlib>
#include <cstring>

namespace bk
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;

	namespace
	{
		size_t align_up(size_t value, size_t alignment)
		{
			return (value + alignment - 1) / alignment * alignment;
		}
		/* AVOCADO_B200_WINOGRAD=chained keeps the batched GEMM and the output transform as two kernels (A/B comparison) */
		bool chained_form_forced()
		{
			static const bool forced = []()
			{
				const char *env = std::getenv("AVOCADO_B200_WINOGRAD");
				return env != nullptr and std::strcmp(env, "chained") == 0;
			}();
			return forced;
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

	avStatus_t launch_winograd_fused_tc(ContextObject &ctx, const ConvArgs &args, avDataType_t xType, avDataType_t yType, const void *alpha1,
			const void *alpha2, const void *beta)
	{
		if (cuda_sm_version(ctx.device) != 100 or xType != yType)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (args.kernel_h != 3 or args.kernel_w != 3)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		/* the tile grid of the input transform is laid over x, that of the output transform over y: they must agree */
		if (args.out_height != args.height or args.out_width != args.width)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		int transform_size;
		avDataType_t matrices_type;
		switch (xType)
		{
			case AVOCADO_DTYPE_FLOAT16:
			case AVOCADO_DTYPE_BFLOAT16:
				transform_size = 2;
				matrices_type = AVOCADO_DTYPE_FLOAT16;
				break;
			case AVOCADO_DTYPE_FLOAT32:
				transform_size = 4;
				matrices_type = AVOCADO_DTYPE_FLOAT32;
				break;
			default:
				return AVOCADO_STATUS_NOT_SUPPORTED;
		}
		const int tile = transform_size + 2;
		const int planes = tile * tile;
		const long long tiles = static_cast<long long>(args.batch) * ((args.height + transform_size - 1) / transform_size)
				* ((args.width + transform_size - 1) / transform_size);
		if (tiles == 0 or args.channels == 0 or args.filters == 0)
			return AVOCADO_STATUS_SUCCESS;
		if (tiles > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;

		const size_t esize = dtype_size(matrices_type);
		const size_t u_bytes = align_up(static_cast<size_t>(planes) * args.filters * args.channels * esize, 256);
		const size_t v_bytes = align_up(static_cast<size_t>(planes) * tiles * args.channels * esize, 256);
		const size_t m_bytes = align_up(static_cast<size_t>(planes) * tiles * args.filters * esize, 256);
		uint8_t *scratch = reinterpret_cast<uint8_t*>(ctx.getWorkspace(u_bytes + v_bytes + m_bytes));
		void *u_ptr = scratch;
		void *v_ptr = scratch + u_bytes;
		void *m_ptr = scratch + u_bytes + v_bytes;

		ConvolutionObject conv;
		conv.mode = args.rotate_kernel ? AVOCADO_CROSS_CORRELATION_MODE : AVOCADO_CONVOLUTION_MODE;
		conv.padding[0] = args.pad_h;
		conv.padding[1] = args.pad_w;
		const TensorObject w = make_tensor(xType, { args.filters, 3, 3, args.channels });
		const TensorObject x = make_tensor(xType, { args.batch, args.height, args.width, args.channels });
		const TensorObject y = make_tensor(xType, { args.batch, args.out_height, args.out_width, args.filters });
		const TensorObject u = make_tensor(matrices_type, { planes, args.filters, args.channels });
		const TensorObject v = make_tensor(matrices_type, { planes, static_cast<int>(tiles), args.channels });
		const TensorObject m = make_tensor(matrices_type, { planes, static_cast<int>(tiles), args.filters });

		/* the weight transform rides along with the launch of the input transform when that launch can carry it */
		WeightRide ride = { args.w, u_ptr, args.filters, args.channels, transform_size, args.rotate_kernel, xType, matrices_type };
		bool ride_taken = false;
		avStatus_t status = winograd_input_transform(ctx, conv, transform_size, w, x, args.x, v, v_ptr, nullptr, &ride, &ride_taken);
		if (status != AVOCADO_STATUS_SUCCESS)
			return status;
		if (not ride_taken)
		{
			status = winograd_weight_transform(ctx, conv, transform_size, w, args.w, u, u_ptr);
			if (status != AVOCADO_STATUS_SUCCESS)
				return status;
		}
		if (transform_size == 2 and not chained_form_forced())
		{
			/* contraction and output transform in one kernel; M is never written */
			status = winograd_f23_contract_output(ctx, args, yType, tiles, v_ptr, u_ptr, alpha1, alpha2, beta, ctx.getDeviceStatus());
			if (status != AVOCADO_STATUS_NOT_SUPPORTED)
				return status;
		}
		status = gemm_batched(ctx, false, true, nullptr, v, v_ptr, u, u_ptr, nullptr, m, m_ptr);
		if (status != AVOCADO_STATUS_SUCCESS)
			return status;
		return winograd_output_transform(ctx, conv, transform_size, w, alpha1, m, m_ptr, y, args.y, args.bias, alpha2, args.z, beta, args.activation);
	}
} /* namespace bk */
