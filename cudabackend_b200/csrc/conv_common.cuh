/*
 * conv_common.cuh -- argument bundle and epilogue shared by the one-call convolution entry points
 * (cudaConvolutionImplicitGemmForward, cudaConvolutionWinogradFusedForward).
 *
 * Formula of both entry points (reference include/Avocado/cuda_backend.h:794-818):
 *     y = activation(alpha1 * conv(x, w) + alpha2 * z + b) + beta * y
 * evaluated in the order of the reference's output-transform epilogue (src/winograd_nonfused.cu:407-417):
 *     t = alpha1 * conv;  t += b[k];  t += alpha2 * z;  t = activation(t);  t += beta * y.
 *
 * Quantised form (int8 x, int8 w, int32 accumulator acc, optional int32 bias, optional float32 scale per output
 * channel), defined by this library because the reference's int8 kernel has no requantisation
 * (src/conv2d_implicit_gemm.cu:278, :330-339):
 *     t = acc + b[k]                      int32
 *     r = float(t)                        round to nearest even, as cvt.rn.f32.s32
 *     r = alpha1 * r   (if alpha1 != 1);  r = r * scale[k]   (if scales are attached)     one rounding each
 *     r = r + alpha2 * float(z)           (if z is given)
 *     r = activation(r)
 *     y = saturate_int8(round_to_nearest_even(r))            as cvt.rni.sat.s8.f32 (NaN saturates to -128)
 * With an int32 y the raw t is stored.
 */
#ifndef B200_CONV_COMMON_CUH_
#define B200_CONV_COMMON_CUH_

#include "device_utils.cuh"

namespace bk
{
	struct ConvArgs
	{
			int batch, height, width, channels; /* x: NHWC */
			int filters, kernel_h, kernel_w; /* w: [K, kh, kw, C] */
			int out_height, out_width;
			int pad_h, pad_w;
			bool rotate_kernel; /* AVOCADO_CROSS_CORRELATION_MODE */
			const void *x, *w, *bias, *z, *scales;
			void *y;
			avocado::backend::avActivationType_t activation;
	};

	/* the requantisation rule above; every step is a single correctly rounded float operation */
	__device__ __forceinline__ int8_t requantize(int32_t accPlusBias, float alpha1, bool useAlpha1, const float *scales, int k, const int8_t *z,
			size_t index, float alpha2, avocado::backend::avActivationType_t activation)
	{
		float r = int_to_float_rn(accPlusBias);
		if (useAlpha1)
			r = __fmul_rn(alpha1, r);
		if (scales != nullptr)
			r = __fmul_rn(r, scales[k]);
		if (z != nullptr)
			r = __fadd_rn(r, __fmul_rn(alpha2, small_int_to_float(z[index])));
		if (activation == avocado::backend::AVOCADO_ACTIVATION_RELU)
			r = fmaxf(r, 0.0f);
		else if (activation != avocado::backend::AVOCADO_ACTIVATION_LINEAR)
			r = activation_forward(activation, r);
		return static_cast<int8_t>(float_to_int8_rn_sat(r));
	}
} /* namespace bk */

#endif /* B200_CONV_COMMON_CUH_ */
