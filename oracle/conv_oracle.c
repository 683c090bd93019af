/*
 * conv_oracle.c -- CPU restatement of the reference's convolution path.  TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the product imports, links or runs this file: it is the checker used by tests/, by
 * __graft_entry__.smoke() and by the cpu_baseline / reference arm of bench.py.
 *
 * What it restates, and from where in the reference:
 *   - direct 2-D convolution, loop nest b -> k -> oh -> ow -> (i, j) -> c and index rule
 *     x = padding + i + oh (stride 1, dilation 1, groups 1): the only CPU convolution in the reference, the
 *     commented-out kernel_convolution_2d of app/CudaBackend.cu:122-200; kernel flip for
 *     AVOCADO_CROSS_CORRELATION_MODE as at :170-179;
 *   - epilogue order  t = alpha1*conv; t += bias[k]; t += alpha2*z; t = act(t); t += beta*y :
 *     src/winograd_nonfused.cu:407-417; activation formulas: src/activations.cuh:202-425;
 *   - the five Winograd tile transforms out = T * X * T^T with the coefficient tables of
 *     src/winograd_nonfused.cu:532-582 and the layouts of src/activations.cuh:43-57 (NHWC, tile index
 *     (b*tilesH + h)*tilesW + w) and :109-120 (matrices[(r*tile + c)*nbTiles + t][f]); kernels :256-521;
 *   - int8 convolution with int32 accumulation; the requantisation rule (bias add in int32, one float
 *     multiply by the per-channel scale, round to nearest even, saturate to [-128,127]) is this project's
 *     definition because the reference's int8 kernel (src/conv2d_implicit_gemm.cu:150-289) is unfinished
 *     and has no requantisation.
 *
 * PARITY PIN: pinned against outputs of the reference itself.  The reference's own kernels (src/winograd_nonfused.cu and
 * the cuBLAS wrapper src/gemm.cpp, compiled unmodified by oracle/build_ref.py) were run on a B200; their U, V, M, y,
 * G, Mw and dw for the seeded cases of oracle/run_ref.py are committed as tests/golden/reference_small.npz, and
 * tests/test_oracle.py checks that this oracle reproduces every one of them to the rounding of the storage type (float32
 * and float16; F(2x2,3x3), F(4x4,3x3), F(2x2,5x5)).  tests/test_reference_comparator.py repeats the comparison live on
 * larger shapes.  The transforms are also pinned by construction (chained with an exact GEMM they reproduce the direct
 * convolution and the exact weight gradient to 1e-12).  The reference's tests themselves store no vectors
 * (test/test_winograd.cpp compares against a fixture library that is not in its tree).
 * The int8 requantisation stays "parity unpinned" by the reference: its int8 kernel is unfinished and has none.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <fenv.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum
{
	ACT_LINEAR = 0, ACT_SIGMOID, ACT_TANH, ACT_RELU, ACT_SELU, ACT_ELU, ACT_EXPONENTIAL, ACT_SOFTPLUS, ACT_SOFTSIGN
};

static double activate(int activation, double x)
{
	switch (activation)
	{
		default:
		case ACT_LINEAR:
			return x;
		case ACT_SIGMOID:
			return 1.0 / (1.0 + exp(-x));
		case ACT_TANH:
			return tanh(x);
		case ACT_RELU:
			return x > 0.0 ? x : 0.0;
		case ACT_SELU:
			return x >= 0.0 ? (double) 1.05070098f * x : (double) 1.05070098f * (double) 1.67326324f * expm1(x);
		case ACT_ELU:
			return x >= 0.0 ? x : expm1(x);
		case ACT_EXPONENTIAL:
			return exp(x);
		case ACT_SOFTPLUS:
			return log1p(exp(x));
		case ACT_SOFTSIGN:
			return x / (fabs(x) + 1.0);
	}
}

/* number of threads the OpenMP loops below use from now on (a launcher may have exported OMP_NUM_THREADS=1) */
void oracle_set_threads(int threads)
{
#ifdef _OPENMP
	if (threads > 0)
		omp_set_num_threads(threads);
#else
	(void) threads;
#endif
}

int oracle_max_threads(void)
{
#ifdef _OPENMP
	return omp_get_max_threads();
#else
	return 1;
#endif
}

/* ---------------------------------------------------------------------------------------------------------
 * Direct convolution, float64.  x[N,H,W,C], w[K,kh,kw,C], y[N,Ho,Wo,K].  mode 0 applies the kernel as stored,
 * mode 1 rotates it by 180 degrees.  bias, z may be NULL.  y is read only when beta != 0.
 * --------------------------------------------------------------------------------------------------------- */
void oracle_conv2d_forward_f64(const double *x, const double *w, const double *bias, const double *z, double *y, int N, int H, int W, int C, int Ho,
		int Wo, int K, int kh, int kw, int pad_h, int pad_w, int mode, double padding_value, double alpha1, double alpha2, double beta, int activation)
{
#pragma omp parallel for collapse(2) schedule(static)
	for (int b = 0; b < N; b++)
		for (int oh = 0; oh < Ho; oh++)
			for (int ow = 0; ow < Wo; ow++)
				for (int k = 0; k < K; k++)
				{
					double acc = 0.0;
					for (int i = 0; i < kh; i++)
						for (int j = 0; j < kw; j++)
						{
							const int h = pad_h + i + oh;
							const int v = pad_w + j + ow;
							const int wi = (mode == 0) ? i : kh - 1 - i;
							const int wj = (mode == 0) ? j : kw - 1 - j;
							const double *wp = w + (((size_t) k * kh + wi) * kw + wj) * C;
							if (h >= 0 && h < H && v >= 0 && v < W)
							{
								const double *xp = x + (((size_t) b * H + h) * W + v) * C;
								for (int c = 0; c < C; c++)
									acc += wp[c] * xp[c];
							}
							else if (padding_value != 0.0)
							{
								for (int c = 0; c < C; c++)
									acc += wp[c] * padding_value;
							}
						}
					const size_t idx = (((size_t) b * Ho + oh) * Wo + ow) * K + k;
					double t = alpha1 * acc;
					if (bias != NULL)
						t += bias[k];
					if (z != NULL)
						t += alpha2 * z[idx];
					t = activate(activation, t);
					if (beta != 0.0)
						t += beta * y[idx];
					y[idx] = t;
				}
}

/* dx[n,h,w,c] = sum_{k,i,j} dy[n, h-pad_h-i, w-pad_w-j, k] * w[k,i,j,c]  (adjoint of the mode-0 forward) */
void oracle_conv2d_backward_data_f64(const double *dy, const double *w, double *dx, int N, int H, int W, int C, int Ho, int Wo, int K, int kh, int kw,
		int pad_h, int pad_w)
{
#pragma omp parallel for collapse(2) schedule(static)
	for (int b = 0; b < N; b++)
		for (int h = 0; h < H; h++)
			for (int v = 0; v < W; v++)
			{
				double *out = dx + (((size_t) b * H + h) * W + v) * C;
				for (int c = 0; c < C; c++)
					out[c] = 0.0;
				for (int i = 0; i < kh; i++)
					for (int j = 0; j < kw; j++)
					{
						const int oh = h - pad_h - i;
						const int ow = v - pad_w - j;
						if (oh < 0 || oh >= Ho || ow < 0 || ow >= Wo)
							continue;
						const double *g = dy + (((size_t) b * Ho + oh) * Wo + ow) * K;
						for (int k = 0; k < K; k++)
						{
							const double *wp = w + (((size_t) k * kh + i) * kw + j) * C;
							const double gv = g[k];
							for (int c = 0; c < C; c++)
								out[c] += gv * wp[c];
						}
					}
			}
}

/* dw[k,i,j,c] = sum_{n,oh,ow} dy[n,oh,ow,k] * x[n, pad_h+i+oh, pad_w+j+ow, c] */
void oracle_conv2d_backward_weights_f64(const double *x, const double *dy, double *dw, int N, int H, int W, int C, int Ho, int Wo, int K, int kh, int kw,
		int pad_h, int pad_w)
{
#pragma omp parallel for collapse(2) schedule(static)
	for (int k = 0; k < K; k++)
		for (int i = 0; i < kh; i++)
			for (int j = 0; j < kw; j++)
			{
				double *out = dw + (((size_t) k * kh + i) * kw + j) * C;
				for (int c = 0; c < C; c++)
					out[c] = 0.0;
				for (int b = 0; b < N; b++)
					for (int oh = 0; oh < Ho; oh++)
					{
						const int h = pad_h + i + oh;
						if (h < 0 || h >= H)
							continue;
						for (int ow = 0; ow < Wo; ow++)
						{
							const int v = pad_w + j + ow;
							if (v < 0 || v >= W)
								continue;
							const double gv = dy[(((size_t) b * Ho + oh) * Wo + ow) * K + k];
							const double *xp = x + (((size_t) b * H + h) * W + v) * C;
							for (int c = 0; c < C; c++)
								out[c] += gv * xp[c];
						}
					}
			}
}

/* ---------------------------------------------------------------------------------------------------------
 * The naive float32 convolution the reference's scratch driver uses as its CPU baseline
 * (app/CudaBackend.cu:122-200): float accumulation, same loop nest, parallel over (image, output row).
 * This is the timed cpu_baseline ("port"); it is never used as the correctness oracle.
 * --------------------------------------------------------------------------------------------------------- */
void oracle_conv2d_forward_f32_naive(const float *x, const float *w, const float *bias, float *y, int N, int H, int W, int C, int K, int kh, int kw,
		int pad_h, int pad_w, int relu)
{
#pragma omp parallel for collapse(2) schedule(static)
	for (int b = 0; b < N; b++)
		for (int oh = 0; oh < H; oh++)
			for (int k = 0; k < K; k++)
				for (int ow = 0; ow < W; ow++)
				{
					float acc = 0.0f;
					for (int i = 0; i < kh; i++)
						for (int j = 0; j < kw; j++)
						{
							const int h = pad_h + i + oh;
							const int v = pad_w + j + ow;
							if (h >= 0 && h < H && v >= 0 && v < W)
							{
								const float *wp = w + (((size_t) k * kh + i) * kw + j) * C;
								const float *xp = x + (((size_t) b * H + h) * W + v) * C;
								for (int c = 0; c < C; c++)
									acc += wp[c] * xp[c];
							}
						}
					if (bias != NULL)
						acc += bias[k];
					if (relu && acc < 0.0f)
						acc = 0.0f;
					y[(((size_t) b * H + oh) * W + ow) * K + k] = acc;
				}
}

/* ---------------------------------------------------------------------------------------------------------
 * int8 convolution for quantised inference.
 *   acc  = sum int32(x) * int32(w)                       exact
 *   t    = acc + bias[k]                                  int32 (bias may be NULL)
 *   f    = (float) t                                      round-to-nearest-even int -> float
 *   r    = alpha1 * f (only when alpha1 != 1), then r = r * scale[k]      one IEEE float multiply each
 *   r   += alpha2 * (float) z                             when z != NULL
 *   r    = act(r)                                         float
 *   q    = saturate_int8(nearbyintf(r))                   round to nearest even, clamp to [-128, 127]
 * With y_int32 != NULL the raw t is stored instead (the int32-output form of the entry point).
 * --------------------------------------------------------------------------------------------------------- */
static float activate_f32(int activation, float x)
{
	switch (activation)
	{
		default:
		case ACT_LINEAR:
			return x;
		case ACT_RELU:
			return x > 0.0f ? x : 0.0f;
		case ACT_SIGMOID:
			return 1.0f / (1.0f + expf(-x));
		case ACT_TANH:
			return tanhf(x);
	}
}
void oracle_conv2d_forward_int8(const int8_t *x, const int8_t *w, const int32_t *bias, const float *scale, const int8_t *z, int8_t *y_int8,
		int32_t *y_int32, int N, int H, int W, int C, int K, int kh, int kw, int pad_h, int pad_w, float alpha1, float alpha2, int activation)
{
#pragma omp parallel
	{
		fesetround(FE_TONEAREST);
#pragma omp for collapse(2) schedule(static)
		for (int b = 0; b < N; b++)
			for (int oh = 0; oh < H; oh++)
				for (int ow = 0; ow < W; ow++)
					for (int k = 0; k < K; k++)
					{
						int32_t acc = 0;
						for (int i = 0; i < kh; i++)
							for (int j = 0; j < kw; j++)
							{
								const int h = pad_h + i + oh;
								const int v = pad_w + j + ow;
								if (h >= 0 && h < H && v >= 0 && v < W)
								{
									const int8_t *wp = w + (((size_t) k * kh + i) * kw + j) * C;
									const int8_t *xp = x + (((size_t) b * H + h) * W + v) * C;
									for (int c = 0; c < C; c++)
										acc += (int32_t) wp[c] * (int32_t) xp[c];
								}
							}
						const size_t idx = (((size_t) b * H + oh) * W + ow) * K + k;
						const int32_t t = acc + (bias != NULL ? bias[k] : 0);
						if (y_int32 != NULL)
						{
							y_int32[idx] = t;
							continue;
						}
						volatile float r = (float) t;
						if (alpha1 != 1.0f)
							r = alpha1 * r;
						if (scale != NULL)
							r = r * scale[k];
						if (z != NULL)
						{
							volatile float zz = alpha2 * (float) z[idx];
							r = r + zz;
						}
						r = activate_f32(activation, r);
						float q = nearbyintf(r);
						if (q != q)
							q = -128.0f; /* NaN saturates to -128, the library's convention */
						if (q < -128.0f)
							q = -128.0f;
						if (q > 127.0f)
							q = 127.0f;
						y_int8[idx] = (int8_t) q;
					}
	}
}

/* ---------------------------------------------------------------------------------------------------------
 * Winograd tile transforms, float64.
 * --------------------------------------------------------------------------------------------------------- */
#define A23 (2.0 / 3.0)
#define B13 (1.0 / 3.0)
#define C43 (4.0 / 3.0)
#define E83 (8.0 / 3.0)
#define S16 (1.0 / 6.0)

/* kind: 0 weight, 1 input, 2 output, 3 gradient, 4 update.  Returns the matrix and its shape. */
static const double* table(int ts, int ks, int kind, int *rows, int *cols)
{
	static const double w23[] = { 1, 0, 0, 1, 1, 1, 1, -1, 1, 0, 0, 1 };
	static const double i23[] = { 1, 0, -1, 0, 0, 1, 1, 0, 0, -1, 1, 0, 0, -1, 0, 1 };
	static const double o23[] = { 1, .5, .5, 0, 0, .5, -.5, 1 };
	static const double g23[] = { 1, 0, 1, 1, 1, -1, 0, 1 };
	static const double u23[] = { 1, .5, .5, 0, 0, .5, -.5, 0, 0, .5, .5, 1 };

	static const double w43[] = { 1, 0, 0, A23, A23, A23, A23, -A23, A23, B13, A23, C43, B13, -A23, C43, 0, 0, 2 };
	static const double i43[] = { 1, 0, -1.25, 0, .25, 0, 0, 1, 1, -.25, -.25, 0, 0, -1, 1, .25, -.25, 0, 0, -1, -.5, 1, .5, 0, 0, 1, -.5, -1, .5, 0, 0, 1, 0,
			-1.25, 0, .25 };
	static const double o43[] = { 1, 1, 1, .25, .25, 0, 0, 1, -1, .5, -.5, 0, 0, 1, 1, 1, 1, 0, 0, 1, -1, 2, -2, 2 };
	static const double g43[] = { 1, 0, 0, 0, A23, A23, A23, A23, A23, -A23, A23, -A23, B13, A23, C43, E83, B13, -A23, C43, -E83, 0, 0, 0, 2 };
	static const double u43[] = { 1, 1, 1, .25, .25, 0, 0, 1, -1, .5, -.5, 0, 0, 1, 1, 1, 1, 2 };

	static const double w25[] = { 1, 0, 0, 0, 0, A23, A23, A23, A23, A23, A23, -A23, A23, -A23, A23, S16, B13, A23, C43, E83, S16, -B13, A23, -C43, E83, 0, 0,
			0, 0, 2 };
	static const double o25[] = { 1, 1, 1, .5, .5, 0, 0, 1, -1, 1, -1, 2 };
	static const double g25[] = { 1, 0, A23, A23, A23, -A23, B13, A23, B13, -A23, 0, 1 };
	static const double u25[] = { 1, 1, 1, .25, .25, 0, 0, 1, -1, .5, -.5, 0, 0, 1, 1, 1, 1, 0, 0, 1, -1, 2, -2, 0, 0, 1, 1, 4, 4, 4 };

	const int tile = ts + ks - 1;
	const int r[5] = { tile, tile, ts, tile, ks };
	const int c[5] = { ks, tile, tile, ts, tile };
	*rows = r[kind];
	*cols = c[kind];
	if (ts == 2 && ks == 3)
	{
		const double *t[5] = { w23, i23, o23, g23, u23 };
		return t[kind];
	}
	if (ts == 4 && ks == 3)
	{
		const double *t[5] = { w43, i43, o43, g43, u43 };
		return t[kind];
	}
	if (ts == 2 && ks == 5)
	{
		const double *t[5] = { w25, i43, o25, g25, u25 };
		return t[kind];
	}
	return NULL;
}

/* out[rows x rows] = T * in[cols x cols] * T^T */
static void sandwich(const double *T, int rows, int cols, const double *in, double *out)
{
	double tmp[8 * 8];
	for (int i = 0; i < rows; i++)
		for (int c = 0; c < cols; c++)
		{
			double acc = 0.0;
			for (int r = 0; r < cols; r++)
				acc += T[i * cols + r] * in[r * cols + c];
			tmp[i * cols + c] = acc;
		}
	for (int i = 0; i < rows; i++)
		for (int j = 0; j < rows; j++)
		{
			double acc = 0.0;
			for (int c = 0; c < cols; c++)
				acc += T[j * cols + c] * tmp[i * cols + c];
			out[i * rows + j] = acc;
		}
}

/* copies the coefficient matrix of one transform into `out` (row-major) and returns rows*cols, 0 if unknown */
int oracle_winograd_table(int ts, int ks, int kind, double *out, int *rows, int *cols)
{
	const double *T = table(ts, ks, kind, rows, cols);
	if (T == NULL)
		return 0;
	memcpy(out, T, sizeof(double) * (size_t) (*rows) * (size_t) (*cols));
	return (*rows) * (*cols);
}

/* w[K,ks,ks,C] -> matrices[tile*tile, K, C]; invert rotates the kernel by 180 degrees first */
int oracle_winograd_weight_transform_f64(const double *w, double *matrices, int K, int C, int ts, int ks, int invert)
{
	int rows, cols;
	const double *T = table(ts, ks, 0, &rows, &cols);
	if (T == NULL)
		return 1;
#pragma omp parallel for schedule(static)
	for (int k = 0; k < K; k++)
		for (int c = 0; c < C; c++)
		{
			double in[25], out[36];
			for (int i = 0; i < ks; i++)
				for (int j = 0; j < ks; j++)
				{
					const double v = w[(((size_t) k * ks + i) * ks + j) * C + c];
					if (invert)
						in[(ks - 1 - i) * ks + (ks - 1 - j)] = v;
					else
						in[i * ks + j] = v;
				}
			sandwich(T, rows, cols, in, out);
			for (int p = 0; p < rows * rows; p++)
				matrices[((size_t) p * K + k) * C + c] = out[p];
		}
	return 0;
}

/* x[N,H,W,C] -> matrices[tile*tile, N*tilesH*tilesW, C] */
int oracle_winograd_input_transform_f64(const double *x, double *matrices, int N, int H, int W, int C, int ts, int ks, int pad_h, int pad_w,
		double padding_value)
{
	int rows, cols;
	const double *T = table(ts, ks, 1, &rows, &cols);
	if (T == NULL)
		return 1;
	const int tile = ts + ks - 1;
	const int tiles_h = (H + ts - 1) / ts, tiles_w = (W + ts - 1) / ts;
	const size_t nb_tiles = (size_t) N * tiles_h * tiles_w;
#pragma omp parallel for collapse(2) schedule(static)
	for (int b = 0; b < N; b++)
		for (int th = 0; th < tiles_h; th++)
			for (int tw = 0; tw < tiles_w; tw++)
			{
				const size_t t = ((size_t) b * tiles_h + th) * tiles_w + tw;
				for (int c = 0; c < C; c++)
				{
					double in[36], out[36];
					for (int r = 0; r < tile; r++)
						for (int q = 0; q < tile; q++)
						{
							const int h = pad_h + th * ts + r;
							const int v = pad_w + tw * ts + q;
							in[r * tile + q] = (h >= 0 && h < H && v >= 0 && v < W) ? x[(((size_t) b * H + h) * W + v) * C + c] : padding_value;
						}
					sandwich(T, rows, cols, in, out);
					for (int p = 0; p < tile * tile; p++)
						matrices[((size_t) p * nb_tiles + t) * C + c] = out[p];
				}
			}
	return 0;
}

/* matrices[tile*tile, tiles, K] -> y[N,H,W,K] with the fused epilogue */
int oracle_winograd_output_transform_f64(const double *matrices, double *y, const double *bias, const double *z, int N, int H, int W, int K, int ts,
		int ks, double alpha1, double alpha2, double beta, int activation)
{
	int rows, cols;
	const double *T = table(ts, ks, 2, &rows, &cols);
	if (T == NULL)
		return 1;
	const int tile = ts + ks - 1;
	const int tiles_h = (H + ts - 1) / ts, tiles_w = (W + ts - 1) / ts;
	const size_t nb_tiles = (size_t) N * tiles_h * tiles_w;
#pragma omp parallel for collapse(2) schedule(static)
	for (int b = 0; b < N; b++)
		for (int th = 0; th < tiles_h; th++)
			for (int tw = 0; tw < tiles_w; tw++)
			{
				const size_t t = ((size_t) b * tiles_h + th) * tiles_w + tw;
				for (int k = 0; k < K; k++)
				{
					double in[36], out[16];
					for (int p = 0; p < tile * tile; p++)
						in[p] = matrices[((size_t) p * nb_tiles + t) * K + k];
					sandwich(T, rows, cols, in, out);
					for (int r = 0; r < ts; r++)
						for (int q = 0; q < ts; q++)
						{
							const int h = th * ts + r, v = tw * ts + q;
							if (h >= H || v >= W)
								continue;
							const size_t idx = (((size_t) b * H + h) * W + v) * K + k;
							double val = alpha1 * out[r * ts + q];
							if (bias != NULL)
								val += bias[k];
							if (z != NULL)
								val += alpha2 * z[idx];
							val = activate(activation, val);
							if (beta != 0.0)
								val += beta * y[idx];
							y[idx] = val;
						}
				}
			}
	return 0;
}

/* dy[N,H,W,K] -> matrices[tile*tile, tiles, K], zero past the image edge */
int oracle_winograd_gradient_transform_f64(const double *dy, double *matrices, int N, int H, int W, int K, int ts, int ks)
{
	int rows, cols;
	const double *T = table(ts, ks, 3, &rows, &cols);
	if (T == NULL)
		return 1;
	const int tile = ts + ks - 1;
	const int tiles_h = (H + ts - 1) / ts, tiles_w = (W + ts - 1) / ts;
	const size_t nb_tiles = (size_t) N * tiles_h * tiles_w;
#pragma omp parallel for collapse(2) schedule(static)
	for (int b = 0; b < N; b++)
		for (int th = 0; th < tiles_h; th++)
			for (int tw = 0; tw < tiles_w; tw++)
			{
				const size_t t = ((size_t) b * tiles_h + th) * tiles_w + tw;
				for (int k = 0; k < K; k++)
				{
					double in[16], out[36];
					for (int r = 0; r < ts; r++)
						for (int q = 0; q < ts; q++)
						{
							const int h = th * ts + r, v = tw * ts + q;
							in[r * ts + q] = (h < H && v < W) ? dy[(((size_t) b * H + h) * W + v) * K + k] : 0.0;
						}
					sandwich(T, rows, cols, in, out);
					for (int p = 0; p < tile * tile; p++)
						matrices[((size_t) p * nb_tiles + t) * K + k] = out[p];
				}
			}
	return 0;
}

/* matrices[tile*tile, K, C] -> dw[K,ks,ks,C] = alpha * transform + beta * dw */
int oracle_winograd_update_transform_f64(const double *matrices, double *dw, int K, int C, int ts, int ks, double alpha, double beta)
{
	int rows, cols;
	const double *T = table(ts, ks, 4, &rows, &cols);
	if (T == NULL)
		return 1;
	const int tile = ts + ks - 1;
#pragma omp parallel for schedule(static)
	for (int k = 0; k < K; k++)
		for (int c = 0; c < C; c++)
		{
			double in[36], out[25];
			for (int p = 0; p < tile * tile; p++)
				in[p] = matrices[((size_t) p * K + k) * C + c];
			sandwich(T, rows, cols, in, out);
			for (int i = 0; i < ks * ks; i++)
			{
				const size_t idx = ((size_t) k * ks * ks + i) * C + c;
				double val = alpha * out[i];
				if (beta != 0.0)
					val += beta * dw[idx];
				dw[idx] = val;
			}
		}
	return 0;
}

/* C[b] = alpha * op(A[b]) * op(B[b]) + beta * C[b], row-major, float64 (ref src/gemm.cpp:126-209 semantics) */
void oracle_gemm_batched_f64(int batch, int transA, int transB, int M, int N, int Kc, double alpha, const double *A, const double *B, double beta,
		double *C)
{
	const size_t strideA = (size_t) M * Kc, strideB = (size_t) N * Kc, strideC = (size_t) M * N;
#pragma omp parallel for collapse(2) schedule(static)
	for (int b = 0; b < batch; b++)
		for (int m = 0; m < M; m++)
			for (int n = 0; n < N; n++)
			{
				double acc = 0.0;
				for (int k = 0; k < Kc; k++)
				{
					const double a = transA ? A[b * strideA + (size_t) k * M + m] : A[b * strideA + (size_t) m * Kc + k];
					const double bb = transB ? B[b * strideB + (size_t) n * Kc + k] : B[b * strideB + (size_t) k * N + n];
					acc += a * bb;
				}
				double *out = C + b * strideC + (size_t) m * N + n;
				*out = alpha * acc + (beta != 0.0 ? beta * (*out) : 0.0);
			}
}
