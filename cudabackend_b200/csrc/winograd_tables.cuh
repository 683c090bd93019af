/*
 * winograd_tables.cuh -- coefficient matrices of the Winograd transforms and the small dense
 * "T * X * T^T" machinery every transform kernel is built from.
 *
 * The matrices are the ones the reference uploads to constant memory (src/winograd_nonfused.cu:532-582):
 * F(2x2,3x3), F(4x4,3x3) and F(2x2,5x5), each with a weight, input, output, gradient and update matrix.
 * Here they are compile-time constants: after full unrolling every coefficient is an immediate, zero terms
 * vanish and +-1 terms become plain adds, so no table is read at run time and nothing has to be initialised
 * per device (the reference initialises once per process, which leaves a second GPU with zeroed tables).
 */
#ifndef B200_WINOGRAD_TABLES_CUH_
#define B200_WINOGRAD_TABLES_CUH_

namespace winograd
{
	enum class Transform
	{
		Weight, Input, Output, Gradient, Update
	};

	template<int TransformSize, int KernelSize>
	struct Coefficients;

	/* F(2x2, 3x3): tile 4 */
	template<>
	struct Coefficients<2, 3>
	{
			__host__ __device__ static constexpr double weight(int i, int j) /* 4 x 3 */
			{
				constexpr double t[12] = { 1.0, 0.0, 0.0, /**/1.0, 1.0, 1.0, /**/1.0, -1.0, 1.0, /**/0.0, 0.0, 1.0 };
				return t[i * 3 + j];
			}
			__host__ __device__ static constexpr double input(int i, int j) /* 4 x 4 */
			{
				constexpr double t[16] = { 1.0, 0.0, -1.0, 0.0, /**/0.0, 1.0, 1.0, 0.0, /**/0.0, -1.0, 1.0, 0.0, /**/0.0, -1.0, 0.0, 1.0 };
				return t[i * 4 + j];
			}
			__host__ __device__ static constexpr double output(int i, int j) /* 2 x 4 */
			{
				constexpr double t[8] = { 1.0, 0.5, 0.5, 0.0, /**/0.0, 0.5, -0.5, 1.0 };
				return t[i * 4 + j];
			}
			__host__ __device__ static constexpr double gradient(int i, int j) /* 4 x 2 */
			{
				constexpr double t[8] = { 1.0, 0.0, /**/1.0, 1.0, /**/1.0, -1.0, /**/0.0, 1.0 };
				return t[i * 2 + j];
			}
			__host__ __device__ static constexpr double update(int i, int j) /* 3 x 4 */
			{
				constexpr double t[12] = { 1.0, 0.5, 0.5, 0.0, /**/0.0, 0.5, -0.5, 0.0, /**/0.0, 0.5, 0.5, 1.0 };
				return t[i * 4 + j];
			}
	};

	/* F(4x4, 3x3): tile 6 */
	template<>
	struct Coefficients<4, 3>
	{
			__host__ __device__ static constexpr double weight(int i, int j) /* 6 x 3 */
			{
				constexpr double a = 2.0 / 3.0, b = 1.0 / 3.0, c = 4.0 / 3.0;
				constexpr double t[18] = { 1.0, 0.0, 0.0, /**/a, a, a, /**/a, -a, a, /**/b, a, c, /**/b, -a, c, /**/0.0, 0.0, 2.0 };
				return t[i * 3 + j];
			}
			__host__ __device__ static constexpr double input(int i, int j) /* 6 x 6 */
			{
				constexpr double t[36] = { 1.0, 0.0, -1.25, 0.0, 0.25, 0.0, /**/0.0, 1.0, 1.0, -0.25, -0.25, 0.0, /**/0.0, -1.0, 1.0, 0.25, -0.25, 0.0,
				/**/0.0, -1.0, -0.5, 1.0, 0.5, 0.0, /**/0.0, 1.0, -0.5, -1.0, 0.5, 0.0, /**/0.0, 1.0, 0.0, -1.25, 0.0, 0.25 };
				return t[i * 6 + j];
			}
			__host__ __device__ static constexpr double output(int i, int j) /* 4 x 6 */
			{
				constexpr double t[24] = { 1.0, 1.0, 1.0, 0.25, 0.25, 0.0, /**/0.0, 1.0, -1.0, 0.5, -0.5, 0.0, /**/0.0, 1.0, 1.0, 1.0, 1.0, 0.0,
				/**/0.0, 1.0, -1.0, 2.0, -2.0, 2.0 };
				return t[i * 6 + j];
			}
			__host__ __device__ static constexpr double gradient(int i, int j) /* 6 x 4 */
			{
				constexpr double a = 2.0 / 3.0, b = 1.0 / 3.0, c = 4.0 / 3.0, e = 8.0 / 3.0;
				constexpr double t[24] = { 1.0, 0.0, 0.0, 0.0, /**/a, a, a, a, /**/a, -a, a, -a, /**/b, a, c, e, /**/b, -a, c, -e, /**/0.0, 0.0, 0.0, 2.0 };
				return t[i * 4 + j];
			}
			__host__ __device__ static constexpr double update(int i, int j) /* 3 x 6 */
			{
				constexpr double t[18] = { 1.0, 1.0, 1.0, 0.25, 0.25, 0.0, /**/0.0, 1.0, -1.0, 0.5, -0.5, 0.0, /**/0.0, 1.0, 1.0, 1.0, 1.0, 2.0 };
				return t[i * 6 + j];
			}
	};

	/* F(2x2, 5x5): tile 6 */
	template<>
	struct Coefficients<2, 5>
	{
			__host__ __device__ static constexpr double weight(int i, int j) /* 6 x 5 */
			{
				constexpr double a = 2.0 / 3.0, b = 1.0 / 3.0, c = 4.0 / 3.0, e = 8.0 / 3.0, s = 1.0 / 6.0;
				constexpr double t[30] = { 1.0, 0.0, 0.0, 0.0, 0.0, /**/a, a, a, a, a, /**/a, -a, a, -a, a, /**/s, b, a, c, e, /**/s, -b, a, -c, e,
				/**/0.0, 0.0, 0.0, 0.0, 2.0 };
				return t[i * 5 + j];
			}
			__host__ __device__ static constexpr double input(int i, int j) /* 6 x 6, same points as F(4x4,3x3) */
			{
				return Coefficients<4, 3>::input(i, j);
			}
			__host__ __device__ static constexpr double output(int i, int j) /* 2 x 6 */
			{
				constexpr double t[12] = { 1.0, 1.0, 1.0, 0.5, 0.5, 0.0, /**/0.0, 1.0, -1.0, 1.0, -1.0, 2.0 };
				return t[i * 6 + j];
			}
			__host__ __device__ static constexpr double gradient(int i, int j) /* 6 x 2 */
			{
				constexpr double a = 2.0 / 3.0, b = 1.0 / 3.0;
				constexpr double t[12] = { 1.0, 0.0, /**/a, a, /**/a, -a, /**/b, a, /**/b, -a, /**/0.0, 1.0 };
				return t[i * 2 + j];
			}
			__host__ __device__ static constexpr double update(int i, int j) /* 5 x 6 */
			{
				constexpr double t[30] = { 1.0, 1.0, 1.0, 0.25, 0.25, 0.0, /**/0.0, 1.0, -1.0, 0.5, -0.5, 0.0, /**/0.0, 1.0, 1.0, 1.0, 1.0, 0.0,
				/**/0.0, 1.0, -1.0, 2.0, -2.0, 0.0, /**/0.0, 1.0, 1.0, 4.0, 4.0, 4.0 };
				return t[i * 6 + j];
			}
	};

	/* Shape and coefficient access of one of the five transforms: out[Rows x Rows] = T * in[Cols x Cols] * T^T
	 * with T of shape Rows x Cols. */
	template<Transform Type, int TS, int KS>
	struct Matrix
	{
			static constexpr int Tile = TS + KS - 1;
			static constexpr int Rows = (Type == Transform::Weight or Type == Transform::Input or Type == Transform::Gradient) ? Tile :
										(Type == Transform::Output) ? TS : KS;
			static constexpr int Cols = (Type == Transform::Weight) ? KS : (Type == Transform::Gradient) ? TS : Tile;
			__host__ __device__ static constexpr double at(int i, int j)
			{
				return (Type == Transform::Weight) ? Coefficients<TS, KS>::weight(i, j) :
						(Type == Transform::Input) ? Coefficients<TS, KS>::input(i, j) :
						(Type == Transform::Output) ? Coefficients<TS, KS>::output(i, j) :
						(Type == Transform::Gradient) ? Coefficients<TS, KS>::gradient(i, j) : Coefficients<TS, KS>::update(i, j);
			}
	};

#ifdef __CUDACC__
	/* acc += c * x with c known at compile time after unrolling */
	template<typename CT>
	__device__ __forceinline__ void accumulate(CT &acc, bool &started, const double c, const CT x)
	{
		if (c == 0.0)
			return;
		if (not started)
		{
			acc = (c == 1.0) ? x : (c == -1.0) ? -x : static_cast<CT>(c) * x;
			started = true;
			return;
		}
		if (c == 1.0)
			acc += x;
		else if (c == -1.0)
			acc -= x;
		else
			acc = fma(static_cast<CT>(c), x, acc);
	}

	/* out = T * in * T^T for one channel; `in` is Cols x Cols, `out` is Rows x Rows, both row-major in registers */
	template<class M, typename CT>
	__device__ __forceinline__ void transform_2d(const CT (&in)[M::Cols * M::Cols], CT (&out)[M::Rows * M::Rows])
	{
		CT tmp[M::Rows * M::Cols]; /* T * in */
#pragma unroll
		for (int i = 0; i < M::Rows; i++)
#pragma unroll
			for (int c = 0; c < M::Cols; c++)
			{
				CT acc = static_cast<CT>(0);
				bool started = false;
#pragma unroll
				for (int r = 0; r < M::Cols; r++)
					accumulate(acc, started, M::at(i, r), in[r * M::Cols + c]);
				tmp[i * M::Cols + c] = acc;
			}
#pragma unroll
		for (int i = 0; i < M::Rows; i++)
#pragma unroll
			for (int j = 0; j < M::Rows; j++)
			{
				CT acc = static_cast<CT>(0);
				bool started = false;
#pragma unroll
				for (int c = 0; c < M::Cols; c++)
					accumulate(acc, started, M::at(j, c), tmp[i * M::Cols + c]);
				out[i * M::Rows + j] = acc;
			}
	}
#endif
} /* namespace winograd */

#endif /* B200_WINOGRAD_TABLES_CUH_ */
