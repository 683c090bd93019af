/*
 * winograd_nonfused.cu -- the five tile transforms of the non-fused Winograd pipeline.
 *
 * Entry points and their reference counterparts (src/winograd_nonfused.cu):
 *   cudaWinogradWeightTransform   :881  kernel :256   w[K,k,k,C]        -> U[t*t, K, C]
 *   cudaWinogradInputTransform    :906  kernel :302   x[N,H,W,C]        -> V[t*t, tiles, C]
 *   cudaWinogradOutputTransform   :932  kernel :366   M[t*t, tiles, K]  -> y[N,H,W,K]  (+ bias, z, activation, beta)
 *   cudaWinogradGradientTransform :963  kernel :424   dy[N,H,W,K]       -> [t*t, tiles, K]
 *   cudaWinogradUpdateTransform   :983  kernel :476   [t*t, K, C]       -> dw[K,k,k,C]
 *
 * All five are bandwidth-bound.  One thread owns one tile (or one filter) for VEC adjacent channels: the
 * channel index is the fastest-varying thread index, so every load and store of a warp is one contiguous
 * run of VEC * 32 channels, and all loads of a tile are issued before the first use.  Arithmetic is float
 * (double for float64 tensors) with one rounding on store.  The transform-domain tensor may be float32 while
 * the activations are 16-bit, which is what keeps F(4x4,3x3) within 1e-2 of an exact convolution.
 */
#include <Avocado/cuda_backend.h>

#include "objects.hpp"
#include "device_utils.cuh"
#include "winograd_tables.cuh"
#include "winograd_f43.cuh"
#include "winograd_internal.hpp"
#include "conv_kernels.hpp"

#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;
	using namespace ::bk;
	using winograd::Transform;
	using winograd::Matrix;

	constexpr int kThreads = 256;

	struct ConvGeometry
	{
			int batch, height, width, channels; /* of the NHWC tensor being tiled */
			int tiles_h, tiles_w;
			int pad_h, pad_w;
			__host__ __device__ long long nb_tiles() const
			{
				return static_cast<long long>(batch) * tiles_h * tiles_w;
			}
	};

	template<int TS, int KS, typename T, typename MT, int VEC>
	__global__ void __launch_bounds__(kThreads) kernel_weight_transform(MT *__restrict__ matrices, const T *__restrict__ weights, int filtersOut,
			int filtersIn, bool invert)
	{
		using CT = typename ComputeType<T>::type;
		using M = Matrix<Transform::Weight, TS, KS>;
		chain_wait();
		chain_release();
		const int cvecs = filtersIn / VEC;
		const long long g = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
		if (g >= static_cast<long long>(filtersOut) * cvecs)
			return;
		const int c0 = static_cast<int>(g % cvecs) * VEC;
		const int k = static_cast<int>(g / cvecs);

		CT in[VEC][KS * KS];
#pragma unroll
		for (int i = 0; i < KS * KS; i++)
		{
			const Vec<T, VEC> tmp = load_vec<T, VEC>(weights + (static_cast<size_t>(k) * KS * KS + i) * filtersIn + c0);
			const int dst = invert ? (KS * KS - 1 - i) : i; /* 180 degree rotation of the kernel */
#pragma unroll
			for (int v = 0; v < VEC; v++)
				in[v][dst] = to_compute(tmp.v[v]);
		}
		CT out[VEC][M::Rows * M::Rows];
#pragma unroll
		for (int v = 0; v < VEC; v++)
			winograd::transform_2d<M, CT>(in[v], out[v]);
#pragma unroll
		for (int p = 0; p < M::Rows * M::Rows; p++)
		{
			Vec<MT, VEC> tmp;
#pragma unroll
			for (int v = 0; v < VEC; v++)
				tmp.v[v] = from_compute<MT>(out[v][p]);
			store_vec<MT, VEC>(matrices + (static_cast<size_t>(p) * filtersOut + k) * filtersIn + c0, tmp);
		}
	}

	template<int TS, int KS, typename T, typename MT, int VEC>
	__global__ void __launch_bounds__(kThreads) kernel_input_transform(MT *__restrict__ matrices, const T *__restrict__ input, ConvGeometry geo,
			typename ComputeType<T>::type paddingValue)
	{
		using CT = typename ComputeType<T>::type;
		using M = Matrix<Transform::Input, TS, KS>;
		constexpr int TL = M::Tile;
		const int cvecs = geo.channels / VEC;
		const long long nb_tiles = geo.nb_tiles();
		const long long g = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
		if (g >= nb_tiles * cvecs)
			return;
		const int c0 = static_cast<int>(g % cvecs) * VEC;
		const long long tile = g / cvecs;
		const int tw = static_cast<int>(tile % geo.tiles_w);
		const int th = static_cast<int>((tile / geo.tiles_w) % geo.tiles_h);
		const int n = static_cast<int>(tile / (static_cast<long long>(geo.tiles_w) * geo.tiles_h));

		CT in[VEC][TL * TL];
#pragma unroll
		for (int r = 0; r < TL; r++)
		{
			const int h = geo.pad_h + th * TS + r;
#pragma unroll
			for (int c = 0; c < TL; c++)
			{
				const int w = geo.pad_w + tw * TS + c;
				if (h >= 0 and h < geo.height and w >= 0 and w < geo.width)
				{
					const Vec<T, VEC> tmp = load_vec<T, VEC>(input + ((static_cast<size_t>(n) * geo.height + h) * geo.width + w) * geo.channels + c0);
#pragma unroll
					for (int v = 0; v < VEC; v++)
						in[v][r * TL + c] = to_compute(tmp.v[v]);
				}
				else
				{
#pragma unroll
					for (int v = 0; v < VEC; v++)
						in[v][r * TL + c] = paddingValue;
				}
			}
		}
		CT out[VEC][TL * TL];
#pragma unroll
		for (int v = 0; v < VEC; v++)
			winograd::transform_2d<M, CT>(in[v], out[v]);
#pragma unroll
		for (int p = 0; p < TL * TL; p++)
		{
			Vec<MT, VEC> tmp;
#pragma unroll
			for (int v = 0; v < VEC; v++)
				tmp.v[v] = from_compute<MT>(out[v][p]);
			store_vec<MT, VEC>(matrices + (static_cast<size_t>(p) * nb_tiles + tile) * geo.channels + c0, tmp);
		}
	}

	template<int TS, int KS, typename T, typename MT, int VEC>
	__global__ void __launch_bounds__(kThreads) kernel_gradient_transform(MT *__restrict__ matrices, const T *__restrict__ gradient, ConvGeometry geo)
	{
		using CT = typename ComputeType<T>::type;
		using M = Matrix<Transform::Gradient, TS, KS>;
		constexpr int TL = M::Tile;
		const int cvecs = geo.channels / VEC;
		const long long nb_tiles = geo.nb_tiles();
		const long long g = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
		if (g >= nb_tiles * cvecs)
			return;
		const int c0 = static_cast<int>(g % cvecs) * VEC;
		const long long tile = g / cvecs;
		const int tw = static_cast<int>(tile % geo.tiles_w);
		const int th = static_cast<int>((tile / geo.tiles_w) % geo.tiles_h);
		const int n = static_cast<int>(tile / (static_cast<long long>(geo.tiles_w) * geo.tiles_h));

		CT in[VEC][TS * TS];
#pragma unroll
		for (int r = 0; r < TS; r++)
		{
			const int h = th * TS + r;
#pragma unroll
			for (int c = 0; c < TS; c++)
			{
				const int w = tw * TS + c;
				if (h < geo.height and w < geo.width)
				{
					const Vec<T, VEC> tmp = load_vec<T, VEC>(gradient + ((static_cast<size_t>(n) * geo.height + h) * geo.width + w) * geo.channels + c0);
#pragma unroll
					for (int v = 0; v < VEC; v++)
						in[v][r * TS + c] = to_compute(tmp.v[v]);
				}
				else
				{
#pragma unroll
					for (int v = 0; v < VEC; v++)
						in[v][r * TS + c] = static_cast<CT>(0);
				}
			}
		}
		CT out[VEC][TL * TL];
#pragma unroll
		for (int v = 0; v < VEC; v++)
			winograd::transform_2d<M, CT>(in[v], out[v]);
#pragma unroll
		for (int p = 0; p < TL * TL; p++)
		{
			Vec<MT, VEC> tmp;
#pragma unroll
			for (int v = 0; v < VEC; v++)
				tmp.v[v] = from_compute<MT>(out[v][p]);
			store_vec<MT, VEC>(matrices + (static_cast<size_t>(p) * nb_tiles + tile) * geo.channels + c0, tmp);
		}
	}

	/* BT is the bias type: float for 16-bit and float32 tensors, double for float64
	 * (ref src/winograd_nonfused.cu:758, :944-958). */
	template<int TS, int KS, typename T, typename MT, typename BT, int VEC>
	__global__ void __launch_bounds__(kThreads) kernel_output_transform(const MT *__restrict__ matrices, T *output, ConvGeometry geo,
			const BT *__restrict__ bias, const T *__restrict__ ext, typename ComputeType<T>::type alpha1, typename ComputeType<T>::type alpha2,
			typename ComputeType<T>::type beta, avActivationType_t activation)
	{
		using CT = typename ComputeType<T>::type;
		using M = Matrix<Transform::Output, TS, KS>;
		constexpr int TL = M::Tile;
		const int cvecs = geo.channels / VEC;
		const long long nb_tiles = geo.nb_tiles();
		const long long g = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
		if (g >= nb_tiles * cvecs)
			return;
		const int c0 = static_cast<int>(g % cvecs) * VEC;
		const long long tile = g / cvecs;
		const int tw = static_cast<int>(tile % geo.tiles_w);
		const int th = static_cast<int>((tile / geo.tiles_w) % geo.tiles_h);
		const int n = static_cast<int>(tile / (static_cast<long long>(geo.tiles_w) * geo.tiles_h));

		CT in[VEC][TL * TL];
#pragma unroll
		for (int p = 0; p < TL * TL; p++)
		{
			const Vec<MT, VEC> tmp = load_vec<MT, VEC>(matrices + (static_cast<size_t>(p) * nb_tiles + tile) * geo.channels + c0);
#pragma unroll
			for (int v = 0; v < VEC; v++)
				in[v][p] = static_cast<CT>(to_compute(tmp.v[v]));
		}
		CT out[VEC][TS * TS];
#pragma unroll
		for (int v = 0; v < VEC; v++)
			winograd::transform_2d<M, CT>(in[v], out[v]);

		CT b[VEC];
#pragma unroll
		for (int v = 0; v < VEC; v++)
			b[v] = (bias != nullptr) ? static_cast<CT>(bias[c0 + v]) : static_cast<CT>(0);

#pragma unroll
		for (int r = 0; r < TS; r++)
		{
			const int h = th * TS + r;
#pragma unroll
			for (int c = 0; c < TS; c++)
			{
				const int w = tw * TS + c;
				if (h < geo.height and w < geo.width)
				{
					const size_t index = ((static_cast<size_t>(n) * geo.height + h) * geo.width + w) * geo.channels + c0;
					CT val[VEC];
#pragma unroll
					for (int v = 0; v < VEC; v++)
						val[v] = alpha1 * out[v][r * TS + c] + b[v];
					if (ext != nullptr)
					{
						const Vec<T, VEC> tmp = load_vec<T, VEC>(ext + index);
#pragma unroll
						for (int v = 0; v < VEC; v++)
							val[v] += alpha2 * to_compute(tmp.v[v]);
					}
#pragma unroll
					for (int v = 0; v < VEC; v++)
						val[v] = activation_forward(activation, val[v]);
					if (beta != static_cast<CT>(0))
					{
						const Vec<T, VEC> tmp = load_vec<T, VEC>(output + index);
#pragma unroll
						for (int v = 0; v < VEC; v++)
							val[v] += beta * to_compute(tmp.v[v]);
					}
					Vec<T, VEC> result;
#pragma unroll
					for (int v = 0; v < VEC; v++)
						result.v[v] = from_compute<T>(val[v]);
					store_vec<T, VEC>(output + index, result);
				}
			}
		}
	}

	template<int TS, int KS, typename T, int VEC>
	__global__ void __launch_bounds__(kThreads) kernel_update_transform(const T *__restrict__ matrices, T *update, int filtersOut, int filtersIn,
			typename ComputeType<T>::type alpha, typename ComputeType<T>::type beta)
	{
		using CT = typename ComputeType<T>::type;
		using M = Matrix<Transform::Update, TS, KS>;
		constexpr int TL = M::Tile;
		const int cvecs = filtersIn / VEC;
		const long long g = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
		if (g >= static_cast<long long>(filtersOut) * cvecs)
			return;
		const int c0 = static_cast<int>(g % cvecs) * VEC;
		const int k = static_cast<int>(g / cvecs);

		CT in[VEC][TL * TL];
#pragma unroll
		for (int p = 0; p < TL * TL; p++)
		{
			const Vec<T, VEC> tmp = load_vec<T, VEC>(matrices + (static_cast<size_t>(p) * filtersOut + k) * filtersIn + c0);
#pragma unroll
			for (int v = 0; v < VEC; v++)
				in[v][p] = to_compute(tmp.v[v]);
		}
		CT out[VEC][KS * KS];
#pragma unroll
		for (int v = 0; v < VEC; v++)
			winograd::transform_2d<M, CT>(in[v], out[v]);
#pragma unroll
		for (int i = 0; i < KS * KS; i++)
		{
			const size_t index = (static_cast<size_t>(k) * KS * KS + i) * filtersIn + c0;
			Vec<T, VEC> result;
			if (beta != static_cast<CT>(0))
			{
				const Vec<T, VEC> old = load_vec<T, VEC>(update + index);
#pragma unroll
				for (int v = 0; v < VEC; v++)
					result.v[v] = from_compute<T>(alpha * out[v][i] + beta * to_compute(old.v[v]));
			}
			else
			{
#pragma unroll
				for (int v = 0; v < VEC; v++)
					result.v[v] = from_compute<T>(alpha * out[v][i]);
			}
			store_vec<T, VEC>(update + index, result);
		}
	}

	/* ------------------------------------------------------------------------------------------------------ */

	inline unsigned int blocks_for(long long threads)
	{
		return static_cast<unsigned int>((threads + kThreads - 1) / kThreads);
	}
	inline bool aligned_to(const void *ptr, size_t bytes)
	{
		return (reinterpret_cast<uintptr_t>(ptr) % bytes) == 0;
	}
	/* widest vector (in elements) that divides the channel count and matches the alignment of every pointer */
	template<typename T, typename MT>
	int pick_vec(int channels, int maxVec, std::initializer_list<const void*> tensorPtrs, std::initializer_list<const void*> matrixPtrs)
	{
		for (int vec = maxVec; vec > 1; vec /= 2)
		{
			bool ok = (channels % vec == 0);
			for (const void *p : tensorPtrs)
				ok = ok and (p == nullptr or aligned_to(p, sizeof(T) * vec));
			for (const void *p : matrixPtrs)
				ok = ok and (p == nullptr or aligned_to(p, sizeof(MT) * vec));
			if (ok)
				return vec;
		}
		return 1;
	}

	bool tile_config_supported(const TensorObject &wDesc, int transformSize)
	{
		if (wDesc.nb_dims != 4)
			return false;
		if (is_conv(3, wDesc))
			return transformSize == 2 or transformSize == 4;
		if (is_conv(5, wDesc))
			return transformSize == 2;
		return false;
	}

	/* Calls f(TS, KS) with the sizes as compile-time constants. */
#define DISPATCH_TILE(kernelSize, transformSize, ...) \
	if ((kernelSize) == 3 and (transformSize) == 2) { constexpr int TS = 2, KS = 3; __VA_ARGS__ } \
	else if ((kernelSize) == 3 and (transformSize) == 4) { constexpr int TS = 4, KS = 3; __VA_ARGS__ } \
	else if ((kernelSize) == 5 and (transformSize) == 2) { constexpr int TS = 2, KS = 5; __VA_ARGS__ } \
	else return AVOCADO_STATUS_NOT_SUPPORTED;

#define DISPATCH_VEC2(vec, ...) \
	if ((vec) == 2) { constexpr int VEC = 2; __VA_ARGS__ } else { constexpr int VEC = 1; __VA_ARGS__ }

	template<typename T, typename MT>
	avStatus_t launch_weight_transform(ContextObject &ctx, const ConvolutionObject &config, const TensorObject &wDesc, const void *wPtr,
			const TensorObject &matricesDesc, void *matricesPtr, int transformSize)
	{
		const int K = wDesc.dims[0], ks = wDesc.dims[1], C = wDesc.dims[3];
		const int tile = transformSize + ks - 1;
		if (matricesDesc.nb_dims != 3 or matricesDesc.dims[0] != tile * tile or matricesDesc.dims[1] != K or matricesDesc.dims[2] != C)
			return AVOCADO_STATUS_BAD_PARAM;
		if (K == 0 or C == 0)
			return AVOCADO_STATUS_SUCCESS;
		const bool invert = (config.mode == AVOCADO_CROSS_CORRELATION_MODE);
		const int vec = pick_vec<T, MT>(C, sizeof(T) == 8 ? 1 : 2, { wPtr }, { matricesPtr });
		const unsigned int grid = blocks_for(static_cast<long long>(K) * (C / vec));
		DISPATCH_TILE(ks, transformSize,
				DISPATCH_VEC2(vec, launch_chained(kernel_weight_transform<TS, KS, T, MT, VEC>, dim3(grid), dim3(kThreads), 0, ctx.getStream(), reinterpret_cast<MT*>(matricesPtr), reinterpret_cast<const T*>(wPtr), K, C, invert);))
		return checkForErrors();
	}

	ConvGeometry make_geometry(const TensorObject &desc, int transformSize, const ConvolutionObject &config)
	{
		ConvGeometry geo;
		geo.batch = desc.dims[0];
		geo.height = desc.dims[1];
		geo.width = desc.dims[2];
		geo.channels = desc.dims[3];
		geo.tiles_h = (geo.height + transformSize - 1) / transformSize;
		geo.tiles_w = (geo.width + transformSize - 1) / transformSize;
		geo.pad_h = config.padding[0];
		geo.pad_w = config.padding[1];
		return geo;
	}
	bool matrices_match(const TensorObject &matricesDesc, int tile, const ConvGeometry &geo)
	{
		return matricesDesc.nb_dims == 3 and matricesDesc.dims[0] == tile * tile and matricesDesc.dims[1] == geo.nb_tiles()
				and matricesDesc.dims[2] == geo.channels;
	}


	/* ------------------------------------------------------------------------------------------------------
	 * F(4x4,3x3) fast paths (winograd_f43.cuh).  Each returns NOT_SUPPORTED when the case is outside what the
	 * fast kernel covers; the caller then launches the generic kernel.
	 * ------------------------------------------------------------------------------------------------------ */
	template<typename T> struct TmaType;
	template<> struct TmaType<half>
	{
			static constexpr CUtensorMapDataType value = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
	};
	template<> struct TmaType<__nv_bfloat16>
	{
			static constexpr CUtensorMapDataType value = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
	};
	template<> struct TmaType<float>
	{
			static constexpr CUtensorMapDataType value = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
	};

	/* AVOCADO_B200_INPUT_PAIRS=1 keeps one pair of channels per lane in the F(2x2) input transform (for A/B timing) */
	bool wide_lanes_enabled()
	{
		static const bool enabled = []()
		{
			const char *env = std::getenv("AVOCADO_B200_INPUT_PAIRS");
			return not (env != nullptr and std::strcmp(env, "1") == 0);
		}();
		return enabled;
	}

	template<int TS, typename T, typename MT, int Q>
	avStatus_t launch_f43_input_q(ContextObject &ctx, const ConvolutionObject &config, const ConvGeometry &geo, const void *xPtr, void *matricesPtr,
			int *deviceStatus, const bk::WeightRide *ride, bool *rideTaken)
	{
		if (cuda_sm_version(ctx.device) != 100 or not config.paddingValueIsZero())
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if ((geo.channels * sizeof(T)) % 16 != 0 or not aligned_to(xPtr, 16) or not aligned_to(matricesPtr, 2 * Q * sizeof(MT)))
			return AVOCADO_STATUS_NOT_SUPPORTED;
		constexpr int kWarpChannels = f43::kChannelBlock * Q; /* channels one warp covers */
		/* a strip's halo box is at most 48 KB; F(4x4) strips hold at most 8 tiles (one per warp), F(2x2) strips up to 32 */
		const int max_pixels = 48 * 1024 / (kWarpChannels * static_cast<int>(sizeof(T)));
		const int max_tiles = (TS == 4) ? 8 : 32;
		const int max_tw = std::min((TS == 4) ? 8 : 16, (max_pixels / (TS + 2) - 2) / TS);
		const int segments = (geo.tiles_w + max_tw - 1) / max_tw;
		f43::InputGeometry g;
		g.strip_tiles_w = (geo.tiles_w + segments - 1) / segments;
		g.box_w = TS * g.strip_tiles_w + 2;
		g.strip_tiles_h = std::max(1, std::min(std::min(geo.tiles_h, max_tiles / g.strip_tiles_w), (max_pixels / g.box_w - 2) / TS));
		const int box_h = TS * g.strip_tiles_h + 2;
		if (g.box_w > 256 or box_h > 256)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		g.batch = geo.batch;
		g.tiles_h = geo.tiles_h;
		g.tiles_w = geo.tiles_w;
		g.channels = geo.channels;
		g.pad_h = geo.pad_h;
		g.pad_w = geo.pad_w;
		g.row_groups = (geo.tiles_h + g.strip_tiles_h - 1) / g.strip_tiles_h;
		g.w_segments = (geo.tiles_w + g.strip_tiles_w - 1) / g.strip_tiles_w;
		g.c_blocks = (geo.channels + kWarpChannels - 1) / kWarpChannels;
		g.stage_bytes = box_h * g.box_w * kWarpChannels * static_cast<int>(sizeof(T));
		g.nb_tiles = geo.nb_tiles();
		const long long items = static_cast<long long>(geo.batch) * g.row_groups * g.w_segments * g.c_blocks;
		if (items > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		g.num_items = static_cast<int>(items);

		CUtensorMap map;
		const uint64_t dims[4] = { static_cast<uint64_t>(geo.channels), static_cast<uint64_t>(geo.width), static_cast<uint64_t>(geo.height),
				static_cast<uint64_t>(geo.batch) };
		const uint64_t strides[3] = { static_cast<uint64_t>(geo.channels) * sizeof(T), static_cast<uint64_t>(geo.width) * geo.channels * sizeof(T),
				static_cast<uint64_t>(geo.height) * geo.width * geo.channels * sizeof(T) };
		const uint32_t box[4] = { static_cast<uint32_t>(kWarpChannels), static_cast<uint32_t>(g.box_w), static_cast<uint32_t>(box_h), 1u };
		if (not umma::make_tensor_map(&map, TmaType<T>::value, 4, const_cast<void*>(xPtr), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
			return AVOCADO_STATUS_NOT_SUPPORTED;

		auto kernel = f43::kernel_input_tma<TS, T, MT, Q>;
		constexpr int ring_bytes = 96 * 1024; /* shared memory per block for the halo ring: two blocks per SM stay resident */
		g.stages = std::max(2, std::min(f43::kMaxStages, ring_bytes / g.stage_bytes));
		const int smem_bytes = g.stages * g.stage_bytes + 128;
		static PerDeviceOnce configured;
		if (configured.run(ctx.device, [&]() -> cudaError_t { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024 + 128); }) != cudaSuccess)
		{
			cudaGetLastError();
			return AVOCADO_STATUS_EXECUTION_FAILED;
		}
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		const int threads = 32 * std::min(8, g.strip_tiles_h * g.strip_tiles_w);
		const int ctas_per_sm = std::max(1, std::min(4, (220 * 1024) / (smem_bytes + 1024)));
		/* a weight transform waiting for a launch to ride along with (3x3 kernel, even channel count, aligned pairs) */
		f43::WeightJob job = { };
		if (ride != nullptr and ride->transformSize == TS and ride->filters > 0 and ride->channels > 0 and ride->channels % 2 == 0
				and aligned_to(ride->weights, 2 * sizeof(T)) and aligned_to(ride->matrices, 2 * sizeof(MT)))
		{
			job.weights = ride->weights;
			job.matrices = ride->matrices;
			job.filters = ride->filters;
			job.channels = ride->channels;
			job.invert = ride->invert ? 1 : 0;
			const long long pairs = static_cast<long long>(ride->filters) * (ride->channels / 2);
			job.ctas = static_cast<int>(std::min<long long>((pairs + threads - 1) / threads, std::max(1, sms / 4)));
		}
		const int grid = std::max(1, std::min(g.num_items, ctas_per_sm * sms - job.ctas)) + job.ctas;
		const cudaError_t launched = launch_chained(kernel, dim3(grid), dim3(threads), smem_bytes, ctx.getStream(), map, reinterpret_cast<MT*>(matricesPtr), g,
				deviceStatus != nullptr ? deviceStatus : ctx.getDeviceStatus(), job);
		if (launched != cudaSuccess)
			return convertStatus(launched);
		if (rideTaken != nullptr)
			rideTaken[0] = job.ctas > 0;
		return checkForErrors();
	}

	template<int TS, typename T, typename MT>
	avStatus_t launch_f43_input(ContextObject &ctx, const ConvolutionObject &config, const ConvGeometry &geo, const void *xPtr, void *matricesPtr,
			int *deviceStatus, const bk::WeightRide *ride, bool *rideTaken)
	{
		/* two pairs of channels per lane where a tile is small enough for the registers (F(2x2), 16-bit activations) and the
		 * layer has whole groups of four channels, at least a warp's worth of them */
		if constexpr (TS == 2 and sizeof(T) == 2)
		{
			if (wide_lanes_enabled() and geo.channels % 4 == 0 and geo.channels >= 2 * f43::kChannelBlock and aligned_to(matricesPtr, 4 * sizeof(MT)))
			{
				const avStatus_t status = launch_f43_input_q<TS, T, MT, 2>(ctx, config, geo, xPtr, matricesPtr, deviceStatus, ride, rideTaken);
				if (status != AVOCADO_STATUS_NOT_SUPPORTED)
					return status;
			}
		}
		return launch_f43_input_q<TS, T, MT, 1>(ctx, config, geo, xPtr, matricesPtr, deviceStatus, ride, rideTaken);
	}

	f43::PlaneGeometry plane_geometry(const ConvGeometry &geo)
	{
		f43::PlaneGeometry g;
		g.batch = geo.batch;
		g.height = geo.height;
		g.width = geo.width;
		g.channels = geo.channels;
		g.tiles_h = geo.tiles_h;
		g.tiles_w = geo.tiles_w;
		g.nb_tiles = geo.nb_tiles();
		return g;
	}

	template<int TS, typename T, typename MT>
	avStatus_t launch_f43_output(ContextObject &ctx, const ConvGeometry &geo, const void *matricesPtr, void *yPtr, const void *bPtr, const void *zPtr,
			float alpha1, float alpha2, float beta, avActivationType_t activation)
	{
		if (geo.channels % 2 != 0 or not aligned_to(matricesPtr, 2 * sizeof(MT)) or not aligned_to(yPtr, 2 * sizeof(T))
				or (zPtr != nullptr and not aligned_to(zPtr, 2 * sizeof(T))) or (bPtr != nullptr and not aligned_to(bPtr, 8)))
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (static_cast<long long>(geo.height) * geo.width * geo.channels > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const f43::PlaneGeometry g = plane_geometry(geo);
		if (g.nb_tiles > 0x7FFFFFFFll or geo.channels > 65535 * f43::kChannelBlock)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const dim3 grid(static_cast<unsigned int>((g.nb_tiles + 7) / 8), (geo.channels + f43::kChannelBlock - 1) / f43::kChannelBlock);
		const MT *m = reinterpret_cast<const MT*>(matricesPtr);
		T *y = reinterpret_cast<T*>(yPtr);
		const float *b = reinterpret_cast<const float*>(bPtr);
		const T *z = reinterpret_cast<const T*>(zPtr);
		cudaStream_t stream = ctx.getStream();
		if (activation == AVOCADO_ACTIVATION_LINEAR)
			launch_chained(f43::kernel_output<TS, T, MT, 0>, grid, dim3(f43::kThreads), 0, stream, m, y, g, b, z, alpha1, alpha2, beta, activation);
		else if (activation == AVOCADO_ACTIVATION_RELU)
			launch_chained(f43::kernel_output<TS, T, MT, 1>, grid, dim3(f43::kThreads), 0, stream, m, y, g, b, z, alpha1, alpha2, beta, activation);
		else
			launch_chained(f43::kernel_output<TS, T, MT, 2>, grid, dim3(f43::kThreads), 0, stream, m, y, g, b, z, alpha1, alpha2, beta, activation);
		return checkForErrors();
	}

	template<int TS, typename T, typename MT>
	avStatus_t launch_f43_gradient(ContextObject &ctx, const ConvGeometry &geo, const void *dyPtr, void *matricesPtr)
	{
		if (geo.channels % 2 != 0 or not aligned_to(matricesPtr, 2 * sizeof(MT)) or not aligned_to(dyPtr, 2 * sizeof(T)))
			return AVOCADO_STATUS_NOT_SUPPORTED;
		if (static_cast<long long>(geo.height) * geo.width * geo.channels > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const f43::PlaneGeometry g = plane_geometry(geo);
		if (g.nb_tiles > 0x7FFFFFFFll or geo.channels > 65535 * f43::kChannelBlock)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		const dim3 grid(static_cast<unsigned int>((g.nb_tiles + 7) / 8), (geo.channels + f43::kChannelBlock - 1) / f43::kChannelBlock);
		f43::kernel_gradient<TS, T, MT> <<<grid, f43::kThreads, 0, ctx.getStream()>>>(reinterpret_cast<MT*>(matricesPtr), reinterpret_cast<const T*>(dyPtr), g);
		return checkForErrors();
	}

	/* the generic kernels stay reachable for A/B comparison: AVOCADO_B200_WINOGRAD=generic disables the fast paths */
	bool fast_paths_enabled()
	{
		static const bool enabled = []()
		{
			const char *env = std::getenv("AVOCADO_B200_WINOGRAD");
			return not (env != nullptr and std::strcmp(env, "generic") == 0);
		}();
		return enabled;
	}


	/* float64 has no fast kernel: these wrappers keep the double instantiations out of the fast templates */
	template<int TS, typename T, typename MT>
	avStatus_t launch_f43_input_if(ContextObject &ctx, const ConvolutionObject &config, const ConvGeometry &geo, const void *xPtr, void *matricesPtr,
			int *deviceStatus, const bk::WeightRide *ride, bool *rideTaken)
	{
		if constexpr (sizeof(T) <= 4)
			return launch_f43_input<TS, T, MT>(ctx, config, geo, xPtr, matricesPtr, deviceStatus, ride, rideTaken);
		else
			return AVOCADO_STATUS_NOT_SUPPORTED;
	}
	template<int TS, typename T, typename MT>
	avStatus_t launch_f43_output_if(ContextObject &ctx, const ConvGeometry &geo, const void *matricesPtr, void *yPtr, const void *bPtr, const void *zPtr,
			double alpha1, double alpha2, double beta, avActivationType_t activation)
	{
		if constexpr (sizeof(T) <= 4)
			return launch_f43_output<TS, T, MT>(ctx, geo, matricesPtr, yPtr, bPtr, zPtr, static_cast<float>(alpha1), static_cast<float>(alpha2),
					static_cast<float>(beta), activation);
		else
			return AVOCADO_STATUS_NOT_SUPPORTED;
	}
	template<int TS, typename T, typename MT>
	avStatus_t launch_f43_gradient_if(ContextObject &ctx, const ConvGeometry &geo, const void *dyPtr, void *matricesPtr)
	{
		if constexpr (sizeof(T) <= 4)
			return launch_f43_gradient<TS, T, MT>(ctx, geo, dyPtr, matricesPtr);
		else
			return AVOCADO_STATUS_NOT_SUPPORTED;
	}

	template<typename T, typename MT>
	avStatus_t launch_input_transform(ContextObject &ctx, const ConvolutionObject &config, const TensorObject &wDesc, const TensorObject &xDesc,
			const void *xPtr, const TensorObject &matricesDesc, void *matricesPtr, int transformSize, int *deviceStatus, const bk::WeightRide *ride,
			bool *rideTaken)
	{
		using CT = typename ComputeType<T>::type;
		if (xDesc.nb_dims != 4)
			return AVOCADO_STATUS_BAD_PARAM;
		const int ks = wDesc.dims[1];
		const ConvGeometry geo = make_geometry(xDesc, transformSize, config);
		if (not matrices_match(matricesDesc, transformSize + ks - 1, geo))
			return AVOCADO_STATUS_BAD_PARAM;
		if (geo.nb_tiles() == 0 or geo.channels == 0)
			return AVOCADO_STATUS_SUCCESS;
		if (ks == 3 and sizeof(T) <= 4 and fast_paths_enabled())
		{
			const avStatus_t fast = (transformSize == 4) ? launch_f43_input_if<4, T, MT>(ctx, config, geo, xPtr, matricesPtr, deviceStatus, ride, rideTaken) :
					launch_f43_input_if<2, T, MT>(ctx, config, geo, xPtr, matricesPtr, deviceStatus, ride, rideTaken);
			if (fast != AVOCADO_STATUS_NOT_SUPPORTED)
				return fast;
		}
		const CT padding_value = static_cast<CT>(to_compute(config.getPaddingValue<T>()));
		const int vec = pick_vec<T, MT>(geo.channels, sizeof(T) == 8 ? 1 : 2, { xPtr }, { matricesPtr });
		const unsigned int grid = blocks_for(geo.nb_tiles() * (geo.channels / vec));
		DISPATCH_TILE(ks, transformSize,
				DISPATCH_VEC2(vec, kernel_input_transform<TS, KS, T, MT, VEC> <<<grid, kThreads, 0, ctx.getStream()>>>(reinterpret_cast<MT*>(matricesPtr), reinterpret_cast<const T*>(xPtr), geo, padding_value);))
		return checkForErrors();
	}

	template<typename T, typename MT>
	avStatus_t launch_gradient_transform(ContextObject &ctx, const ConvolutionObject &config, const TensorObject &wDesc, const TensorObject &dyDesc,
			const void *dyPtr, const TensorObject &matricesDesc, void *matricesPtr, int transformSize)
	{
		if (dyDesc.nb_dims != 4)
			return AVOCADO_STATUS_BAD_PARAM;
		const int ks = wDesc.dims[1];
		const ConvGeometry geo = make_geometry(dyDesc, transformSize, config);
		if (not matrices_match(matricesDesc, transformSize + ks - 1, geo))
			return AVOCADO_STATUS_BAD_PARAM;
		if (geo.nb_tiles() == 0 or geo.channels == 0)
			return AVOCADO_STATUS_SUCCESS;
		if (ks == 3 and sizeof(T) <= 4 and fast_paths_enabled())
		{
			const avStatus_t fast = (transformSize == 4) ? launch_f43_gradient_if<4, T, MT>(ctx, geo, dyPtr, matricesPtr) :
					launch_f43_gradient_if<2, T, MT>(ctx, geo, dyPtr, matricesPtr);
			if (fast != AVOCADO_STATUS_NOT_SUPPORTED)
				return fast;
		}
		const int vec = pick_vec<T, MT>(geo.channels, sizeof(T) == 8 ? 1 : 2, { dyPtr }, { matricesPtr });
		const unsigned int grid = blocks_for(geo.nb_tiles() * (geo.channels / vec));
		DISPATCH_TILE(ks, transformSize,
				DISPATCH_VEC2(vec, kernel_gradient_transform<TS, KS, T, MT, VEC> <<<grid, kThreads, 0, ctx.getStream()>>>(reinterpret_cast<MT*>(matricesPtr), reinterpret_cast<const T*>(dyPtr), geo);))
		return checkForErrors();
	}

	template<typename T, typename MT, typename BT>
	avStatus_t launch_output_transform(ContextObject &ctx, const ConvolutionObject &config, const TensorObject &wDesc, const void *alpha1,
			const TensorObject &matricesDesc, const void *matricesPtr, const TensorObject &yDesc, void *yPtr, const void *bPtr, const void *alpha2,
			const void *zPtr, const void *beta, avActivationType_t activation, int transformSize)
	{
		using CT = typename ComputeType<T>::type;
		if (yDesc.nb_dims != 4)
			return AVOCADO_STATUS_BAD_PARAM;
		const int ks = wDesc.dims[1];
		const ConvGeometry geo = make_geometry(yDesc, transformSize, config);
		if (not matrices_match(matricesDesc, transformSize + ks - 1, geo))
			return AVOCADO_STATUS_BAD_PARAM;
		if (geo.nb_tiles() == 0 or geo.channels == 0)
			return AVOCADO_STATUS_SUCCESS;
		const CT a1 = getAlphaValue<CT>(alpha1);
		const CT a2 = getAlphaValue<CT>(alpha2);
		const CT b = getBetaValue<CT>(beta);
		if (ks == 3 and sizeof(T) <= 4 and fast_paths_enabled())
		{
			const avStatus_t fast = (transformSize == 4) ? launch_f43_output_if<4, T, MT>(ctx, geo, matricesPtr, yPtr, bPtr, zPtr, a1, a2, b, activation) :
					launch_f43_output_if<2, T, MT>(ctx, geo, matricesPtr, yPtr, bPtr, zPtr, a1, a2, b, activation);
			if (fast != AVOCADO_STATUS_NOT_SUPPORTED)
				return fast;
		}
		const int vec = pick_vec<T, MT>(geo.channels, sizeof(T) == 8 ? 1 : 2, { yPtr, zPtr }, { matricesPtr });
		const unsigned int grid = blocks_for(geo.nb_tiles() * (geo.channels / vec));
		DISPATCH_TILE(ks, transformSize,
				DISPATCH_VEC2(vec, kernel_output_transform<TS, KS, T, MT, BT, VEC> <<<grid, kThreads, 0, ctx.getStream()>>>(reinterpret_cast<const MT*>(matricesPtr), reinterpret_cast<T*>(yPtr), geo, reinterpret_cast<const BT*>(bPtr), reinterpret_cast<const T*>(zPtr), a1, a2, b, activation);))
		return checkForErrors();
	}

	template<typename T>
	avStatus_t launch_update_transform(ContextObject &ctx, const void *alpha, const TensorObject &matricesDesc, const void *matricesPtr, const void *beta,
			const TensorObject &dwDesc, void *dwPtr, int transformSize)
	{
		using CT = typename ComputeType<T>::type;
		const int K = dwDesc.dims[0], ks = dwDesc.dims[1], C = dwDesc.dims[3];
		const int tile = transformSize + ks - 1;
		if (matricesDesc.nb_dims != 3 or matricesDesc.dims[0] != tile * tile or matricesDesc.dims[1] != K or matricesDesc.dims[2] != C)
			return AVOCADO_STATUS_BAD_PARAM;
		if (K == 0 or C == 0)
			return AVOCADO_STATUS_SUCCESS;
		const CT a = getAlphaValue<CT>(alpha);
		const CT b = getBetaValue<CT>(beta);
		const int vec = pick_vec<T, T>(C, sizeof(T) == 8 ? 1 : 2, { dwPtr }, { matricesPtr });
		const unsigned int grid = blocks_for(static_cast<long long>(K) * (C / vec));
		DISPATCH_TILE(ks, transformSize,
				DISPATCH_VEC2(vec, kernel_update_transform<TS, KS, T, VEC> <<<grid, kThreads, 0, ctx.getStream()>>>(reinterpret_cast<const T*>(matricesPtr), reinterpret_cast<T*>(dwPtr), K, C, a, b);))
		return checkForErrors();
	}

	/* which (tensor dtype, matrices dtype) pairs exist: equal types, 16-bit tensors with float32 matrices, and bfloat16
	 * tensors with float16 matrices (the 10-bit mantissa keeps F(2x2,3x3) inside 1e-2 where a bfloat16 domain does not) */
	enum class Pairing
	{
		F16_F16, F16_F32, BF16_BF16, BF16_F16, BF16_F32, F32_F32, F64_F64, Unsupported
	};
	Pairing classify(avDataType_t tensorType, avDataType_t matrixType)
	{
		switch (tensorType)
		{
			case AVOCADO_DTYPE_FLOAT16:
				return matrixType == AVOCADO_DTYPE_FLOAT16 ? Pairing::F16_F16 : matrixType == AVOCADO_DTYPE_FLOAT32 ? Pairing::F16_F32 : Pairing::Unsupported;
			case AVOCADO_DTYPE_BFLOAT16:
				return matrixType == AVOCADO_DTYPE_BFLOAT16 ? Pairing::BF16_BF16 : matrixType == AVOCADO_DTYPE_FLOAT16 ? Pairing::BF16_F16 :
						matrixType == AVOCADO_DTYPE_FLOAT32 ? Pairing::BF16_F32 : Pairing::Unsupported;
			case AVOCADO_DTYPE_FLOAT32:
				return matrixType == AVOCADO_DTYPE_FLOAT32 ? Pairing::F32_F32 : Pairing::Unsupported;
			case AVOCADO_DTYPE_FLOAT64:
				return matrixType == AVOCADO_DTYPE_FLOAT64 ? Pairing::F64_F64 : Pairing::Unsupported;
			default:
				return Pairing::Unsupported;
		}
	}
}

namespace bk
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;

	avStatus_t winograd_weight_transform(ContextObject &ctx, const ConvolutionObject &conv, int transformSize, const TensorObject &w, const void *wPtr, const TensorObject &m, void *mPtr)
	{
		if (not tile_config_supported(w, transformSize))
			return (w.nb_dims != 4) ? AVOCADO_STATUS_BAD_PARAM : AVOCADO_STATUS_NOT_SUPPORTED;
		if (wPtr == nullptr or mPtr == nullptr)
			return AVOCADO_STATUS_BAD_PARAM;
		ctx.setDevice();
		switch (classify(w.dtype, m.dtype))
		{
			case Pairing::F16_F16:
				return launch_weight_transform<half, half>(ctx, conv, w, wPtr, m, mPtr, transformSize);
			case Pairing::F16_F32:
				return launch_weight_transform<half, float>(ctx, conv, w, wPtr, m, mPtr, transformSize);
			case Pairing::BF16_BF16:
				return launch_weight_transform<__nv_bfloat16, __nv_bfloat16>(ctx, conv, w, wPtr, m, mPtr, transformSize);
			case Pairing::BF16_F16:
				return launch_weight_transform<__nv_bfloat16, half>(ctx, conv, w, wPtr, m, mPtr, transformSize);
			case Pairing::BF16_F32:
				return launch_weight_transform<__nv_bfloat16, float>(ctx, conv, w, wPtr, m, mPtr, transformSize);
			case Pairing::F32_F32:
				return launch_weight_transform<float, float>(ctx, conv, w, wPtr, m, mPtr, transformSize);
			case Pairing::F64_F64:
				return launch_weight_transform<double, double>(ctx, conv, w, wPtr, m, mPtr, transformSize);
			default:
				return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
		}
	}

	avStatus_t winograd_input_transform(ContextObject &ctx, const ConvolutionObject &conv, int transformSize, const TensorObject &w, const TensorObject &x, const void *xPtr,
			const TensorObject &m, void *mPtr, int *deviceStatus, const WeightRide *ride, bool *rideTaken)
	{
		if (rideTaken != nullptr)
			rideTaken[0] = false;
		/* the job rides only with a launch of matching types: its tensors have the dtypes of this call's */
		if (ride != nullptr and (ride->weightType != w.dtype or ride->matrixType != m.dtype))
			ride = nullptr;
		if (not tile_config_supported(w, transformSize))
			return (w.nb_dims != 4) ? AVOCADO_STATUS_BAD_PARAM : AVOCADO_STATUS_NOT_SUPPORTED;
		if (xPtr == nullptr or mPtr == nullptr)
			return AVOCADO_STATUS_BAD_PARAM;
		ctx.setDevice();
		/* the reference switches on the dtype of w (src/winograd_nonfused.cu:914); x must agree with it */
		if (x.dtype != w.dtype)
			return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
		switch (classify(w.dtype, m.dtype))
		{
			case Pairing::F16_F16:
				return launch_input_transform<half, half>(ctx, conv, w, x, xPtr, m, mPtr, transformSize, deviceStatus, ride, rideTaken);
			case Pairing::F16_F32:
				return launch_input_transform<half, float>(ctx, conv, w, x, xPtr, m, mPtr, transformSize, deviceStatus, ride, rideTaken);
			case Pairing::BF16_BF16:
				return launch_input_transform<__nv_bfloat16, __nv_bfloat16>(ctx, conv, w, x, xPtr, m, mPtr, transformSize, deviceStatus, ride, rideTaken);
			case Pairing::BF16_F16:
				return launch_input_transform<__nv_bfloat16, half>(ctx, conv, w, x, xPtr, m, mPtr, transformSize, deviceStatus, ride, rideTaken);
			case Pairing::BF16_F32:
				return launch_input_transform<__nv_bfloat16, float>(ctx, conv, w, x, xPtr, m, mPtr, transformSize, deviceStatus, ride, rideTaken);
			case Pairing::F32_F32:
				return launch_input_transform<float, float>(ctx, conv, w, x, xPtr, m, mPtr, transformSize, deviceStatus, ride, rideTaken);
			case Pairing::F64_F64:
				return launch_input_transform<double, double>(ctx, conv, w, x, xPtr, m, mPtr, transformSize, deviceStatus, ride, rideTaken);
			default:
				return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
		}
	}

	avStatus_t flush_deferred_weights(ContextObject &ctx)
	{
		if (not ctx.deferred_weights.valid)
			return AVOCADO_STATUS_SUCCESS;
		const DeferredWeightTransform d = ctx.deferred_weights;
		ctx.deferred_weights.valid = false;
		noteDeferred(-1);
		return winograd_weight_transform(ctx, d.conv, d.transform_size, d.w, d.wPtr, d.u, d.uPtr);
	}

	avStatus_t winograd_output_transform(ContextObject &ctx, const ConvolutionObject &conv, int transformSize, const TensorObject &w, const void *alpha1, const TensorObject &m,
			const void *mPtr, const TensorObject &y, void *yPtr, const void *bPtr, const void *alpha2, const void *zPtr, const void *beta,
			avActivationType_t activation)
	{
		if (not tile_config_supported(w, transformSize))
			return (w.nb_dims != 4) ? AVOCADO_STATUS_BAD_PARAM : AVOCADO_STATUS_NOT_SUPPORTED;
		if (yPtr == nullptr or mPtr == nullptr)
			return AVOCADO_STATUS_BAD_PARAM;
		if (y.dtype != w.dtype)
			return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
		ctx.setDevice();
		switch (classify(w.dtype, m.dtype))
		{
			case Pairing::F16_F16:
				return launch_output_transform<half, half, float>(ctx, conv, w, alpha1, m, mPtr, y, yPtr, bPtr, alpha2, zPtr, beta, activation,
						transformSize);
			case Pairing::F16_F32:
				return launch_output_transform<half, float, float>(ctx, conv, w, alpha1, m, mPtr, y, yPtr, bPtr, alpha2, zPtr, beta, activation,
						transformSize);
			case Pairing::BF16_BF16:
				return launch_output_transform<__nv_bfloat16, __nv_bfloat16, float>(ctx, conv, w, alpha1, m, mPtr, y, yPtr, bPtr, alpha2, zPtr, beta,
						activation, transformSize);
			case Pairing::BF16_F16:
				return launch_output_transform<__nv_bfloat16, half, float>(ctx, conv, w, alpha1, m, mPtr, y, yPtr, bPtr, alpha2, zPtr, beta, activation,
						transformSize);
			case Pairing::BF16_F32:
				return launch_output_transform<__nv_bfloat16, float, float>(ctx, conv, w, alpha1, m, mPtr, y, yPtr, bPtr, alpha2, zPtr, beta, activation,
						transformSize);
			case Pairing::F32_F32:
				return launch_output_transform<float, float, float>(ctx, conv, w, alpha1, m, mPtr, y, yPtr, bPtr, alpha2, zPtr, beta, activation,
						transformSize);
			case Pairing::F64_F64:
				return launch_output_transform<double, double, double>(ctx, conv, w, alpha1, m, mPtr, y, yPtr, bPtr, alpha2, zPtr, beta, activation,
						transformSize);
			default:
				return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
		}
	}
} /* namespace bk */

namespace avocado
{
	namespace backend
	{
		avStatus_t cudaWinogradWeightTransform(avContextDescriptor_t context, const avConvolutionDescriptor_t config, int transformSize,
				const avTensorDescriptor_t wDesc, const avMemoryDescriptor_t wMem, const avTensorDescriptor_t matricesDesc, avMemoryDescriptor_t matricesMem)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				const ConvolutionObject &conv = getConvolution(config);
				const TensorObject &w = getTensor(wDesc);
				const TensorObject &u = getTensor(matricesDesc);
				const void *wPtr = getPointer(wMem);
				void *uPtr = getPointer(matricesMem);
				/* with fusion switched on, a 3x3 weight transform whose arguments are valid is held back: the input transform
				 * that usually follows carries it in its own launch */
				if (ctx.fuse_weights and not ctx.is_default and w.nb_dims == 4 and is_conv(3, w) and (transformSize == 2 or transformSize == 4) and wPtr != nullptr
						and uPtr != nullptr and classify(w.dtype, u.dtype) != Pairing::Unsupported and w.dtype != AVOCADO_DTYPE_FLOAT64 and u.nb_dims == 3
						and u.dims[0] == (transformSize + 2) * (transformSize + 2) and u.dims[1] == w.dims[0] and u.dims[2] == w.dims[3] and w.dims[0] > 0
						and w.dims[3] > 0)
				{
					DeferredWeightTransform &d = ctx.deferred_weights;
					d.valid = true;
					d.conv = conv;
					d.transform_size = transformSize;
					d.w = w;
					d.u = u;
					d.wPtr = wPtr;
					d.uPtr = uPtr;
					noteDeferred(+1);
					return AVOCADO_STATUS_SUCCESS;
				}
				return bk::winograd_weight_transform(ctx, conv, transformSize, w, wPtr, u, uPtr);
			AVOCADO_API_END
		}

		avStatus_t cudaWinogradInputTransform(avContextDescriptor_t context, const avConvolutionDescriptor_t config, int transformSize,
				const avTensorDescriptor_t wDesc, const avTensorDescriptor_t xDesc, const avMemoryDescriptor_t xMem, const avTensorDescriptor_t matricesDesc,
				avMemoryDescriptor_t matricesMem)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContextKeepDeferred(context);
				const ConvolutionObject &conv = getConvolution(config);
				if (ctx.deferred.valid)
				{
					const avStatus_t flushed = bk::flush_deferred_gemm(ctx);
					if (flushed != AVOCADO_STATUS_SUCCESS)
						return flushed;
				}
				if (ctx.deferred_weights.valid)
				{
					/* a weight transform is waiting: offer it to this launch; if the launch cannot carry it, it runs on its own */
					const DeferredWeightTransform d = ctx.deferred_weights;
					ctx.deferred_weights.valid = false;
					noteDeferred(-1);
					bk::WeightRide ride = { d.wPtr, d.uPtr, d.w.dims[0], d.w.dims[3], d.transform_size, d.conv.mode == AVOCADO_CROSS_CORRELATION_MODE, d.w.dtype,
							d.u.dtype };
					bool taken = false;
					const avStatus_t status = bk::winograd_input_transform(ctx, conv, transformSize, getTensor(wDesc), getTensor(xDesc), getPointer(xMem),
							getTensor(matricesDesc), getPointer(matricesMem), nullptr, &ride, &taken);
					if (not taken)
					{
						const avStatus_t weights = bk::winograd_weight_transform(ctx, d.conv, d.transform_size, d.w, d.wPtr, d.u, d.uPtr);
						if (weights != AVOCADO_STATUS_SUCCESS)
							return weights;
					}
					return status;
				}
				return bk::winograd_input_transform(ctx, conv, transformSize, getTensor(wDesc), getTensor(xDesc), getPointer(xMem), getTensor(matricesDesc), getPointer(matricesMem));
			AVOCADO_API_END
		}

		avStatus_t cudaWinogradOutputTransform(avContextDescriptor_t context, const avConvolutionDescriptor_t config, int transformSize,
				const avTensorDescriptor_t wDesc, const void *alpha1, const avTensorDescriptor_t matricesDesc, const avMemoryDescriptor_t matricesMem,
				const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem, const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem,
				const void *alpha2, const avTensorDescriptor_t zDesc, const avMemoryDescriptor_t zMem, const void *beta, avActivationType_t activation)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContextKeepDeferred(context);
				const ConvolutionObject &conv = getConvolution(config);
				(void) bDesc;
				(void) zDesc;
				if (ctx.deferred.valid)
				{
					/* the context is holding back a batched GEMM: if its result is exactly the tensor this call transforms, one
					 * kernel does the contraction and the transform and the products are never written; anything else launches
					 * the GEMM first */
					const DeferredGemm &d = ctx.deferred;
					const TensorObject &w = getTensor(wDesc);
					const TensorObject &m = getTensor(matricesDesc);
					const TensorObject &y = getTensor(yDesc);
					void *yPtr = getPointer(yMem);
					if (transformSize == 4 and w.nb_dims == 4 and is_conv(3, w) and getPointer(matricesMem) == d.cPtr and m.nb_dims == 3 and m.dtype == d.c.dtype
							and m.dims[0] == d.c.dims[0] and m.dims[1] == d.c.dims[1] and m.dims[2] == d.c.dims[2] and y.dtype == w.dtype and yPtr != nullptr
							and (bMem == AVOCADO_INVALID_DESCRIPTOR or getTensor(bDesc).dtype == AVOCADO_DTYPE_FLOAT32))
					{
						const avStatus_t fused = bk::winograd_f43_contract_output(ctx, d.a, d.aPtr, d.b, d.bPtr, y, yPtr, getPointer(bMem), getPointer(zMem),
								alpha1, alpha2, beta, activation, ctx.getDeviceStatus());
						if (fused != AVOCADO_STATUS_NOT_SUPPORTED)
						{
							ctx.deferred.valid = false;
							noteDeferred(-1);
							return fused;
						}
					}
					const avStatus_t flushed = bk::flush_deferred_gemm(ctx);
					if (flushed != AVOCADO_STATUS_SUCCESS)
						return flushed;
				}
				return bk::winograd_output_transform(ctx, conv, transformSize, getTensor(wDesc), alpha1, getTensor(matricesDesc), getPointer(matricesMem), getTensor(yDesc), getPointer(yMem),
						getPointer(bMem), alpha2, getPointer(zMem), beta, activation);
			AVOCADO_API_END
		}

		avStatus_t cudaWinogradGradientTransform(avContextDescriptor_t context, const avConvolutionDescriptor_t config, int transformSize,
				const avTensorDescriptor_t wDesc, const avTensorDescriptor_t dyDesc, const avMemoryDescriptor_t dyMem, const avTensorDescriptor_t matricesDesc,
				avMemoryDescriptor_t matricesMem)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				const ConvolutionObject &conv = getConvolution(config);
				const TensorObject &w = getTensor(wDesc);
				const TensorObject &dy = getTensor(dyDesc);
				const TensorObject &m = getTensor(matricesDesc);
				const void *dyPtr = getPointer(dyMem);
				void *mPtr = getPointer(matricesMem);
				if (not tile_config_supported(w, transformSize))
					return (w.nb_dims != 4) ? AVOCADO_STATUS_BAD_PARAM : AVOCADO_STATUS_NOT_SUPPORTED;
				if (dyPtr == nullptr or mPtr == nullptr)
					return AVOCADO_STATUS_BAD_PARAM;
				if (dy.dtype != w.dtype or m.dtype != w.dtype)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				ctx.setDevice();
				/* float32 and float64 only, as in the reference (src/winograd_nonfused.cu:971-979) */
				switch (w.dtype)
				{
					case AVOCADO_DTYPE_FLOAT32:
						return launch_gradient_transform<float, float>(ctx, conv, w, dy, dyPtr, m, mPtr, transformSize);
					case AVOCADO_DTYPE_FLOAT64:
						return launch_gradient_transform<double, double>(ctx, conv, w, dy, dyPtr, m, mPtr, transformSize);
					default:
						return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				}
			AVOCADO_API_END
		}

		avStatus_t cudaWinogradUpdateTransform(avContextDescriptor_t context, const avConvolutionDescriptor_t config, int transformSize, const void *alpha,
				const avTensorDescriptor_t matricesDesc, const avMemoryDescriptor_t matricesMem, const void *beta, const avTensorDescriptor_t dwDesc,
				avMemoryDescriptor_t dwMem)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				(void) getConvolution(config);
				const TensorObject &m = getTensor(matricesDesc);
				const TensorObject &dw = getTensor(dwDesc);
				const void *mPtr = getPointer(matricesMem);
				void *dwPtr = getPointer(dwMem);
				if (not tile_config_supported(dw, transformSize))
					return (dw.nb_dims != 4) ? AVOCADO_STATUS_BAD_PARAM : AVOCADO_STATUS_NOT_SUPPORTED;
				if (dwPtr == nullptr or mPtr == nullptr)
					return AVOCADO_STATUS_BAD_PARAM;
				if (m.dtype != dw.dtype)
					return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				ctx.setDevice();
				switch (dw.dtype)
				{
					case AVOCADO_DTYPE_FLOAT32:
						return launch_update_transform<float>(ctx, alpha, m, mPtr, beta, dw, dwPtr, transformSize);
					case AVOCADO_DTYPE_FLOAT64:
						return launch_update_transform<double>(ctx, alpha, m, mPtr, beta, dw, dwPtr, transformSize);
					default:
						return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				}
			AVOCADO_API_END
		}
	} /* namespace backend */
} /* namespace avocado */
