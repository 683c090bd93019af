/*
 * im2row.cu -- cudaIm2Row: the explicit lowering of a convolution to a matrix product.
 *
 * Counterpart of the reference's kernel_im2row_conv2d (src/im2row.cu:29-66) and entry point (:85-125): the input
 * tensor x[N,H,W,C] becomes the matrix rows[N*Ho*Wo, kh*kw*C] whose row for output pixel (n, oh, ow) holds, tap after
 * tap, the C channels of the input pixel that tap covers, so that  rows x w[K, kh*kw*C]^T  is the convolution
 * (cudaGemm with op(B) = T).  Conventions, read off the reference's scatter loop:
 *   - tap (i, j) of CONVOLUTION_MODE reads input pixel (oh + i + padding_h, ow + j + padding_w), padding being the
 *     (negative) offset of the descriptor; CROSS_CORRELATION_MODE stores the taps in the opposite order, i.e. tap
 *     (i, j) reads the pixel of tap (kh-1-i, kw-1-j)
 *   - positions outside the image hold the descriptor's padding value
 *   - the element type matters only through its size: 1, 2, 4, 8 or 16 bytes are moved as opaque words
 *   - Ho = H - 2*padding_h - (kh - 1), Wo likewise (stride 1, no dilation: the reference supports nothing else here)
 *
 * The reference scatters (one thread per input element writes up to kh*kw places); this kernel gathers: one thread per
 * 16 bytes of the OUTPUT, so every store is a full 16-byte, fully coalesced write and every row position is written
 * exactly once (the reference leaves positions it never reaches uninitialised).
 *
 * Bound: HBM, by the kh*kw-fold larger output: algorithmic bytes = (1 + kh*kw) * N*H*W*C*b for "same" padding.
 */
#include <Avocado/cuda_backend.h>

#include "objects.hpp"
#include "device_utils.cuh"

#include "conv_kernels.hpp"

#include <algorithm>
#include <cstring>

namespace
{
	using namespace avocado::backend;
	using namespace avocado::backend::b200;

	struct Im2RowShape
	{
			int batch, height, width; /* input */
			int out_height, out_width;
			int kernel_h, kernel_w;
			int pad_h, pad_w; /* offsets added to the output coordinate (negative = padding) */
			int rotate; /* CROSS_CORRELATION_MODE */
	};

	/* WORD = the unit a thread moves: uint4 when a pixel is a whole number of 16-byte words, else the element itself.
	 * A block walks rows of output pixels (n, oh); inside a row the index is decomposed with two 32-bit divisions, which
	 * is all the integer work there is per 16 bytes moved (a flat 64-bit index costs five 64-bit divisions and made the
	 * kernel instruction-bound at a third of the memory rate). */
	template<typename WORD>
	__global__ void __launch_bounds__(256) kernel_im2row(const WORD *__restrict__ input, WORD *__restrict__ rows, Im2RowShape s, int words_per_pixel, WORD padding,
			int pixel_rows)
	{
		const unsigned int taps = static_cast<unsigned int>(s.kernel_h * s.kernel_w);
		const unsigned int words_per_output_pixel = taps * static_cast<unsigned int>(words_per_pixel);
		const unsigned int words_per_row = static_cast<unsigned int>(s.out_width) * words_per_output_pixel;
		for (int row = blockIdx.x; row < pixel_rows; row += gridDim.x)
		{
			const int n = row / s.out_height;
			const int oh = row - n * s.out_height;
			const WORD *image = input + static_cast<long long>(n) * s.height * s.width * words_per_pixel;
			WORD *dst = rows + static_cast<long long>(row) * words_per_row;
			for (unsigned int e = threadIdx.x; e < words_per_row; e += blockDim.x)
			{
				const unsigned int ow = e / words_per_output_pixel;
				const unsigned int r = e - ow * words_per_output_pixel;
				unsigned int tap = r / static_cast<unsigned int>(words_per_pixel);
				const unsigned int word = r - tap * static_cast<unsigned int>(words_per_pixel);
				if (s.rotate)
					tap = taps - 1 - tap;
				const int ti = static_cast<int>(tap) / s.kernel_w, tj = static_cast<int>(tap) - ti * s.kernel_w;
				const int h = oh + ti + s.pad_h, w = static_cast<int>(ow) + tj + s.pad_w;
				WORD value = padding;
				if (h >= 0 and h < s.height and w >= 0 and w < s.width)
					value = image[(h * s.width + w) * words_per_pixel + static_cast<int>(word)];
				dst[e] = value;
			}
		}
	}

	template<typename WORD>
	avStatus_t launch(ContextObject &ctx, const void *input, void *rows, const Im2RowShape &s, int words_per_pixel, const uint8_t (&padding_bytes)[16],
			int element_size)
	{
		/* the padding word: the element's padding value repeated to fill the word */
		WORD padding;
		uint8_t pattern[sizeof(WORD)];
		for (size_t i = 0; i < sizeof(WORD); i++)
			pattern[i] = padding_bytes[i % element_size];
		std::memcpy(&padding, pattern, sizeof(WORD));
		const long long pixel_rows = static_cast<long long>(s.batch) * s.out_height;
		const long long words_per_row = static_cast<long long>(s.out_width) * s.kernel_h * s.kernel_w * words_per_pixel;
		if (pixel_rows == 0 or words_per_row == 0)
			return AVOCADO_STATUS_SUCCESS;
		/* one image and one row of output pixels are indexed with 32-bit integers */
		if (pixel_rows > 0x7FFFFFFFll or words_per_row > 0x7FFFFFFFll or static_cast<long long>(s.height) * s.width * words_per_pixel > 0x7FFFFFFFll)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		int sms = 148;
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device);
		const int grid = static_cast<int>(std::min<long long>(pixel_rows, static_cast<long long>(sms) * 8));
		kernel_im2row<WORD> <<<grid, 256, 0, ctx.getStream()>>>(reinterpret_cast<const WORD*>(input), reinterpret_cast<WORD*>(rows), s, words_per_pixel, padding,
				static_cast<int>(pixel_rows));
		return checkForErrors();
	}
}

namespace bk
{
	avStatus_t im2row_words(ContextObject &ctx, const void *input, void *rows, int batch, int height, int width, int outHeight, int outWidth, int kernelH,
			int kernelW, int padH, int padW, bool rotate, long long pixelBytes)
	{
		Im2RowShape s;
		s.batch = batch;
		s.height = height;
		s.width = width;
		s.out_height = outHeight;
		s.out_width = outWidth;
		s.kernel_h = kernelH;
		s.kernel_w = kernelW;
		s.pad_h = padH;
		s.pad_w = padW;
		s.rotate = rotate ? 1 : 0;
		const uint8_t zero_padding[16] = { };
		if (pixelBytes % 16 != 0 or pixelBytes > 0x7FFFFFFFll or reinterpret_cast<uintptr_t>(input) % 16 != 0 or reinterpret_cast<uintptr_t>(rows) % 16 != 0)
			return AVOCADO_STATUS_NOT_SUPPORTED;
		ctx.setDevice();
		return launch<uint4>(ctx, input, rows, s, static_cast<int>(pixelBytes / 16), zero_padding, 4);
	}
} /* namespace bk */

namespace avocado
{
	namespace backend
	{
		avStatus_t cudaIm2Row(avContextDescriptor_t context, const avConvolutionDescriptor_t config, const avTensorDescriptor_t filterDesc,
				const avTensorDescriptor_t srcDesc, const avMemoryDescriptor_t srcMem, const avTensorDescriptor_t rowDesc, avMemoryDescriptor_t rowMem)
		{
			AVOCADO_API_BEGIN
				ContextObject &ctx = getContext(context);
				const ConvolutionObject &conv = getConvolution(config);
				const TensorObject &filter = getTensor(filterDesc);
				const TensorObject &src = getTensor(srcDesc);
				const TensorObject &row = getTensor(rowDesc);
				const void *src_ptr = getPointer(srcMem);
				void *row_ptr = getPointer(rowMem);
				if (src.nb_dims != 4 or filter.nb_dims != 4 or src_ptr == nullptr or row_ptr == nullptr)
					return AVOCADO_STATUS_BAD_PARAM;
				if (filter.dims[3] != src.dims[3] or row.dtype != src.dtype)
					return AVOCADO_STATUS_BAD_PARAM;
				if (conv.strides[0] != 1 or conv.strides[1] != 1 or conv.dilation[0] != 1 or conv.dilation[1] != 1 or conv.groups != 1)
					return AVOCADO_STATUS_NOT_SUPPORTED;

				Im2RowShape s;
				s.batch = src.dims[0];
				s.height = src.dims[1];
				s.width = src.dims[2];
				s.kernel_h = filter.dims[1];
				s.kernel_w = filter.dims[2];
				s.pad_h = conv.padding[0];
				s.pad_w = conv.padding[1];
				s.out_height = s.height - 2 * s.pad_h - (s.kernel_h - 1);
				s.out_width = s.width - 2 * s.pad_w - (s.kernel_w - 1);
				s.rotate = (conv.mode == AVOCADO_CROSS_CORRELATION_MODE) ? 1 : 0;
				if (s.out_height < 0 or s.out_width < 0 or s.kernel_h < 1 or s.kernel_w < 1)
					return AVOCADO_STATUS_BAD_PARAM;
				const int element_size = static_cast<int>(dtype_size(src.dtype));
				const long long channels = src.dims[3];
				const long long expected = static_cast<long long>(s.batch) * s.out_height * s.out_width * s.kernel_h * s.kernel_w * channels;
				if (row.volume() != expected)
					return AVOCADO_STATUS_BAD_PARAM;
				const long long pixel_bytes = channels * element_size;
				if (pixel_bytes > 0x7FFFFFFFll)
					return AVOCADO_STATUS_NOT_SUPPORTED;
				ctx.setDevice();

				const bool aligned = (pixel_bytes % 16 == 0) and (reinterpret_cast<uintptr_t>(src_ptr) % 16 == 0) and (reinterpret_cast<uintptr_t>(row_ptr) % 16 == 0);
				if (aligned)
					return launch<uint4>(ctx, src_ptr, row_ptr, s, static_cast<int>(pixel_bytes / 16), conv.padding_value, element_size);
				switch (element_size)
				{
					case 1:
						return launch<uint8_t>(ctx, src_ptr, row_ptr, s, static_cast<int>(channels), conv.padding_value, element_size);
					case 2:
						return launch<uint16_t>(ctx, src_ptr, row_ptr, s, static_cast<int>(channels), conv.padding_value, element_size);
					case 4:
						return launch<uint32_t>(ctx, src_ptr, row_ptr, s, static_cast<int>(channels), conv.padding_value, element_size);
					case 8:
						return launch<uint2>(ctx, src_ptr, row_ptr, s, static_cast<int>(channels), conv.padding_value, element_size);
					default:
						return AVOCADO_STATUS_UNSUPPORTED_DATATYPE;
				}
			AVOCADO_API_END
		}
	} /* namespace backend */
} /* namespace avocado */
