#include "conv_kernels.hpp"
namespace bk
{
	avocado::backend::avStatus_t launch_implicit_gemm_tc(avocado::backend::b200::ContextObject &, const ConvArgs &, avocado::backend::avDataType_t,
			avocado::backend::avDataType_t, const void *, const void *, const void *)
	{
		return avocado::backend::AVOCADO_STATUS_NOT_SUPPORTED;
	}
}
