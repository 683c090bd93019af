/*
 * Avocado/cuda_backend_ext.h -- additive entry points of the B200 convolution backend.
 *
 * None of these has a counterpart in the reference's include/Avocado/cuda_backend.h; they add what the fixed
 * signatures of that header cannot carry.  No existing signature changes, so a caller that ignores this
 * header keeps working.
 */
#ifndef AVOCADO_CUDA_BACKEND_EXT_H_
#define AVOCADO_CUDA_BACKEND_EXT_H_

#include <Avocado/backend_defs.h>

#ifdef __cplusplus
namespace avocado
{
	namespace backend
	{
		extern "C"
		{
#endif

/* Attaches per-output-channel requantisation scales (float32[K], device memory) to a convolution descriptor.
 * cudaConvolutionImplicitGemmForward uses them when x and w are INT8 and y is INT8:
 *   q[k] = saturate_int8(round_to_nearest_even(activation(alpha1 * float(acc + bias[k]) * scale[k] + alpha2 * z)))
 * Pass AVOCADO_INVALID_DESCRIPTOR to detach.  No counterpart in the reference: its int8 kernel
 * (src/conv2d_implicit_gemm.cu:330-339) has a single scalar alpha and an int32 output only. */
DLL_PUBLIC avStatus_t cudaSetConvolutionQuantization(avConvolutionDescriptor_t desc, const avMemoryDescriptor_t scalesMem);

/* Raw device pointer behind a memory handle, for interoperation with a communication library (the dW
 * all-reduce of the training step).  No counterpart in the reference. */
DLL_PUBLIC avStatus_t cudaGetMemoryPointer(const avMemoryDescriptor_t desc, void **result);

/* cudaStream_t of a context (null for a default context), so a caller can order its own work after the
 * library's.  No counterpart in the reference. */
DLL_PUBLIC avStatus_t cudaGetContextStream(avContextDescriptor_t context, void **result);

/* Waits for the context's stream, then returns and clears the error word that tensor-core kernels set when one
 * of their bounded waits (TMA arrival, MMA completion) gave up: 0 = none.  No counterpart in the reference,
 * whose kernels have no device-side waits. */
DLL_PUBLIC avStatus_t cudaGetLastDeviceStatus(avContextDescriptor_t context, int *result);

/* Records the work that API calls enqueue on a context instead of running it, and replays it later with one launch.
 * Between Begin and End every call on `context` is captured into a CUDA graph; host scalars (alpha, beta) are read at
 * capture time and baked in; the memory handles used must stay alive while the graph exists.  Run the same call
 * sequence once before capturing, so that one-time set-up (kernel attributes, scratch allocation) is already done.
 * The default context cannot capture.  No counterpart in the reference, which launches kernel by kernel. */
DLL_PUBLIC avStatus_t cudaContextBeginCapture(avContextDescriptor_t context);
DLL_PUBLIC avStatus_t cudaContextEndCapture(avContextDescriptor_t context, av_int64 *graph);
DLL_PUBLIC avStatus_t cudaContextLaunchGraph(avContextDescriptor_t context, av_int64 graph);
DLL_PUBLIC avStatus_t cudaDestroyCapturedGraph(av_int64 graph);

#ifdef __cplusplus
		} /* extern "C" */
	} /* namespace backend */
} /* namespace avocado */
#endif

#endif /* AVOCADO_CUDA_BACKEND_EXT_H_ */
