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

/* Failure-detection self test: launches one small kernel that waits, with a limit of `limitMicroseconds`, on a barrier
 * nobody will ever signal.  The wait must run out, the kernel must return normally, bit 5 of the context's device status
 * word must be set (read it with cudaGetLastDeviceStatus) and the context must stay usable.  This exercises, without
 * faulting or hanging the GPU, the path every tensor-core kernel takes when one of its waits gives up.
 * No counterpart in the reference. */
DLL_PUBLIC avStatus_t cudaRunBoundedWaitSelfTest(avContextDescriptor_t context, int limitMicroseconds);

/* The same self test with the kernel pointed at the error word of cudaConvolutionWinogradFusedForwardNoAlloc's fixed
 * array on the context's device (shared by all contexts of that device) instead of the context's own word: the report
 * must surface through cudaGetLastDeviceStatus all the same.  Returns AVOCADO_STATUS_BAD_PARAM while no call of that
 * entry point has been made on the device.  No counterpart in the reference. */
DLL_PUBLIC avStatus_t cudaRunBoundedWaitSelfTestNoAlloc(avContextDescriptor_t context, int limitMicroseconds);

/* Switches fusion inside the non-fused Winograd pipeline on or off for one context; `flags` is 0 or a combination of the
 * two values below.  The call sequence of the reference stays as it is (ref app/CudaBackend.cu:401-420: weight transform,
 * input transform, cudaGemmBatched, cudaWinogradOutputTransform); what changes is how many kernels it becomes.
 *
 * AVOCADO_WINOGRAD_FUSE_WEIGHTS: a cudaWinogradWeightTransform of a 3x3 kernel is held back and rides along in the launch
 *   of the cudaWinogradInputTransform that follows it (a few blocks at the front of that grid).  Its result is written as
 *   usual, bit for bit; only the separate launch, a few microseconds of latency for 74 KB of weights, disappears.
 * AVOCADO_WINOGRAD_FUSE_OUTPUT: a cudaGemmBatched call that is the contraction of an F(4x4,3x3) pipeline (36 planes, (N, T),
 *   float16 / bfloat16, alpha 1, beta 0) is held back; if the next call on the context is the cudaWinogradOutputTransform
 *   of exactly the tensor it was to write, ONE kernel contracts and transforms and the transform-domain products are
 *   NEVER WRITTEN to the caller's workspace -- the workspace keeps whatever it held.  That is the one observable
 *   difference, and the reason fusion is opt-in.
 *
 * Any other call on the context (another operator, a copy, a synchronisation, the end of a capture, destruction of the
 * context or of any memory descriptor) launches what was held back first, in the order it was asked for, so nothing
 * else can tell that it was deferred.  Default contexts cannot fuse.  No counterpart in the reference, whose calls always
 * run as one kernel each (src/winograd_nonfused.cu:608-651, src/gemm.cpp:126-209, src/winograd_nonfused.cu:703-777). */
#define AVOCADO_WINOGRAD_FUSE_WEIGHTS 1
#define AVOCADO_WINOGRAD_FUSE_OUTPUT 2
DLL_PUBLIC avStatus_t cudaContextSetWinogradFusion(avContextDescriptor_t context, int flags);

/* Orders two contexts on the device without blocking the host: everything enqueued on `waiting` after this call runs
 * after everything enqueued on `signalling` before it.  The reference has only cudaSynchronizeWithContext, which blocks
 * the calling thread; with this a caller can run independent steps on two contexts (for instance the weight transform
 * next to the input transform of the same layer) and join them.  Inside a capture (below) the second context's work
 * becomes a parallel branch of the captured graph: let it wait for the capturing context first, and let the capturing
 * context wait for it before the capture ends.  No counterpart in the reference. */
DLL_PUBLIC avStatus_t cudaContextWaitForContext(avContextDescriptor_t waiting, avContextDescriptor_t signalling);

/* Records the work that API calls enqueue on a context instead of running it, and replays it later with one launch.
 * Between Begin and End every call on `context` is captured into a CUDA graph; host scalars (alpha, beta) are read at
 * capture time and baked in; the memory handles used must stay alive while the graph exists.  Run the same call
 * sequence once before capturing, so that one-time set-up (kernel attributes, scratch allocation) is already done.
 * The default context cannot capture.  No counterpart in the reference, which launches kernel by kernel. */
DLL_PUBLIC avStatus_t cudaContextBeginCapture(avContextDescriptor_t context);
DLL_PUBLIC avStatus_t cudaContextEndCapture(avContextDescriptor_t context, av_int64 *graph);
DLL_PUBLIC avStatus_t cudaContextLaunchGraph(avContextDescriptor_t context, av_int64 graph);
DLL_PUBLIC avStatus_t cudaDestroyCapturedGraph(av_int64 graph);

/* Size of the fixed scratch array behind cudaConvolutionWinogradFusedForwardNoAlloc.  Every GPU on which the library's
 * device code is loaded holds this much device memory (plus 256 bytes) until the process exits. */
#define AVOCADO_NO_ALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)

/* cudaConvolutionWinogradFusedForward for callers that may not cause a device allocation -- a host that has given
 * all GPU memory to its own pool, a latency-bound loop that cannot absorb the synchronisation cudaMalloc implies, a
 * process under a no-allocation-after-start-up rule.  Same arguments and same result, but the transform-domain
 * tensors live in a fixed array inside the library image instead of the context's cudaMalloc'ed scratch, and nothing
 * on this path allocates or frees.  It has no counterpart in the reference (whose fused entry point takes no
 * workspace and allocates none because it was never finished).
 *  - float16 / bfloat16 tensors, 3x3 kernel, unit stride and dilation, C and K multiples of 8, y the size of x;
 *    anything else returns UNSUPPORTED_DATATYPE / NOT_SUPPORTED.
 *  - 32 * (K*C + tiles*C) bytes, tiles = N*ceil(H/2)*ceil(W/2), must fit AVOCADO_NO_ALLOC_SCRATCH_BYTES (plus
 *    32 * tiles*K when y, z or the bias is not 16 / 16 / 4-byte aligned, because the products are then written out);
 *    a larger problem returns AVOCADO_STATUS_BAD_PARAM and launches nothing.
 *  - The first call on a device resolves the array's device address and, with the runtime's lazy loading, is when the
 *    driver places the array and the kernels on the device: make it at start-up, before the host's own pool takes the
 *    remaining memory and before any stream capture.
 *  - All calls on one device share the array: calls that overlap on the GPU race.  It keeps the last call's contents;
 *    the only part that must start at zero, the kernels' 256-byte error word, starts as zero and is cleared when
 *    cudaGetLastDeviceStatus (of any context on the device) reads it, so a report is never lost. */
DLL_PUBLIC avStatus_t cudaConvolutionWinogradFusedForwardNoAlloc(avContextDescriptor_t context, const avConvolutionDescriptor_t config, const void *alpha1,
		const avTensorDescriptor_t xDesc, const avMemoryDescriptor_t xMem, const avTensorDescriptor_t wDesc, const avMemoryDescriptor_t wMem,
		const avTensorDescriptor_t bDesc, const avMemoryDescriptor_t bMem, const void *alpha2, const avTensorDescriptor_t zDesc,
		const avMemoryDescriptor_t zMem, const void *beta, const avTensorDescriptor_t yDesc, avMemoryDescriptor_t yMem, avActivationType_t activation);

#ifdef __cplusplus
		} /* extern "C" */
	} /* namespace backend */
} /* namespace avocado */
#endif

#endif /* AVOCADO_CUDA_BACKEND_EXT_H_ */
