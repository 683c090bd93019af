"""The chains of C-API calls that make up one convolution, as a caller of the library issues them.

The reference has no driver for its non-fused Winograd path other than a commented-out scratch function
(app/CudaBackend.cu:345-443: weight transform -> input transform -> cudaGemmBatched(N, T) -> output transform);
the backward chains follow from its kernels (src/winograd_nonfused.cu:424-521, :616):

  forward   U = weight_transform(w);   V = input_transform(x);   M = V x U^T;   y = output_transform(M)
  dX        U' = weight_transform(w, rotated); V' = input_transform(dy); M' = V' x U'; dx = output_transform(M')
  dW        V = input_transform(x);  G = gradient_transform(dy);  Mw = G^T x V;  dw = update_transform(Mw)

Everything here is host-side bookkeeping around calls into libAvocadoCudaBackend.so; the workspaces are owned by the
caller, as the C API requires.
"""
import ctypes

from . import api

_VP = ctypes.c_void_p


def tiles(n, h, w, transform_size):
    return n * ((h + transform_size - 1) // transform_size) * ((w + transform_size - 1) // transform_size)


class WinogradNonFused:
    """Workspaces and call sequence of the non-fused Winograd convolution for one layer shape.

    `dtype` is the dtype of x, w and y; `matrices_dtype` is the dtype of the transform-domain tensors (equal to
    `dtype`, or "float32" with 16-bit tensors).
    """

    def __init__(self, ctx, n, h, w, c, k, dtype, matrices_dtype=None, transform_size=4, kernel_size=3, padding=None, device=0, training=False,
                 side_ctx=None):
        self.ctx = ctx
        # optional second context: the weight transform depends on nothing the input transform touches, so forward() issues
        # it there and joins before the contraction (a parallel branch when the step is captured into a graph)
        self.side_ctx = side_ctx
        self.n, self.h, self.w, self.c, self.k = n, h, w, c, k
        self.ts, self.ks = transform_size, kernel_size
        self.dtype = dtype
        self.mdtype = matrices_dtype or dtype
        pad = -(kernel_size // 2) if padding is None else padding
        self.padding = (pad, pad)
        self.conv = api.ConvolutionDescriptor(api.CONVOLUTION_MODE, self.padding)
        self.conv_rotated = api.ConvolutionDescriptor(api.CROSS_CORRELATION_MODE, self.padding)
        tile = transform_size + kernel_size - 1
        self.planes = tile * tile
        self.nb_tiles = tiles(n, h, w, transform_size)
        self.x = api.DeviceTensor((n, h, w, c), dtype, device)
        self.wt = api.DeviceTensor((k, kernel_size, kernel_size, c), dtype, device)
        self.y = api.DeviceTensor((n, h, w, k), dtype, device)
        self.u = api.DeviceTensor((self.planes, k, c), self.mdtype, device)
        self.v = api.DeviceTensor((self.planes, self.nb_tiles, c), self.mdtype, device)
        self.m = api.DeviceTensor((self.planes, self.nb_tiles, k), self.mdtype, device)
        self.bias = None
        self.z = None
        if training:
            self.dy = api.DeviceTensor((n, h, w, k), dtype, device)
            self.dx = api.DeviceTensor((n, h, w, c), dtype, device)
            self.dw = api.DeviceTensor((k, kernel_size, kernel_size, c), dtype, device)
            self.g = api.DeviceTensor((self.planes, self.nb_tiles, k), self.mdtype, device)
            self.mw = api.DeviceTensor((self.planes, k, c), self.mdtype, device)

    def set_bias(self, values):
        bias_dtype = "float64" if self.dtype == "float64" else "float32"
        self.bias = api.DeviceTensor((self.k,), bias_dtype, self.x.mem.device)
        return self.bias.upload(self.ctx, values)

    def set_z(self, values):
        self.z = api.DeviceTensor((self.n, self.h, self.w, self.k), self.dtype, self.x.mem.device)
        return self.z.upload(self.ctx, values)

    def enable_fusion(self, flags=True):
        """Switches the context's Winograd fusion (api.FUSE_WEIGHTS, api.FUSE_OUTPUT, both with True, none with False / 0)."""
        self.ctx.set_winograd_fusion(flags)

    # ---- individual stages --------------------------------------------------------------------------------
    def weight_transform(self, rotated=False, ctx=None):
        conv = self.conv_rotated if rotated else self.conv
        api.call("cudaWinogradWeightTransform", (ctx or self.ctx).handle, conv.handle, self.ts, self.wt.desc.handle, self.wt.mem.handle, self.u.desc.handle,
                 self.u.mem.handle)

    def input_transform(self, source=None, dest=None):
        source = source or self.x
        dest = dest or self.v
        api.call("cudaWinogradInputTransform", self.ctx.handle, self.conv.handle, self.ts, self.wt.desc.handle, source.desc.handle, source.mem.handle,
                 dest.desc.handle, dest.mem.handle)

    def gemm(self, a, b, c, trans_a=False, trans_b=True):
        api.call("cudaGemmBatched", self.ctx.handle, api.GEMM_T if trans_a else api.GEMM_N, api.GEMM_T if trans_b else api.GEMM_N, None, a.desc.handle,
                 a.mem.handle, b.desc.handle, b.mem.handle, None, c.desc.handle, c.mem.handle)

    def output_transform(self, matrices=None, dest=None, alpha1=None, alpha2=None, beta=None, activation="linear", use_bias=True, use_z=True):
        matrices = matrices or self.m
        dest = dest or self.y
        a1, k1 = api.scalar_pointer(alpha1, self.dtype)
        a2, k2 = api.scalar_pointer(alpha2, self.dtype)
        b, k3 = api.scalar_pointer(beta, self.dtype)
        bias = self.bias if use_bias else None
        z = self.z if use_z else None
        api.call("cudaWinogradOutputTransform", self.ctx.handle, self.conv.handle, self.ts, self.wt.desc.handle, a1, matrices.desc.handle,
                 matrices.mem.handle, dest.desc.handle, dest.mem.handle, bias.desc.handle if bias else api.INVALID,
                 bias.mem.handle if bias else api.INVALID, a2, z.desc.handle if z else api.INVALID, z.mem.handle if z else api.INVALID, b,
                 api.ACTIVATIONS[activation])
        del k1, k2, k3

    def gradient_transform(self):
        api.call("cudaWinogradGradientTransform", self.ctx.handle, self.conv.handle, self.ts, self.wt.desc.handle, self.dy.desc.handle,
                 self.dy.mem.handle, self.g.desc.handle, self.g.mem.handle)

    def update_transform(self, alpha=None, beta=None):
        a, k1 = api.scalar_pointer(alpha, self.dtype)
        b, k2 = api.scalar_pointer(beta, self.dtype)
        api.call("cudaWinogradUpdateTransform", self.ctx.handle, self.conv.handle, self.ts, a, self.mw.desc.handle, self.mw.mem.handle, b,
                 self.dw.desc.handle, self.dw.mem.handle)
        del k1, k2

    # ---- whole passes ------------------------------------------------------------------------------------
    def forward(self, activation="linear", transform_weights=True):
        side = self.side_ctx if transform_weights else None
        if side is not None:
            side.wait_for(self.ctx)                  # U may still be read by this context's previous contraction
            self.weight_transform(ctx=side)
        elif transform_weights:
            self.weight_transform()
        self.input_transform()
        if side is not None:
            self.ctx.wait_for(side)
        self.gemm(self.v, self.u, self.m, False, True)
        self.output_transform(activation=activation)

    def backward_data(self):
        """dx from dy: the forward chain run on dy with the 180-degree rotated kernel and a (N, N) contraction."""
        self.weight_transform(rotated=True)
        self.input_transform(self.dy, self.g)          # [planes, tiles, K]
        self.gemm(self.g, self.u, self.v, False, False)  # [planes, tiles, K] x [planes, K, C] -> [planes, tiles, C]
        self.output_transform(self.v, self.dx, use_bias=False, use_z=False)

    def backward_weights(self, reuse_v=False):
        """dw from x and dy: input transform of x, gradient transform of dy, (T, N) contraction over the tiles, update transform.

        reuse_v=True skips the input transform: V still holds the transform of x that forward() wrote (nothing in between
        may have overwritten it -- backward_data() does)."""
        if not reuse_v:
            self.input_transform()
        self.gradient_transform()
        self.gemm(self.g, self.v, self.mw, True, False)  # [planes, tiles, K]^T x [planes, tiles, C] -> [planes, K, C]
        self.update_transform()

    def training_step(self):
        """forward, dW, dX.  dW runs right after the forward pass so that it can take V = input transform(x) from it
        instead of recomputing it; dX comes last because its contraction writes its result into the V workspace."""
        self.forward()
        self.backward_weights(reuse_v=True)
        self.backward_data()


class DirectConvolution:
    """One-call convolutions: cudaConvolutionWinogradFusedForward / cudaConvolutionImplicitGemmForward."""

    def __init__(self, ctx, n, h, w, c, k, dtype, out_dtype=None, kernel_size=3, device=0, bias_dtype=None):
        self.ctx = ctx
        self.dtype = dtype
        self.out_dtype = out_dtype or dtype
        pad = -(kernel_size // 2)
        self.conv = api.ConvolutionDescriptor(api.CONVOLUTION_MODE, (pad, pad))
        self.x = api.DeviceTensor((n, h, w, c), dtype, device)
        self.wt = api.DeviceTensor((k, kernel_size, kernel_size, c), dtype, device)
        self.y = api.DeviceTensor((n, h, w, k), self.out_dtype, device)
        self.bias_dtype = bias_dtype or ("int32" if dtype == "int8" else "float64" if dtype == "float64" else "float32")
        self.bias = None
        self.z = None
        self.scales = None
        self.k = k
        self.device = device

    def set_bias(self, values):
        self.bias = api.DeviceTensor((self.k,), self.bias_dtype, self.device)
        return self.bias.upload(self.ctx, values)

    def set_z(self, values):
        self.z = api.DeviceTensor(self.y.shape, self.out_dtype, self.device)
        return self.z.upload(self.ctx, values)

    def set_scales(self, values):
        self.scales = api.DeviceTensor((self.k,), "float32", self.device)
        stored = self.scales.upload(self.ctx, values)
        self.conv.set_quantization(self.scales.mem)
        return stored

    def _run(self, entry, alpha1, alpha2, beta, activation):
        scalar_dtype = "float64" if self.dtype == "float64" else "float32"
        a1, k1 = api.scalar_pointer(alpha1, scalar_dtype)
        a2, k2 = api.scalar_pointer(alpha2, scalar_dtype)
        b, k3 = api.scalar_pointer(beta, scalar_dtype)
        bias, z = self.bias, self.z
        api.call(entry, self.ctx.handle, self.conv.handle, a1, self.x.desc.handle, self.x.mem.handle, self.wt.desc.handle, self.wt.mem.handle,
                 bias.desc.handle if bias else api.INVALID, bias.mem.handle if bias else api.INVALID, a2, z.desc.handle if z else api.INVALID,
                 z.mem.handle if z else api.INVALID, b, self.y.desc.handle, self.y.mem.handle, api.ACTIVATIONS[activation])
        del k1, k2, k3

    def winograd_fused(self, alpha1=None, alpha2=None, beta=None, activation="linear"):
        self._run("cudaConvolutionWinogradFusedForward", alpha1, alpha2, beta, activation)

    def winograd_fused_no_alloc(self, alpha1=None, alpha2=None, beta=None, activation="linear"):
        """Same convolution through the entry point that keeps its scratch in a fixed array inside the library."""
        self._run("cudaConvolutionWinogradFusedForwardNoAlloc", alpha1, alpha2, beta, activation)

    def implicit_gemm(self, alpha1=None, alpha2=None, beta=None, activation="linear"):
        self._run("cudaConvolutionImplicitGemmForward", alpha1, alpha2, beta, activation)
