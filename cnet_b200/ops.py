"""Direct calls of the C-ABI operators (include/cnet_b200.h) on torch CUDA tensors.

torch only owns the memory and the stream; every operator below is one call into
libcnet_b200.so.  Complex tensors are (re, im) pairs of contiguous float32 tensors.
"""
import ctypes as C

from . import lib as _lib


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class Context:
    """cnb_create: a device arena for scratch, twiddles and GEMM staging."""

    def __init__(self, device=0, arena_bytes=256 << 20):
        import torch
        if not torch.cuda.is_available():
            raise _lib.CnetError("no CUDA device: the path has no CPU fallback")
        self.lib = _lib.load()
        self.torch = torch
        self.h = C.c_void_p()
        _lib.check(self.lib.cnb_create(device, arena_bytes, C.byref(self.h)), "cnb_create")

    def close(self):
        if self.h:
            self.lib.cnb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def _new(self, *shape):
        return (self.torch.empty(*shape, dtype=self.torch.float32, device="cuda"),
                self.torch.empty(*shape, dtype=self.torch.float32, device="cuda"))

    # ------------------------------------------------------------------ Linear
    def linear_fwd(self, x, w, res=None):
        B, n_in = x[0].shape
        n_out = w[0].shape[0]
        y = self._new(B, n_out)
        _lib.check(self.lib.cnb_linear_fwd(self.h, _p(x[0]), _p(x[1]), _p(w[0]), _p(w[1]),
                                           _p(res[0]) if res else None, _p(res[1]) if res else None,
                                           _p(y[0]), _p(y[1]), B, n_in, n_out, self._stream()), "linear_fwd")
        return y

    def linear_bwd_x(self, g, w, out=None):
        B, n_out = g[0].shape
        n_in = w[0].shape[1]
        acc = 1 if out is not None else 0
        dx = out if out is not None else self._new(B, n_in)
        _lib.check(self.lib.cnb_linear_bwd_x(self.h, _p(g[0]), _p(g[1]), _p(w[0]), _p(w[1]), _p(dx[0]), _p(dx[1]),
                                             B, n_in, n_out, acc, self._stream()), "linear_bwd_x")
        return dx

    def linear_bwd_w(self, g, x, out=None):
        B, n_out = g[0].shape
        n_in = x[0].shape[1]
        acc = 1 if out is not None else 0
        dw = out if out is not None else self._new(n_out, n_in)
        _lib.check(self.lib.cnb_linear_bwd_w(self.h, _p(g[0]), _p(g[1]), _p(x[0]), _p(x[1]), _p(dw[0]), _p(dw[1]),
                                             B, n_in, n_out, acc, self._stream()), "linear_bwd_w")
        return dw

    # operands split once (fp32 hi, bf16 hi and lo) and reused by several products
    def split(self, x):
        n = x[0].numel()
        out = self.torch.empty(self.lib.cnb_split_floats(n), dtype=self.torch.float32, device="cuda")
        _lib.check(self.lib.cnb_split_planes(self.h, _p(x[0]), _p(x[1]), n, _p(out), self._stream()), "split_planes")
        return out

    def linear_fwd_split(self, x_split, w_split, B, n_in, n_out, res=None, out=None):
        y = out if out is not None else self._new(B, n_out)
        _lib.check(self.lib.cnb_linear_fwd_split(self.h, _p(x_split), _p(w_split), _p(res[0]) if res else None,
                                                 _p(res[1]) if res else None, _p(y[0]), _p(y[1]), B, n_in, n_out,
                                                 self._stream()), "linear_fwd_split")
        return y

    def linear_bwd_x_split(self, g_split, w_split, B, n_in, n_out, out=None, accumulate=False):
        dx = out if out is not None else self._new(B, n_in)
        _lib.check(self.lib.cnb_linear_bwd_x_split(self.h, _p(g_split), _p(w_split), _p(dx[0]), _p(dx[1]), B, n_in,
                                                   n_out, int(accumulate), self._stream()), "linear_bwd_x_split")
        return dx

    def linear_bwd_w_split(self, g_split, x_split, B, n_in, n_out, out=None, accumulate=False):
        dw = out if out is not None else self._new(n_out, n_in)
        _lib.check(self.lib.cnb_linear_bwd_w_split(self.h, _p(g_split), _p(x_split), _p(dw[0]), _p(dw[1]), B, n_in,
                                                   n_out, int(accumulate), self._stream()), "linear_bwd_w_split")
        return dw

    def last_gemm_engine(self):
        return self.lib.cnb_last_gemm_engine()

    # ------------------------------------------------------------ FourierTrans
    def dft_fwd(self, x):
        B, N = x[0].shape
        y = self._new(B, N)
        _lib.check(self.lib.cnb_dft_fwd(self.h, _p(x[0]), _p(x[1]), _p(y[0]), _p(y[1]), B, N, self._stream()), "dft_fwd")
        return y

    def dft_bwd(self, g, out=None):
        B, N = g[0].shape
        acc = 1 if out is not None else 0
        dx = out if out is not None else self._new(B, N)
        _lib.check(self.lib.cnb_dft_bwd(self.h, _p(g[0]), _p(g[1]), _p(dx[0]), _p(dx[1]), B, N, acc, self._stream()),
                   "dft_bwd")
        return dx

    def dft_hadamard_gelu_fwd(self, x, h, u=None, split=None):
        """FourierTrans forward with the Hadamard(h) -> CGelu tail in the same kernel: u = FFT(x) and the operand
        split of y = gelu(u o h) (y itself is not stored).  Returns (u, split)."""
        B, N = x[0].shape
        u = u if u is not None else self._new(B, N)
        if split is None:
            split = self.torch.empty(self.lib.cnb_split_floats(B * N), dtype=self.torch.float32, device="cuda")
        _lib.check(self.lib.cnb_dft_hadamard_gelu_fwd(self.h, _p(x[0]), _p(x[1]), _p(h[0]), _p(h[1]), _p(u[0]), _p(u[1]),
                                                      None, None, _p(split), B, N, self._stream()), "dft_hadamard_gelu_fwd")
        return u, split

    # ------------------------------------------------------------ element-wise
    def hadamard_fwd(self, u, v):
        B, N = u[0].shape
        y = self._new(B, N)
        _lib.check(self.lib.cnb_hadamard_fwd(self.h, _p(u[0]), _p(u[1]), _p(v[0]), _p(v[1]), int(v[0].dim() == 2),
                                             _p(y[0]), _p(y[1]), B, N, self._stream()), "hadamard_fwd")
        return y

    def hadamard_bwd(self, g, u, v):
        B, N = u[0].shape
        du = self._new(B, N)
        dv = self._new(*v[0].shape)
        _lib.check(self.lib.cnb_hadamard_bwd(self.h, _p(g[0]), _p(g[1]), _p(u[0]), _p(u[1]), _p(v[0]), _p(v[1]),
                                             int(v[0].dim() == 2), _p(du[0]), _p(du[1]), 0, _p(dv[0]), _p(dv[1]), 0,
                                             B, N, self._stream()), "hadamard_bwd")
        return du, dv

    def gelu_fwd(self, z):
        y = self._new(*z[0].shape)
        _lib.check(self.lib.cnb_gelu_fwd(self.h, _p(z[0]), _p(z[1]), _p(y[0]), _p(y[1]), z[0].numel(), self._stream()),
                   "gelu_fwd")
        return y

    def gelu_bwd(self, g, z):
        d = self._new(*z[0].shape)
        _lib.check(self.lib.cnb_gelu_bwd(self.h, _p(g[0]), _p(g[1]), _p(z[0]), _p(z[1]), _p(d[0]), _p(d[1]),
                                         z[0].numel(), 0, self._stream()), "gelu_bwd")
        return d

    def hadamard_gelu_fwd(self, u, h):
        B, N = u[0].shape
        a, y = self._new(B, N), self._new(B, N)
        _lib.check(self.lib.cnb_hadamard_gelu_fwd(self.h, _p(u[0]), _p(u[1]), _p(h[0]), _p(h[1]), _p(a[0]), _p(a[1]),
                                                  _p(y[0]), _p(y[1]), B, N, self._stream()), "hadamard_gelu_fwd")
        return a, y

    def hadamard_gelu_bwd(self, g, a, u, h):
        B, N = u[0].shape
        du, dh = self._new(B, N), self._new(N)
        _lib.check(self.lib.cnb_hadamard_gelu_bwd(self.h, _p(g[0]), _p(g[1]), _p(a[0]), _p(a[1]), _p(u[0]), _p(u[1]),
                                                  _p(h[0]), _p(h[1]), _p(du[0]), _p(du[1]), 0, _p(dh[0]), _p(dh[1]), 0,
                                                  B, N, self._stream()), "hadamard_gelu_bwd")
        return du, dh

    def residual_fwd(self, u, v):
        y = self._new(*u[0].shape)
        _lib.check(self.lib.cnb_residual_fwd(self.h, _p(u[0]), _p(u[1]), _p(v[0]), _p(v[1]), _p(y[0]), _p(y[1]),
                                             u[0].numel(), self._stream()), "residual_fwd")
        return y

    def axpy(self, src, dst, accumulate=True):
        _lib.check(self.lib.cnb_axpy(self.h, _p(src[0]), _p(src[1]), _p(dst[0]), _p(dst[1]), src[0].numel(),
                                     int(accumulate), self._stream()), "axpy")
        return dst

    # ---------------------------------------------------------- row reductions
    def softmax_fwd(self, z):
        B, N = z[0].shape
        y = self._new(B, N)
        inv = self.torch.empty(B, dtype=self.torch.float32, device="cuda")
        _lib.check(self.lib.cnb_softmax_fwd(self.h, _p(z[0]), _p(z[1]), _p(y[0]), _p(y[1]), _p(inv), B, N,
                                            self._stream()), "softmax_fwd")
        return y, inv

    def softmax_bwd(self, g, z, inv):
        B, N = z[0].shape
        d = self._new(B, N)
        _lib.check(self.lib.cnb_softmax_bwd(self.h, _p(g[0]), _p(g[1]), _p(z[0]), _p(z[1]), _p(inv), _p(d[0]), _p(d[1]),
                                            B, N, 0, self._stream()), "softmax_bwd")
        return d

    def crossent(self, z, labels, backward=True):
        B, M = z[0].shape
        loss = self.torch.empty(B, dtype=self.torch.float32, device="cuda")
        d = self._new(B, M) if backward else (None, None)
        _lib.check(self.lib.cnb_crossent_fwd_bwd(self.h, _p(z[0]), _p(z[1]), _p(labels), _p(loss), _p(d[0]), _p(d[1]),
                                                 B, M, self._stream()), "crossent")
        return loss, d

    # --------------------------------------------------------------- embedding
    def embed_fwd(self, table, tokens):
        V, D = table[0].shape
        B, T = tokens.shape
        out = self._new(B, T * D)
        _lib.check(self.lib.cnb_embed_fwd(self.h, _p(table[0]), _p(table[1]), _p(tokens), _p(out[0]), _p(out[1]),
                                          B, T, D, V, self._stream()), "embed_fwd")
        return out

    def embed_bwd(self, g, tokens, dtable):
        V, D = dtable[0].shape
        B, T = tokens.shape
        _lib.check(self.lib.cnb_embed_bwd(self.h, _p(g[0]), _p(g[1]), _p(tokens), _p(dtable[0]), _p(dtable[1]),
                                          B, T, D, V, self._stream()), "embed_bwd")
        return dtable

    def sgd_update_split(self, w, g, lr, spans, zero_grad=True):
        """spans: [(begin, count, hi (float32), h16 (bfloat16), l16 (bfloat16))]; the updated floats of each span
        also leave their operand split: hi = w cut to TF32, h16 = bf16(hi), l16 = bf16(w - hi)."""
        arr = (_lib.SplitSpan * len(spans))()
        for k, (begin, count, hi, h16, l16) in enumerate(spans):
            arr[k].begin, arr[k].count = begin, count
            arr[k].hi, arr[k].h16, arr[k].l16 = hi.data_ptr(), h16.data_ptr(), l16.data_ptr()
        _lib.check(self.lib.cnb_sgd_update_split(self.h, _p(w), _p(g), w.numel(), lr, int(zero_grad), arr, len(spans),
                                                 self._stream()), "sgd_update_split")

    def sgd_update(self, w, g, lr, zero_grad=True):
        _lib.check(self.lib.cnb_sgd_update(self.h, _p(w), _p(g), w.numel(), lr, int(zero_grad), self._stream()),
                   "sgd_update")
