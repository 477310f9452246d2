"""numpy restatement of the reference CPU training step.  TEST INFRASTRUCTURE ONLY.

This is the checker, never the thing measured or shipped.  It restates, batched and in
float64 (``dtype`` selectable), the per-sample math of the reference's CPU layers; each
method cites the reference lines it follows.  Parity is PINNED: ``tests/test_oracle.py``
checks this file against outputs of the unmodified reference CPU code (``oracle/_ref``,
built from the reference sources by ``oracle/Makefile``) committed as fixtures under
``tests/golden/`` and, when ``_ref`` is present, against it live.

Step semantics (reference trainer loop, cnet.cpp:58-102, impl/cnet.h:366-421):
    for b in batch: setInput; forward; loss; backward(label_b)   # activation grads per sample,
    update(lr, B):  w -= (lr / B) * sum_b dL/dz*_w               # weight grads summed over b

Only the dL/dz* chain is carried: for the real-valued loss seeded with dz = conj(dz*)
(impl/crossent.h:95-101) every layer here preserves dz == conj(dz*), so dL/dz is the
conjugate of what is stored.
"""
import numpy as np

# layer type ids: the reference's own (impl/cnet.h:31-44)
HADAMARD, EMBEDDING, LINEAR, FOURIER, CROSSENT, RESIDUAL, SOFTMAX, INPUT, CRELU, GELU, L2OUT, TRIFOURIER = range(1, 13)

GELU_K = np.float32(np.sqrt(np.float32(2.0) / np.float32(np.pi)))  # sqrtf(2/pi), impl/relu.h:10


def _gelu(x):
    # impl/relu.h:119-122
    return 0.5 * x * (1.0 + np.tanh(float(GELU_K) * (x + 0.044715 * x ** 3)))


def _dgelu(x):
    # impl/relu.h:124-131
    arg = float(GELU_K) * (x + 0.044715 * x ** 3)
    t = np.tanh(arg)
    sech2 = 1.0 / np.cosh(np.clip(arg, -300, 300)) ** 2
    return 0.5 * (1.0 + t) + x * 0.5 * sech2 * float(GELU_K) * (1.0 + 3.0 * 0.044715 * x * x)


class _Fn:
    def __init__(self, uid, type_, a, b, c, prev):
        self.uid, self.type, self.a, self.b, self.c, self.prev = uid, type_, a, b, c, list(prev)
        self.consumers = []
        if type_ == INPUT:
            self.in_len, self.out = a, a
        elif type_ == EMBEDDING:           # dim a, max tokens b, vocab c (impl/embed.h:43-47)
            self.in_len, self.out = a * c, a * b
        elif type_ == LINEAR:              # in1 = a, in2 = b = in1*out (impl/linear.h:18-23)
            assert b % a == 0
            self.in_len, self.out = a + b, b // a
        elif type_ in (HADAMARD, RESIDUAL):
            self.in_len, self.out = 2 * a, a
        elif type_ in (CROSSENT, L2OUT):
            self.in_len, self.out = a, 1
        else:
            self.in_len, self.out = a, a
        self.is_input = type_ in (INPUT, EMBEDDING)
        self.value = None                  # complex [len] for inputs
        self.wgrad = None                  # accumulated dL/dz* for inputs
        self.momentum = None               # Adam momentum (the reference keeps it in the dz planes)


class OracleNet:
    """Same flat interface as ``oracle.ref.RefNet`` (the compiled reference)."""

    def __init__(self, dtype=np.float64):
        self.rt = np.dtype(dtype)
        self.ct = np.complex128 if self.rt == np.float64 else np.complex64
        self.fn = {}
        self.order = []
        self.act = {}
        self.gstar = {}

    # impl/cnet.h:228-289 (add), impl/cfunc.h:211-224 (addOutput: consumer offset = sum of
    # the earlier producers' out sizes)
    def add(self, type_, a=0, b=0, c=0, prev=()):
        uid = len(self.order) + 1
        f = _Fn(uid, type_, a, b, c, prev)
        off = 0
        for p in prev:
            self.fn[p].consumers.append((uid, off))
            off += self.fn[p].out
        assert off <= f.in_len
        self.fn[uid] = f
        self.order.append(uid)
        if f.is_input:
            f.value = np.zeros(f.in_len, self.ct)
            f.wgrad = np.zeros(f.in_len, self.ct)
        return uid

    def out_size(self, uid):
        return self.fn[uid].out

    def set_values(self, uid, re, im):
        f = self.fn[uid]
        f.value = (np.asarray(re, self.rt) + 1j * np.asarray(im, self.rt)).astype(self.ct).reshape(f.in_len)

    def get_values(self, uid):
        v = self.fn[uid].value
        return v.real.copy(), v.imag.copy()

    def get_wgrad(self, uid):
        g = self.fn[uid].wgrad
        return g.real.copy(), g.imag.copy()

    def zero_wgrads(self):
        for f in self.fn.values():
            if f.is_input:
                f.wgrad[:] = 0

    # ------------------------------------------------------------------ forward
    def _input_block(self, f, B):
        """Concatenate the producers' outputs, batched: [B, in_len] (impl/cnet.h:256-272)."""
        parts = []
        for p in f.prev:
            a = self.act[p]
            if a.ndim == 1:
                a = np.broadcast_to(a, (B, a.shape[0]))
            parts.append(a)
        return parts

    def run_batch(self, main_uid, x=None, tokens=None, labels=None, record=True):
        labels = np.asarray(labels)
        B = labels.shape[0]
        self.act, self.gstar = {}, {}
        ce_uid = None
        for uid in self.order:
            f = self.fn[uid]
            t = f.type
            if t == INPUT:
                # impl/cinput.h:42-52: forward copies the stored planes to every consumer
                if uid == main_uid:
                    xr, xi = x
                    self.act[uid] = (np.asarray(xr, self.rt) + 1j * np.asarray(xi, self.rt)).astype(self.ct)
                else:
                    self.act[uid] = f.value
                continue
            if t == EMBEDDING:
                # impl/embed.h:109-131: gather rows, zero-fill the tail (token < 0 = padding,
                # impl/batch.h:11,83-85)
                tok = np.asarray(tokens).reshape(B, f.b)
                table = f.value.reshape(f.c, f.a)
                rows = table[np.where(tok < 0, 0, tok)]
                rows = np.where((tok < 0)[..., None], 0, rows)
                self.act[uid] = rows.reshape(B, f.b * f.a).astype(self.ct)
                f._tok = tok
                continue
            parts = self._input_block(f, B)
            if t == FOURIER:
                # impl/ft.h:37-55: X_p = N^-1/2 sum_q x_q e^{-2 pi i pq/N} (sign impl/utils.h:218-221)
                self.act[uid] = (np.fft.fft(parts[0], axis=1) / np.sqrt(f.a)).astype(self.ct)
            elif t == HADAMARD:
                self.act[uid] = parts[0] * parts[1]                    # impl/hadamard.h:34-44
            elif t == RESIDUAL:
                self.act[uid] = parts[0] + parts[1]                    # impl/residual.h:40-50
            elif t == GELU:
                z = parts[0]                                           # impl/relu.h:133-142
                self.act[uid] = (_gelu(z.real) + 1j * _gelu(z.imag)).astype(self.ct)
            elif t == LINEAR:
                # impl/linear.h:51-71: y_o = sum_i x_i W[o,i], W row-major [out][in], no conj
                xb = parts[0]
                W = self.act[f.prev[1]].reshape(f.out, f.a)
                self.act[uid] = xb @ W.T
            elif t == SOFTMAX:
                # impl/softmax.h:33-59: y = z / max(||z||, 1e-15)
                z = parts[0]
                n = np.maximum(np.sqrt((np.abs(z) ** 2).sum(1, keepdims=True)), 1e-15)
                f._n = n
                self.act[uid] = z / n
            elif t == CRELU:
                z = parts[0]                                           # impl/relu.h:31-45
                self.act[uid] = np.where((z.real > 0) & (z.imag > 0), z, 0)
            elif t == TRIFOURIER:
                # impl/ft.h:139-161: y_p = N^-1/2 sum_{q <= p} x_q e^{-2 pi i pq/N}
                self.act[uid] = parts[0] @ self._tri(f.a).T
            elif t in (CROSSENT, L2OUT):
                ce_uid = uid
                f._z = parts[0]
            else:
                raise ValueError("unsupported type %d" % t)
        # ---------------------------------------------------------------- loss
        f = self.fn[ce_uid]
        z = f._z
        if f.type == L2OUT:
            # impl/l2out.h:31-57: loss = sum |z|^2; generic out_backward (impl/cfunc.h:327-339) seeds dz* = z
            losses = (np.abs(z) ** 2).sum(1)
            return self._backward(main_uid, ce_uid, z.copy(), losses, B)
        # impl/crossent.h:57-78 + 50-55: S = max(sum |z|^2, 1e-15); p = |z_l / sqrt(S)|^2
        S = np.maximum((np.abs(z) ** 2).sum(1), 1e-15)
        zl = z[np.arange(B), labels]
        p = np.maximum(np.abs(zl) ** 2 / S, 1e-15)
        losses = -np.log(p)
        # ------------------------------------------------------------ backward
        # impl/crossent.h:80-104 (assigns): dz*_k = z_k / S (k != l);
        # dz*_l = -z_l (S - m) / (m S), m = max(|z_l|^2, 1e-15)
        g = z / S[:, None]
        m = np.maximum(np.abs(zl) ** 2, 1e-15)
        g[np.arange(B), labels] = -zl * (S - m) / (m * S)
        return self._backward(main_uid, ce_uid, g, losses, B)

    def _tri(self, n):
        p, q = np.meshgrid(np.arange(n), np.arange(n), indexing="ij")
        return np.where(q <= p, np.exp(-2j * np.pi * ((p * q) % n) / n), 0) / np.sqrt(n)

    def _backward(self, main_uid, ce_uid, g, losses, B):
        gin = {ce_uid: [g]}                 # per function: dL/dz* of its input block parts
        for uid in reversed(self.order):
            f = self.fn[uid]
            # gradient of this function's output = sum over consumers (each consumer block
            # holds its own contribution; producers sum them, e.g. impl/cinput.h:54-65)
            go = None
            for (cu, off) in f.consumers:
                cf = self.fn[cu]
                idx = cf.prev.index(uid)
                part = gin[cu][idx]
                go = part if go is None else go + part
            if f.consumers:
                self.gstar[uid] = go
            t = f.type
            if t == INPUT:
                if uid != main_uid and go is not None:
                    f.wgrad += go.sum(0) if go.ndim == 2 else go     # impl/cinput.h:54-65
                continue
            if t == EMBEDDING:
                # impl/embed.h:133-148: scatter-add dz* rows into the table gradient
                tok = f._tok
                gg = go.reshape(B, f.b, f.a)
                acc = f.wgrad.reshape(f.c, f.a)
                valid = tok >= 0
                np.add.at(acc, tok[valid], gg[valid])
                continue
            if t in (CROSSENT, L2OUT):
                continue
            parts = self._input_block(f, B)
            if t == FOURIER:
                # impl/ft.h:57-80: dz*_q = N^-1/2 sum_p g*_p conj(w^{pq}), w = e^{-2 pi i/N}
                gin[uid] = [np.fft.ifft(go, axis=1) * np.sqrt(f.a)]
            elif t == HADAMARD:
                # impl/hadamard.h:46-68: dz*_u = g* conj(v), dz*_v = g* conj(u)
                gin[uid] = [go * np.conj(parts[1]), go * np.conj(parts[0])]
            elif t == RESIDUAL:
                gin[uid] = [go, go]                                   # impl/residual.h:52-77
            elif t == GELU:
                # impl/relu.h:144-168 with g = conj(g*): dz* = g (dx-dy) + g* (dx+dy)
                z = parts[0]
                dx, dy = 0.5 * _dgelu(z.real), 0.5 * _dgelu(z.imag)
                gin[uid] = [np.conj(go) * (dx - dy) + go * (dx + dy)]
            elif t == CRELU:
                z = parts[0]                                          # impl/relu.h:47-62
                gin[uid] = [np.where((z.real > 0) & (z.imag > 0), go, 0)]
            elif t == TRIFOURIER:
                # impl/ft.h:163-188: dz*_q = N^-1/2 sum_{p >= q} g*_p conj(w^{pq})
                gin[uid] = [go @ np.conj(self._tri(f.a))]
            elif t == LINEAR:
                # impl/linear.h:73-110: dX*[b,i] = sum_o g*[b,o] conj(W[o,i]);
                # dW*[o,i] = g*[b,o] conj(x[b,i]) (per sample; the weight CInput sums over b)
                xb = parts[0]
                W = self.act[f.prev[1]].reshape(f.out, f.a)
                gin[uid] = [go @ np.conj(W), (go.T @ np.conj(xb)).reshape(-1)]
            elif t == SOFTMAX:
                # impl/softmax.h:61-73 through the generic chain rule impl/cfunc.h:290-325,
                # collapsed with g = conj(g*): dz*_i = g*_i/n - z_i/n^3 * Re sum_j g*_j conj(z_j)
                z, n = parts[0], f._n
                s = (go * np.conj(z)).sum(1, keepdims=True).real
                gin[uid] = [go / n - z * s / n ** 3]
        self.losses = losses
        return losses.astype(np.float64)

    # impl/cnet.h:423-431 + impl/cfunc.h:273-287: m = beta m + (1-beta) dz*; w -= (lr/batch) m / (1 - beta^(t+1));
    # dz* zeroed (the momentum lives in the dz planes, which update() would zero but adamUpdate does not)
    def adam(self, lr, batch_size, beta, t):
        for f in self.fn.values():
            if f.is_input:
                if f.momentum is None:
                    f.momentum = np.zeros_like(f.wgrad)
                f.momentum = beta * f.momentum + (1 - beta) * f.wgrad
                f.value = f.value - (lr / batch_size) * f.momentum / (1 - beta ** (t + 1))
                f.wgrad[:] = 0

    def get_record(self, uid, what):
        a = self.act[uid] if what == 0 else self.gstar[uid]
        if what == 2:
            a = np.conj(a)
        return a.real.copy(), a.imag.copy()

    # impl/cnet.h:413-421 + impl/cfunc.h:147-152: w -= (lr / batch) * dz*_w, then zero grads.
    # (The data CInput is updated too in the reference; it is overwritten by the next
    # setInput, so it is left out here.)
    def update(self, lr, batch_size):
        for f in self.fn.values():
            if f.is_input:
                f.value = f.value - (lr / batch_size) * f.wgrad
                f.wgrad[:] = 0
