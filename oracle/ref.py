"""ctypes wrapper of ``oracle/_ref/libcnet_ref.so`` — the unmodified reference CPU path
behind ``oracle/ref_driver.cpp``.  TEST INFRASTRUCTURE ONLY (also the bench's CPU baseline).

Same flat interface as ``oracle.cnet_oracle.OracleNet``.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libcnet_ref.so")
_lib = None

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)


def available():
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(LIB_PATH)
        _lib.ref_create.restype = C.c_void_p
        _lib.ref_destroy.argtypes = [C.c_void_p]
        _lib.ref_add.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, _ip, C.c_int]
        for n in ("ref_set_values", "ref_get_values", "ref_get_wgrad"):
            getattr(_lib, n).argtypes = [C.c_void_p, C.c_int, _fp, _fp, C.c_int]
        _lib.ref_zero_wgrads.argtypes = [C.c_void_p]
        _lib.ref_run_batch.argtypes = [C.c_void_p, C.c_int, _fp, _fp, _ip, C.c_int, _ip, C.c_int, _fp, C.c_int]
        _lib.ref_get_record.argtypes = [C.c_void_p, C.c_int, C.c_int, _fp, _fp]
        _lib.ref_max_threads.restype = C.c_int
        _lib.ref_out_size.argtypes = [C.c_void_p, C.c_int]
        _lib.ref_update.argtypes = [C.c_void_p, C.c_float, C.c_int]
        _lib.ref_set_threads.argtypes = [C.c_int]
        _lib.ref_adam_update.argtypes = [C.c_void_p, C.c_float, C.c_int, C.c_float, C.c_int]
        _lib.ref_save.argtypes = [C.c_void_p, C.c_char_p]
        _lib.ref_restore.argtypes = [C.c_char_p]
        _lib.ref_restore.restype = C.c_void_p
        for n in ("ref_num_funcs",):
            getattr(_lib, n).argtypes = [C.c_void_p]
        for n in ("ref_uid_at", "ref_type_of", "ref_in_len"):
            getattr(_lib, n).argtypes = [C.c_void_p, C.c_int]
    return _lib


def _f(a):
    return a.ctypes.data_as(_fp)


def _i(a):
    return a.ctypes.data_as(_ip)


def set_threads(n):
    lib().ref_set_threads(int(n))


def max_threads():
    return lib().ref_max_threads()


class RefNet:
    def __init__(self):
        lib()
        self.h = C.c_void_p(_lib.ref_create())
        self.in_len = {}
        self.B = 0

    def __del__(self):
        if getattr(self, "h", None):
            lib().ref_destroy(self.h)
            self.h = None

    def save(self, path):
        """ModelSaver::Save of the reference (impl/model_saver.h:799-821)."""
        assert lib().ref_save(self.h, str(path).encode()) == 0

    @classmethod
    def restore(cls, path):
        """ModelSaver::Restore of the reference into a fresh ComplexNet."""
        self = cls.__new__(cls)
        self.h = C.c_void_p(lib().ref_restore(str(path).encode()))
        assert self.h, "reference could not restore " + str(path)
        self.B = 0
        self.in_len = {}
        for i in range(lib().ref_num_funcs(self.h)):
            uid = lib().ref_uid_at(self.h, i)
            self.in_len[uid] = lib().ref_in_len(self.h, uid)
        return self

    def uids(self):
        return [lib().ref_uid_at(self.h, i) for i in range(lib().ref_num_funcs(self.h))]

    def type_of(self, uid):
        return lib().ref_type_of(self.h, uid)

    def add(self, type_, a=0, b=0, c=0, prev=()):
        p = np.asarray(list(prev), np.int32)
        uid = lib().ref_add(self.h, type_, a, b, c, _i(p), len(p))
        assert uid > 0, "ref_add failed"
        from .cnet_oracle import _Fn
        self.in_len[uid] = _Fn(uid, type_, a, b, c, prev).in_len
        return uid

    def out_size(self, uid):
        return lib().ref_out_size(self.h, uid)

    def set_values(self, uid, re, im):
        re = np.ascontiguousarray(re, np.float32).reshape(-1)
        im = np.ascontiguousarray(im, np.float32).reshape(-1)
        assert lib().ref_set_values(self.h, uid, _f(re), _f(im), re.size) == 0

    def _get(self, name, uid):
        n = self.in_len[uid]
        re, im = np.empty(n, np.float32), np.empty(n, np.float32)
        assert getattr(lib(), name)(self.h, uid, _f(re), _f(im), n) == 0
        return re, im

    def get_values(self, uid):
        return self._get("ref_get_values", uid)

    def get_wgrad(self, uid):
        return self._get("ref_get_wgrad", uid)

    def zero_wgrads(self):
        lib().ref_zero_wgrads(self.h)

    def run_batch(self, main_uid, x=None, tokens=None, labels=None, record=True):
        labels = np.ascontiguousarray(labels, np.int32)
        B = labels.size
        self.B = B
        losses = np.empty(B, np.float32)
        if tokens is not None:
            tok = np.ascontiguousarray(tokens, np.int32).reshape(B, -1)
            rc = lib().ref_run_batch(self.h, main_uid, None, None, _i(tok), tok.shape[1], _i(labels), B,
                                     _f(losses), int(record))
        else:
            xr = np.ascontiguousarray(x[0], np.float32)
            xi = np.ascontiguousarray(x[1], np.float32)
            rc = lib().ref_run_batch(self.h, main_uid, _f(xr), _f(xi), None, 0, _i(labels), B,
                                     _f(losses), int(record))
        assert rc == 0, "ref_run_batch failed %d" % rc
        return losses.astype(np.float64)

    def get_record(self, uid, what):
        n = self.out_size(uid)
        re, im = np.empty((self.B, n), np.float32), np.empty((self.B, n), np.float32)
        assert lib().ref_get_record(self.h, uid, what, _f(re), _f(im)) == 0
        return re, im

    def update(self, lr, batch_size):
        lib().ref_update(self.h, float(lr), int(batch_size))

    def adam(self, lr, batch_size, beta, t):
        lib().ref_adam_update(self.h, float(lr), int(batch_size), float(beta), int(t))
