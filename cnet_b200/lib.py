"""ctypes binding of libcnet_b200.so (kernels + C ABI + host facade).

The library is the product: importing this module without it raises — there is no CPU or
PyTorch fallback for any operation of the path.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcnet_b200.so")

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int32)
_vp = C.c_void_p
_sz = C.c_size_t

BUCKET_HOOK = C.CFUNCTYPE(C.c_int, _vp, _vp, _sz, C.c_int, C.c_int)

# name -> (restype, argtypes); the complete export list of include/cnet_b200.h and
# include/cnet_b200_host.h (tests check that every declared symbol is here and exported)
_P = _vp   # device or host pointer passed as an integer address
class SplitSpan(C.Structure):
    """cnb_split_span of include/cnet_b200.h."""
    _fields_ = [("begin", C.c_size_t), ("count", C.c_size_t), ("hi", C.c_void_p), ("h16", C.c_void_p), ("l16", C.c_void_p)]


SIGNATURES = {
    "cnb_last_error": (C.c_char_p, []),
    "cnb_create": (C.c_int, [C.c_int, _sz, C.POINTER(_vp)]),
    "cnb_create_external": (C.c_int, [C.c_int, _P, _sz, C.POINTER(_vp)]),
    "cnb_destroy": (C.c_int, [_vp]),
    "cnb_alloc": (C.c_int, [_vp, _sz, C.POINTER(_vp)]),
    "cnb_reset": (C.c_int, [_vp]),
    "cnb_arena_used": (_sz, [_vp]),
    "cnb_arena_size": (_sz, [_vp]),
    "cnb_device_info": (C.c_int, [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(_sz)]),
    "cnb_h2d": (C.c_int, [_vp, _P, _P, _sz, _vp]),
    "cnb_d2h": (C.c_int, [_vp, _P, _P, _sz, _vp]),
    "cnb_memset0": (C.c_int, [_vp, _P, _sz, _vp]),
    "cnb_sync": (C.c_int, [_vp, _vp]),
    "cnb_check_device_status": (C.c_int, [_vp, _vp]),
    "cnb_linear_fwd": (C.c_int, [_vp] + [_P] * 8 + [C.c_int] * 3 + [_vp]),
    "cnb_linear_bwd_x": (C.c_int, [_vp] + [_P] * 6 + [C.c_int] * 4 + [_vp]),
    "cnb_linear_bwd_w": (C.c_int, [_vp] + [_P] * 6 + [C.c_int] * 4 + [_vp]),
    "cnb_split_floats": (_sz, [_sz]),
    "cnb_split_planes": (C.c_int, [_vp, _P, _P, _sz, _P, _vp]),
    "cnb_linear_split_ok": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "cnb_linear_fwd_split": (C.c_int, [_vp] + [_P] * 6 + [C.c_int] * 3 + [_vp]),
    "cnb_linear_bwd_x_split": (C.c_int, [_vp] + [_P] * 4 + [C.c_int] * 4 + [_vp]),
    "cnb_linear_bwd_w_split": (C.c_int, [_vp] + [_P] * 4 + [C.c_int] * 4 + [_vp]),
    "cnb_set_gemm_sm_limit": (C.c_int, [_vp, C.c_int]),
    "cnb_last_gemm_engine": (C.c_int, []),
    "cnb_linear_workspace": (_sz, [C.c_int, C.c_int, C.c_int]),
    "cnb_reserve_scratch": (C.c_int, [_vp, _sz]),
    "cnb_dft_fwd": (C.c_int, [_vp] + [_P] * 4 + [C.c_int] * 2 + [_vp]),
    "cnb_dft_bwd": (C.c_int, [_vp] + [_P] * 4 + [C.c_int] * 3 + [_vp]),
    "cnb_dft_fused_ok": (C.c_int, [C.c_int]),
    "cnb_dft_hadamard_gelu_fwd": (C.c_int, [_vp] + [_P] * 9 + [C.c_int] * 2 + [_vp]),
    "cnb_tdft_fwd": (C.c_int, [_vp] + [_P] * 4 + [C.c_int] * 2 + [_vp]),
    "cnb_tdft_bwd": (C.c_int, [_vp] + [_P] * 4 + [C.c_int] * 3 + [_vp]),
    "cnb_crelu_fwd": (C.c_int, [_vp] + [_P] * 4 + [_sz, _vp]),
    "cnb_crelu_bwd": (C.c_int, [_vp] + [_P] * 6 + [_sz, C.c_int, _vp]),
    "cnb_l2out_fwd_bwd": (C.c_int, [_vp] + [_P] * 5 + [C.c_int] * 2 + [_vp]),
    "cnb_adam_update": (C.c_int, [_vp, _P, _P, _P, _sz, C.c_float, C.c_float, C.c_int, _vp]),
    "cnb_set_dft_engine": (C.c_int, [_vp, C.c_int]),
    "cnb_hadamard_fwd": (C.c_int, [_vp] + [_P] * 4 + [C.c_int] + [_P] * 2 + [C.c_int] * 2 + [_vp]),
    "cnb_hadamard_bwd": (C.c_int, [_vp] + [_P] * 6 + [C.c_int] + [_P] * 2 + [C.c_int] + [_P] * 2 + [C.c_int] * 3 + [_vp]),
    "cnb_hadamard_bwd_static": (C.c_int, [_P] * 8 + [C.c_int] + [_P] * 2 + [C.c_int] * 3 + [_vp]),
    "cnb_gelu_fwd": (C.c_int, [_vp] + [_P] * 4 + [_sz, _vp]),
    "cnb_gelu_bwd": (C.c_int, [_vp] + [_P] * 6 + [_sz, C.c_int, _vp]),
    "cnb_hadamard_gelu_fwd": (C.c_int, [_vp] + [_P] * 8 + [C.c_int] * 2 + [_vp]),
    "cnb_hadamard_gelu_fwd_split": (C.c_int, [_vp] + [_P] * 9 + [C.c_int] * 2 + [_vp]),
    "cnb_hadamard_gelu_bwd": (C.c_int, [_vp] + [_P] * 10 + [C.c_int] + [_P] * 2 + [C.c_int] * 3 + [_vp]),
    "cnb_residual_fwd": (C.c_int, [_vp] + [_P] * 6 + [_sz, _vp]),
    "cnb_axpy": (C.c_int, [_vp] + [_P] * 4 + [_sz, C.c_int, _vp]),
    "cnb_softmax_fwd": (C.c_int, [_vp] + [_P] * 5 + [C.c_int] * 2 + [_vp]),
    "cnb_softmax_bwd": (C.c_int, [_vp] + [_P] * 7 + [C.c_int] * 3 + [_vp]),
    "cnb_crossent_fwd_bwd": (C.c_int, [_vp] + [_P] * 6 + [C.c_int] * 2 + [_vp]),
    "cnb_embed_fwd": (C.c_int, [_vp] + [_P] * 5 + [C.c_int] * 4 + [_vp]),
    "cnb_embed_bwd": (C.c_int, [_vp] + [_P] * 5 + [C.c_int] * 4 + [_vp]),
    "cnb_sgd_update": (C.c_int, [_vp, _P, _P, _sz, C.c_float, C.c_int, _vp]),
    "cnb_gemm_schedule": (C.c_int, [C.c_int] * 6 + [C.POINTER(C.c_int)]),
    "cnb_sgd_update_split": (C.c_int, [_vp, _P, _P, _sz, C.c_float, C.c_int, _vp, C.c_int, _vp]),
    "cnb_launch_count": (C.c_ulonglong, []),
    # host facade
    "cnh_create": (_vp, [C.c_int, _sz, _P]),
    "cnh_destroy": (None, [_vp]),
    "cnh_set_device": (C.c_int, [_vp, C.c_int, _sz, _P]),
    "cnh_error": (C.c_char_p, [_vp]),
    "cnh_clear_error": (None, [_vp]),
    "cnh_add": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, C.c_int, _ip, C.c_int]),
    "cnh_out_size": (C.c_int, [_vp, C.c_int]),
    "cnh_init_inputs": (C.c_int, [_vp, C.c_uint64]),
    "cnh_set_values": (C.c_int, [_vp, C.c_int, _P, _P, C.c_int]),
    "cnh_get_values": (C.c_int, [_vp, C.c_int, _P, _P, C.c_int]),
    "cnh_get_wgrad": (C.c_int, [_vp, C.c_int, _P, _P, C.c_int]),
    "cnh_set_stream": (C.c_int, [_vp, _vp]),
    "cnh_set_fusion": (C.c_int, [_vp, C.c_int]),
    "cnh_set_bucket_hook": (C.c_int, [_vp, BUCKET_HOOK, _vp]),
    "cnh_required_arena": (_sz, [_vp, C.c_int]),
    "cnh_allocate": (C.c_int, [_vp, C.c_int]),
    "cnh_upload": (C.c_int, [_vp, _P, _P, _P, _P, C.c_int]),
    "cnh_prefetch": (C.c_int, [_vp, _P, _P, _P, _P, C.c_int]),
    "cnh_commit": (C.c_int, [_vp]),
    "cnh_read_losses_async": (C.c_int, [_vp, _P, C.c_int]),
    "cnh_wait_losses": (C.c_int, [_vp]),
    "cnh_forward": (C.c_int, [_vp]),
    "cnh_backward": (C.c_int, [_vp]),
    "cnh_backward_label": (C.c_int, [_vp, C.c_int]),
    "cnh_update": (C.c_int, [_vp, C.c_float]),
    "cnh_adam_update": (C.c_int, [_vp, C.c_float, C.c_float, C.c_int]),
    "cnh_infer": (C.c_int, [_vp]),
    "cnh_get_losses": (C.c_int, [_vp, _P, C.c_int]),
    "cnh_sync": (C.c_int, [_vp]),
    "cnh_read_output": (C.c_int, [_vp, C.c_int, C.c_int, _P, _P]),
    "cnh_grad_arena": (C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_sz), C.POINTER(C.c_int)]),
    "cnh_weight_arena": (C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_sz)]),
    "cnh_context": (_vp, [_vp]),
    "cnh_save": (C.c_int, [_vp, C.c_char_p]),
    "cnh_restore": (C.c_int, [_vp, C.c_char_p]),
    "cnh_num_funcs": (C.c_int, [_vp]),
    "cnh_uid_at": (C.c_int, [_vp, C.c_int]),
    "cnh_type_of": (C.c_int, [_vp, C.c_int]),
    "cnh_in_size": (C.c_int, [_vp, C.c_int]),
    "cnh_dp_unique_id": (C.c_int, [C.c_char_p]),
    "cnh_dp_init": (C.c_int, [_vp, C.c_char_p, C.c_int, C.c_int]),
    "cnh_dp_async_error": (C.c_int, [_vp]),
    "cnh_dp_allreduce_grads": (C.c_int, [_vp]),
    "cnh_dp_set_symmetric": (C.c_int, [_vp, C.c_int, C.c_int, _vp, C.POINTER(_vp), C.POINTER(_vp), C.c_int]),
    "cnb_dp_state_bytes": (_sz, []),
    "cnb_dp_allreduce": (C.c_int, [_vp, _vp, _P, _sz, _vp]),
    "cnh_dp_use_nccl_arena": (C.c_int, [_vp, C.c_int]),
    "cnh_dp_symmetric": (C.c_int, [_vp]),
    "cnh_mnist_open": (_vp, [C.c_char_p, C.c_char_p, C.c_int]),
    "cnh_mnist_close": (None, [_vp]),
    "cnh_mnist_size": (C.c_int, [_vp]),
    "cnh_mnist_shuffle": (C.c_int, [_vp, C.c_uint]),
    "cnh_mnist_has_next": (C.c_int, [_vp, C.c_int]),
    "cnh_mnist_next_batch": (C.c_int, [_vp, C.c_int, _P, _P, _P]),
    "cnh_capture_begin": (C.c_int, [_vp]),
    "cnh_capture_end": (C.c_int, [_vp]),
    "cnh_graph_launch": (C.c_int, [_vp]),
    "cnh_graph_kernel_count": (C.c_ulonglong, [_vp]),
}

_lib = None


class CnetError(RuntimeError):
    pass


def load():
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise CnetError("libcnet_b200.so is not built (run `python -m cnet_b200.build`); "
                        "there is no fallback path")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError if a declared symbol is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc, what=""):
    if rc < 0:
        raise CnetError("%s failed (%d): %s" % (what, rc, load().cnb_last_error().decode()))
    return rc
