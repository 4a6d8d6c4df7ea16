"""ctypes binding of the C ABI declared in include/difflogic_b200.h.

The library is loaded from difflogic_b200/_lib/libdifflogic_b200.so (built in-tree by
`python -m difflogic_b200.build`).  There is no CPU or eager stand-in for these kernels: if
the library is missing, every CUDA code path of the package raises.
"""
import ctypes
import os

import torch

from . import build as _build

_i64 = ctypes.c_int64
_ptr = ctypes.c_void_p
_int = ctypes.c_int
_f32 = ctypes.c_float

DL_OK, DL_ERR_INVALID_ARG, DL_ERR_BAD_BIT_COUNT, DL_ERR_NOT_DIVISIBLE, DL_ERR_CUDA, DL_ERR_TOO_LARGE = range(6)
W_LOGITS, W_PROBS, W_ARGMAX = 0, 1, 2
LAUNCH_PLAIN, LAUNCH_OVERLAP_SETUP = 0, 1
(TUNE_NO_PDL, TUNE_EVAL_KERNEL, TUNE_EVAL_SHAPE, TUNE_GROUPBITSUM_KERNEL, TUNE_GROUPSUM_KERNEL, TUNE_FUSED_CLUSTER,
 TUNE_FORWARD_KERNEL) = range(7)

# name -> (restype, argtypes); mirrors include/difflogic_b200.h one to one
SIGNATURES = {
    "dl_version": (_int, []),
    "dl_last_error_string": (ctypes.c_char_p, []),
    "dl_async_error": (_int, []),
    "dl_selftest_bounded_wait": (_int, [_ptr, ctypes.c_uint32, _ptr]),
    "dl_set_tuning": (_int, [_int, _int]),
    "dl_get_tuning": (_int, [_int]),
    "dl_forward_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _int, _ptr, _ptr, _i64, _i64, _i64, _int, _ptr]),
    "dl_coefs_f32": (_int, [_ptr, _int, _ptr, _i64, _ptr]),
    "dl_backward_w_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _int, _ptr, _i64, _i64, _i64, _int, _ptr]),
    "dl_backward_x_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _f32, _ptr, _i64, _i64, _i64, _int, _ptr]),
    "dl_check_connections": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _ptr, _ptr]),
    "dl_build_backward_plan": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _ptr]),
    "dl_eval_packed": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _int, _ptr]),
    "dl_eval_packed_pitched": (_int, [_ptr, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "dl_argmax_gate_u8": (_int, [_ptr, _ptr, _i64, _ptr]),
    "dl_packbits": (_int, [_ptr, _ptr, _i64, _i64, _int, _ptr]),
    "dl_packbits_batch_major": (_int, [_ptr, _ptr, _i64, _i64, _int, _ptr]),
    "dl_threshold_packbits_batch_major": (_int, [_ptr, _ptr, _int, _ptr, _i64, _i64, _int, _ptr]),
    "dl_groupbitsum": (_int, [_ptr, _ptr, _i64, _i64, _i64, _i64, _int, _ptr]),
    "dl_eval_groupbitsum_applicable": (_int, [_ptr, _i64, _i64, _i64, _int, _i64]),
    "dl_eval_groupbitsum": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "dl_groupsum_workspace_bytes": (ctypes.c_size_t, [_i64, _i64, _i64]),
    "dl_groupsum_f32": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _f32, _ptr]),
    "dl_groupsum_backward_f32": (_int, [_ptr, _ptr, _i64, _i64, _i64, _f32, _ptr]),
    "dl_groupsum_static_limit_bytes": (ctypes.c_size_t, []),
    "dl_groupsum_f32_static": (_int, [_ptr, _ptr, _i64, _i64, _i64, _f32, _ptr]),
    "dl_cross_entropy_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _ptr]),
    "dl_cross_entropy_backward_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _ptr]),
    "dl_groupsum_cross_entropy_backward_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _f32, _ptr]),
    "dl_groupsum_cross_entropy_applicable": (_int, [_i64, _i64, _i64]),
    "dl_groupsum_cross_entropy_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _f32, _ptr]),
    "dl_forward_class_sums_rows": (_i64, [_i64, _i64, _i64]),
    "dl_forward_class_sums_run": (_i64, [_i64]),
    "dl_forward_class_sums_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _int, _ptr, _ptr, _i64, _i64, _i64, _i64, _int, _ptr]),
    "dl_class_sums_cross_entropy_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _f32, _ptr]),
    "dl_backward_w_classes_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _int, _ptr, _i64, _i64, _i64, _i64, _int, _ptr]),
    "dl_backward_w_adam_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _f32, _f32, _f32, _f32,
                                      _f32, _ptr, _int, _ptr]),
    "dl_transpose_f32": (_int, [_ptr, _ptr, _i64, _i64, _ptr]),
    "dl_backward_x_classes_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _f32, _ptr, _i64, _i64, _i64, _i64, _int, _ptr]),
    "dl_comm_alloc": (_int, [ctypes.c_size_t, _ptr]),
    "dl_comm_free": (_int, [_ptr]),
    "dl_comm_export": (_int, [_ptr, _ptr]),
    "dl_comm_import": (_int, [_ptr, _ptr]),
    "dl_comm_close": (_int, [_ptr]),
    "dl_exchange_flag_bytes": (ctypes.c_size_t, []),
    "dl_exchange_flag_word": (_int, [_int, _int, _int]),
    "dl_exchange_announce": (_int, [_ptr, _int, _int, _int, _ptr, _ptr]),
    "dl_exchange_packets_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _int, _int, _ptr, _ptr, _i64, _i64, _i64, _i64, _f32, _f32, _f32, _f32,
                                       _ptr, _int, ctypes.c_uint32, _int, _ptr]),
    "dl_backward_w_push_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr, _int, _int, _i64, _i64, _i64,
                                      _i64, _ptr, _int, _ptr]),
    "dl_rank_barrier": (_int, [_ptr, _int, _int, _int, _ptr, ctypes.c_uint32, _ptr]),
    "dl_exchange_bucket_f32": (_int, [_ptr, _ptr, _ptr, _int, _int, _ptr, _ptr, _i64, _i64, _int, _f32, _f32, _f32, _f32, _ptr, _int,
                                      _int, ctypes.c_uint32, _int, _ptr]),
    "dl_backward_w_announce_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr, _int, _int, _int, _ptr,
                                          _ptr, _ptr, _int, _int, _ptr]),
    "dl_adam_step_f32": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _f32, _f32, _f32, _f32, _f32, _ptr, _ptr]),
    "dl_prefetch_l2": (_int, [_ptr, ctypes.c_size_t, _ptr]),
}

_lib = None
_launches = 0


def launch_count():
    """Number of kernel launches issued through check() so far (every checked entry point launches one kernel)."""
    return _launches


class NativeLibraryMissing(RuntimeError):
    pass


def library_path():
    return _build.LIB_PATH


def lib():
    """The loaded library; raises NativeLibraryMissing when it has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise NativeLibraryMissing(
                "difflogic_b200: %s not found. Build it with `python -m difflogic_b200.build` "
                "(needs nvcc); there is no fallback implementation of the CUDA path." % path)
        handle = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class tuning:
    """Context manager: a kernel-choice switch (dl_set_tuning) set for the duration of a block, for A/B comparisons."""

    def __init__(self, key, value):
        self.key, self.value = key, value

    def __enter__(self):
        self.old = lib().dl_get_tuning(self.key)
        check_status(lib().dl_set_tuning(self.key, self.value))
        return self

    def __exit__(self, *exc):
        lib().dl_set_tuning(self.key, self.old)


def check_status(status):
    """check() for entry points that launch nothing."""
    global _launches
    check(status)
    _launches -= 1


def last_error():
    return lib().dl_last_error_string().decode("utf-8", "replace")


def check(status):
    """Maps a status code to the exception type the reference raises for the same mistake:
    ValueError for a bad bit_count or a non-divisible group count, RuntimeError otherwise."""
    global _launches
    if status == DL_OK:
        _launches += 1
        return
    msg = last_error()
    if status in (DL_ERR_BAD_BIT_COUNT, DL_ERR_NOT_DIVISIBLE):
        raise ValueError(msg)
    raise RuntimeError("difflogic_b200 (status %d): %s" % (status, msg))


def stream_of(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def ptr(t):
    return 0 if t is None else t.data_ptr()


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("difflogic_b200: expected a CUDA tensor, got one on %s" % t.device)
