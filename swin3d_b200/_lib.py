"""ctypes binding of libswin3d_b200.so (the C-ABI declared in include/swin3d_b200.h).

There is no fallback: if the shared library is missing or fails to load, importing this module
raises, and every operator of the package with it.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libswin3d_b200.so")

S3D_OK = 0
S3D_F32 = 0
S3D_F16 = 1

_c_void_p = ctypes.c_void_p
_i32 = ctypes.c_int
_i64 = ctypes.c_int64

# symbol -> (restype, argtypes); must list every declaration of include/swin3d_b200.h
SIGNATURES = {
    "s3d_status_string": (ctypes.c_char_p, [_i32]),
    "s3d_version": (_i32, []),
    "s3d_last_cuda_error_string": (ctypes.c_char_p, []),
    "s3d_debug_force_generic": (_i32, [_i32]),
    "s3d_debug_ffma_probe": (_i32, [_c_void_p, _i32, _i32, _c_void_p]),
    "s3d_attn_fwd": (_i32, [_c_void_p] * 6 + [_c_void_p, _i32] + [_c_void_p] * 4 +
                     [_i64, _i64, _i32, _i32, _i32, _c_void_p, _c_void_p, _c_void_p]),
    "s3d_attn_bwd": (_i32, [_c_void_p] * 6 + [_c_void_p, _i32] + [_c_void_p] * 4 +
                     [_i64, _i64, _i32, _i32, _i32] + [_c_void_p] * 3 + [_c_void_p] * 6 + [_c_void_p]),
    "s3d_attn_fwd_mirrored": (_i32, [_c_void_p] * 6 + [_c_void_p, _i32] + [_c_void_p] * 4 +
                              [_i64, _i64, _i32, _i32, _i32, _c_void_p, _c_void_p, _i32, _c_void_p, _i32, _c_void_p]),
    "s3d_attn_bwd_mirrored": (_i32, [_c_void_p] * 6 + [_c_void_p, _i32] + [_c_void_p] * 4 +
                              [_i64, _i64, _i32, _i32, _i32] + [_c_void_p] * 3 + [_c_void_p] * 6 +
                              [_i32, _c_void_p, _c_void_p, _c_void_p, _c_void_p]),
    "s3d_peer_alloc": (_i32, [_i64, _c_void_p, _c_void_p]),
    "s3d_peer_free": (_i32, [_c_void_p]),
    "s3d_ipc_open": (_i32, [_c_void_p, _c_void_p]),
    "s3d_ipc_close": (_i32, [_c_void_p]),
    "s3d_debug_crse_indices": (_i32, [_c_void_p, _c_void_p, _i32, _i32, _i32, _i32, _i32,
                                      _c_void_p, _c_void_p]),
    "s3d_debug_crse_indices_variant": (_i32, [_c_void_p, _c_void_p, _i32, _i32, _i32, _i32, _i32, _i32,
                                              _c_void_p, _c_void_p]),
    "s3d_debug_crse_index_values": (_i32, [_c_void_p, _c_void_p, _i64, _i32, _i32, _i32, _c_void_p, _c_void_p]),
    "s3d_gather_rows": (_i32, [_c_void_p, _i32, _c_void_p, _i64, _i64, _c_void_p, _i64, _c_void_p]),
    "s3d_scatter_rows": (_i32, [_c_void_p, _i32, _c_void_p, _i64, _i64, _i64, _i64, _i64, _c_void_p, _c_void_p]),
    "s3d_window_build_workspace_bytes": (_i64, [_i64]),
    "s3d_window_build": (_i32, [_c_void_p, _c_void_p, _i64, _i32, _i32, _i32, _i32] +
                         [_c_void_p] * 5 + [_c_void_p, _i64, _c_void_p]),
    "s3d_window_build_static": (_i32, [_c_void_p, _c_void_p, _i64, _i32, _i32, _i32, _i32] +
                                [_c_void_p] * 5 + [_c_void_p]),
    "s3d_knn": (_i32, [_i32, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _i32, _i64, _i64,
                       _c_void_p, _c_void_p, _c_void_p]),
    "s3d_knn_interpolate_fwd": (_i32, [_c_void_p] * 4 + [_i64, _i32, _i32, _i32, _c_void_p]),
    "s3d_knn_interpolate_bwd": (_i32, [_c_void_p] * 4 + [_i64, _i64, _i32, _i32, _i32, _c_void_p]),
    "s3d_knn_maxpool_fwd": (_i32, [_c_void_p] * 4 + [_i64, _i32, _i32, _i32, _c_void_p]),
    "s3d_knn_maxpool_bwd": (_i32, [_c_void_p] * 3 + [_i64, _i64, _i32, _i32, _c_void_p]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m swin3d_b200.build` "
            "(nvcc, sm_100a). swin3d_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class S3DError(RuntimeError):
    pass


def check(status: int, what: str):
    if status != S3D_OK:
        msg = lib.s3d_status_string(status).decode()
        # shape/argument problems surface as ValueError, runtime problems as RuntimeError
        if status in (1, 2):
            raise ValueError(f"{what}: {msg}")
        if status == 3:
            msg += " (" + lib.s3d_last_cuda_error_string().decode() + ")"
        raise S3DError(f"{what}: {msg}")
