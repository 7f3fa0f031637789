"""ctypes binding of ``libminuet_b200.so`` (declared in ``include/minuet_b200.h``).

There is no CPU fallback: importing this module on a machine where the library
was never built raises, and so does every call that reports a non-zero status.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# MINUET_B200_LIB points at another build of the same library (kernel experiments)
LIB_PATH = os.environ.get("MINUET_B200_LIB") or os.path.join(_HERE, "libminuet_b200.so")

MN_OK, MN_ERR_BAD_ARG, MN_ERR_UNSUPPORTED, MN_ERR_WORKSPACE, MN_ERR_CUDA, MN_ERR_DEVICE = range(6)
MN_F32, MN_F16, MN_BF16 = 0, 1, 2
MN_MAX_NDIM = 4
MN_MAX_OFFSETS = 128
MN_CTRL_WORDS = 1024
ABI_VERSION = 14         # must equal MN_ABI_VERSION of the header the library was built from

c_i32p = ctypes.c_void_p
c_ptr = ctypes.c_void_p
c_i64 = ctypes.c_int64
c_int = ctypes.c_int
c_size = ctypes.c_size_t
c_dbl = ctypes.c_double


class KeySpec(ctypes.Structure):
    """Mirror of ``mn_keyspec``."""
    _fields_ = [
        ("ndim", ctypes.c_int32),
        ("total_bits", ctypes.c_int32),
        ("margin", ctypes.c_int32),
        ("cloud_shift", ctypes.c_int32),
        ("cloud_bits", ctypes.c_int32),
        ("shift", ctypes.c_int32 * MN_MAX_NDIM),
        ("bits", ctypes.c_int32 * MN_MAX_NDIM),
        ("base", ctypes.c_int64 * MN_MAX_NDIM),
        ("extent", ctypes.c_int64 * MN_MAX_NDIM),
        ("device_copy", ctypes.c_void_p),
    ]


# name -> (restype, argtypes); mirrors include/minuet_b200.h one to one
PROTOTYPES = {
    "mn_last_error": (ctypes.c_char_p, []),
    "mn_version": (c_int, []),
    "mn_launch_count": (ctypes.c_longlong, []),
    "mn_profile_enable": (None, [c_int]),
    "mn_profile_report": (c_int, [ctypes.c_char_p, c_int]),
    "mn_bbox": (c_int, [c_ptr, c_i64, c_ptr, c_i64, c_int, c_ptr, c_ptr, c_size, c_ptr]),
    "mn_keyspec_make": (c_int, [c_ptr, c_int, c_i64, ctypes.c_int32, ctypes.POINTER(KeySpec)]),
    "mn_pack_keys": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_i64, c_ptr, ctypes.POINTER(KeySpec),
                             c_ptr, c_ptr, c_ptr]),
    "mn_arg_sort_coordinates": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_i64, ctypes.POINTER(KeySpec),
                                        c_ptr, c_ptr, c_ptr, c_size, c_ptr]),
    "mn_unique_coordinates": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_i64, c_ptr, c_ptr, c_ptr,
                                      c_size, c_ptr]),
    "mn_unique_coordinates_static": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_i64, c_ptr, c_ptr, c_ptr]),
    "mn_downsample_coordinates": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_i64, c_ptr,
                                          ctypes.POINTER(KeySpec), c_ptr, c_ptr, c_ptr, c_ptr,
                                          c_ptr, c_size, c_ptr]),
    "mn_keyspec_device": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_i64, ctypes.c_int32, c_ptr,
                                  ctypes.POINTER(KeySpec), c_ptr, c_ptr, c_ptr, c_size, c_ptr]),
    "mn_query_sorted_index_with_offsets": (c_int, [c_ptr, c_i64, c_ptr, c_i64, c_ptr, c_i64,
                                                   ctypes.POINTER(KeySpec), c_ptr, c_ptr]),
    "mn_compute_kernel_map_sizes": (c_int, [c_ptr, c_i64, c_i64, c_ptr, c_ptr]),
    "mn_compute_kernel_map_masks": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_ptr,
                                            c_size, c_ptr]),
    "mn_build_kernel_map": (c_int, [c_ptr, c_i64, c_ptr, c_i64, c_ptr, c_i64,
                                    ctypes.POINTER(KeySpec), c_int, c_ptr, c_ptr, c_ptr, c_ptr,
                                    c_ptr, c_ptr, c_ptr, c_ptr, c_size, c_ptr]),
    "mn_map_workspace_bytes": (c_size, [c_i64, c_i64, c_i64]),
    "mn_plan_buckets": (c_int, [c_ptr, c_i64, c_int, c_dbl, c_ptr, c_ptr, c_ptr]),
    "mn_conv_workspace_bytes": (c_size, [c_ptr, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_int,
                                         c_int, c_dbl]),
    "mn_sparse_convolution_forward": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_ptr,
                                              c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_int,
                                              c_int, c_int, c_dbl, c_ptr, c_ptr, c_ptr, c_size,
                                              c_ptr]),
    "mn_conv_stage": (c_int, [c_int, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_ptr, c_ptr, c_ptr,
                              c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_dbl, c_ptr, c_ptr, c_ptr,
                              c_size, c_ptr]),
    "mn_apply_epilogue": (c_int, [c_ptr, c_i64, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_int, c_ptr]),
    "mn_implicit_supported": (c_int, [c_i64, c_i64, c_i64, c_int]),
    "mn_neighbor_table_workspace_bytes": (c_size, [c_ptr, c_i64, c_i64]),
    "mn_build_neighbor_table": (c_int, [c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_ptr,
                                        c_ptr, c_ptr, c_ptr, c_ptr, c_size, c_ptr]),
    "mn_implicit_workspace_bytes": (c_size, [c_i64, c_i64, c_i64]),
    "mn_sparse_convolution_forward_implicit": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_int,
                                                       c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
                                                       c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_dbl,
                                                       c_int, c_ptr, c_ptr, c_ptr, c_size, c_ptr]),
    "mn_transpose_weights": (c_int, [c_ptr, c_i64, c_i64, c_i64, c_int, c_ptr, c_ptr]),
    "mn_pairs_supported": (c_int, [c_i64, c_i64, c_i64, c_int]),
    "mn_pair_rows": (c_i64, [c_ptr, c_i64, c_i64, c_i64, c_int]),
    "mn_build_pair_list": (c_int, [c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_int, c_ptr, c_ptr]),
    "mn_pairs_workspace_bytes": (c_size, [c_ptr, c_i64, c_i64, c_i64, c_i64, c_i64, c_int]),
    "mn_sparse_convolution_forward_pairs": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_int,
                                                    c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
                                                    c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_ptr,
                                                    c_int, c_ptr, c_ptr, c_ptr, c_size, c_ptr]),
    "mn_dense_supported": (c_int, [c_i64, c_i64, c_int]),
    "mn_arg_sort_coordinates_by_dimension": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_i64, c_ptr, c_ptr,
                                                     c_ptr, c_size, c_ptr]),
    "mn_voxel_mean": (c_int, [c_ptr, c_i64, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_ptr]),
    "mn_dense_forward_simt": (c_int, [c_i64, c_i64, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
                                      c_int, c_ptr, c_ptr]),
    "mn_dense_workspace_bytes": (c_size, [c_i64, c_i64]),
    "mn_dense_forward": (c_int, [c_i64, c_i64, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
                                 c_ptr, c_int, c_ptr, c_ptr, c_ptr, c_size, c_ptr]),
}

_lib = None


def load():
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m minuet_b200.build` "
                "(nvcc, sm_100a). minuet_b200 has no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        lib.mn_version.restype = c_int
        if lib.mn_version() != ABI_VERSION:
            raise ImportError(
                f"{LIB_PATH} implements interface version {lib.mn_version()}, this binding "
                f"expects {ABI_VERSION}: rebuild it with `python -m minuet_b200.build`")
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def last_error() -> str:
    return load().mn_last_error().decode(errors="replace")


def check(status: int, what: str = ""):
    """Turn a non-zero ``mn_status`` into the exception the reference would raise
    (its C++ checks surface as RuntimeError through pybind11)."""
    if status == MN_OK:
        return
    msg = last_error()
    if status == MN_ERR_UNSUPPORTED:
        raise NotImplementedError(f"{what}: {msg}" if what else msg)
    raise RuntimeError(f"{what}: {msg}" if what else msg)
