"""ctypes view of liblmg_b200.so, the C ABI declared in include/lmg_b200.h.

Loading fails loudly when the library has not been built: there is no other code path.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# LMG_B200_LIB overrides the library path (for trying differently built variants)
LIB_PATH = os.environ.get("LMG_B200_LIB") or os.path.join(HERE, "liblmg_b200.so")

LMG_OK, LMG_ERR_OUT_OF_RANGE, LMG_ERR_INVALID_ARGUMENT, LMG_ERR_CUDA, LMG_ERR_WORKSPACE = range(5)
OP_FORWARD, OP_BACKWARD, OP_BACKWARD_GRADIENTS, OP_BACKWARD_RELEVANCE = range(4)

c_float_p = ctypes.POINTER(ctypes.c_float)
c_int_p = ctypes.POINTER(ctypes.c_int)


class GridMakerStruct(ctypes.Structure):
    _fields_ = [("resolution", ctypes.c_float), ("dimension", ctypes.c_float),
                ("radius_scale", ctypes.c_float), ("gaussian_radius_multiple", ctypes.c_float),
                ("final_radius_multiple", ctypes.c_float),
                ("A", ctypes.c_float), ("B", ctypes.c_float), ("C", ctypes.c_float),
                ("D", ctypes.c_float), ("E", ctypes.c_float),
                ("dim", ctypes.c_uint), ("binary", ctypes.c_int), ("radii_type_indexed", ctypes.c_int)]


class TransformStruct(ctypes.Structure):
    _fields_ = [("q", ctypes.c_float * 4), ("center", ctypes.c_float * 3),
                ("translate", ctypes.c_float * 3)]


class AtomsStruct(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int), ("max_atoms", ctypes.c_int), ("ntypes", ctypes.c_int),
                ("n_atoms", ctypes.c_void_p), ("coords", ctypes.c_void_p),
                ("type_index", ctypes.c_void_p), ("type_vector", ctypes.c_void_p),
                ("radii", ctypes.c_void_p), ("centers", ctypes.c_void_p),
                ("center_host", ctypes.c_float * 3),
                ("transforms", ctypes.c_void_p), ("transform_host", ctypes.POINTER(TransformStruct))]


class InterpolaterStruct(ctypes.Structure):
    _fields_ = [("in_resolution", ctypes.c_float), ("in_dimension", ctypes.c_float),
                ("out_resolution", ctypes.c_float), ("out_dimension", ctypes.c_float),
                ("in_dim", ctypes.c_uint), ("out_dim", ctypes.c_uint)]


class RecordSetStruct(ctypes.Structure):
    _fields_ = [("first_record", ctypes.c_longlong), ("count", ctypes.c_int), ("example", ctypes.c_int),
                ("typer", ctypes.c_int), ("type_offset", ctypes.c_int), ("dst_atom", ctypes.c_int),
                ("is_center_set", ctypes.c_int)]


RECORD_TYPES = 28

# every symbol include/lmg_b200.h declares: (name, restype, argtypes)
_VP = ctypes.c_void_p
_GM = ctypes.POINTER(GridMakerStruct)
_AT = ctypes.POINTER(AtomsStruct)
_TR = ctypes.POINTER(TransformStruct)
_GI = ctypes.POINTER(InterpolaterStruct)
SYMBOLS = [
    ("lmg_gridmaker_init", ctypes.c_int, [_GM, ctypes.c_float, ctypes.c_float, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_float, ctypes.c_float]),
    ("lmg_transform_random", ctypes.c_int, [_TR, ctypes.c_float * 3, ctypes.c_float, ctypes.c_int]),
    ("lmg_transform_random_batch", ctypes.c_int, [_VP, ctypes.c_int, ctypes.c_float * 3, ctypes.c_float,
                                                  ctypes.c_int]),
    ("lmg_set_random_seed", None, [ctypes.c_uint]),
    ("lmg_workspace_bytes", ctypes.c_size_t, [_GM, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_int]),
    ("lmg_forward", ctypes.c_int, [_GM, _AT, _VP, _VP, ctypes.c_size_t, _VP]),
    ("lmg_backward", ctypes.c_int, [_GM, _AT, _VP, _VP, _VP, _VP, ctypes.c_size_t, _VP]),
    ("lmg_backward_gradients", ctypes.c_int, [_GM, _AT, _VP, _VP, _VP, _VP, _VP, _VP, _VP,
                                              ctypes.c_size_t, _VP]),
    ("lmg_backward_relevance", ctypes.c_int, [_GM, _AT, _VP, _VP, _VP, _VP, ctypes.c_size_t, _VP]),
    ("lmg_backward_static", ctypes.c_int, [_GM, _AT, _VP, _VP, _VP]),
    ("lmg_static_max_atoms", ctypes.c_size_t, []),
    ("lmg_static_check_status", ctypes.c_int, [_VP]),
    ("lmg_transform_forward", ctypes.c_int, [_TR, ctypes.c_int, _VP, _VP, ctypes.c_int, _VP]),
    ("lmg_transform_backward", ctypes.c_int, [_TR, ctypes.c_int, _VP, _VP, ctypes.c_int, _VP]),
    ("lmg_interpolater_init", ctypes.c_int, [_GI, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                                             ctypes.c_float]),
    ("lmg_interpolate", ctypes.c_int, [_GI, ctypes.c_int, ctypes.c_int, _VP, _TR, c_float_p, c_float_p,
                                       _VP, _VP]),
    ("lmg_interpolate_backward", ctypes.c_int, [_GI, ctypes.c_int, ctypes.c_int, _VP, _TR, c_float_p, c_float_p,
                                                _VP, _VP]),
    ("lmg_decode_records", ctypes.c_int, [_VP, _VP, ctypes.c_int, _VP, _VP, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_int, _VP, _VP, _VP, _VP, _VP, _VP, _VP]),
    ("lmg_gather_host", ctypes.c_int, [_VP, ctypes.c_size_t, ctypes.c_int, _VP, _VP]),
    ("lmg_sum_types", ctypes.c_int, [_VP, _VP, ctypes.c_int, ctypes.c_int, _VP, ctypes.c_int, _VP, _VP]),
    ("lmg_check_status", ctypes.c_int, [_VP, _VP]),
    ("lmg_last_error", ctypes.c_char_p, []),
    ("lmg_version", ctypes.c_int, []),
]
# tuning knobs outside the reference interface
EXTRA_SYMBOLS = [
    ("lmg_set_precise", None, [ctypes.c_int]),
    ("lmg_set_quads", None, [ctypes.c_int]),
    ("lmg_set_interp_tiled", None, [ctypes.c_int]),
    ("lmg_tma_timeouts", ctypes.c_uint, []),
    # bench support
    ("lmg_profile_enable", ctypes.c_int, [ctypes.c_int]),
    ("lmg_profile_collect", ctypes.c_int, [ctypes.POINTER(ctypes.c_double), c_int_p]),
    ("lmg_launch_count", ctypes.c_long, []),
]

_lib = None


def lib():
    """The loaded library; raises if it is missing (build it with ``python -m libmolgrid_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "liblmg_b200.so is not built (%s); run `python -m libmolgrid_b200.build`. "
                "There is no CPU fallback." % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, res, args in SYMBOLS + EXTRA_SYMBOLS:
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc):
    """Re-raise a C ABI status as the exception type the reference's Python module raises."""
    if rc == LMG_OK:
        return
    msg = lib().lmg_last_error().decode()
    if rc == LMG_ERR_OUT_OF_RANGE:
        raise IndexError(msg)
    if rc == LMG_ERR_INVALID_ARGUMENT:
        raise ValueError(msg)
    raise RuntimeError(msg)
