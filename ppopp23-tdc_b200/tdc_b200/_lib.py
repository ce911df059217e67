"""ctypes binding of libtdc_b200.so — one Python prototype per declaration in
include/tdc_b200.h, nothing else.  There is no CPU fallback: if the library is missing the
import raises, and every call that fails raises TdcError with the library's message."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# TDC_B200_LIB names another build of the same library (a measurement build, say); the default is the one build.py makes
LIB_PATH = os.environ.get("TDC_B200_LIB") or os.path.join(_HERE, "libtdc_b200.so")

OK, ERR_NULL, ERR_SHAPE, ERR_UNSUPPORTED, ERR_TILE, ERR_SMEM, ERR_CUDA, ERR_WORKSPACE, ERR_NO_DEVICE = range(9)
W_KCRS, W_CRSK = 0, 1
EPI_NONE, EPI_RELU = 0, 1


class TdcError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("tdc_b200 status %d: %s" % (code, msg))
        self.code = code


class Tile(C.Structure):
    """tdc_tile; th/tw/tc as in the reference generators' TH/TW/TC
    (A100-evaluation/TDC-LAYERS-ORACLE/gen_from_occupancy.py:113-139)."""
    _fields_ = [(n, C.c_int) for n in ("th", "tw", "tc", "tn", "nog", "gy", "gx", "imgs", "ks", "kc")]

    def as_tuple(self):
        return tuple(getattr(self, n) for n, _ in self._fields_)

    def __repr__(self):
        return "Tile(" + ", ".join("%s=%d" % (n, getattr(self, n)) for n, _ in self._fields_) + ")"


class Epilogue(C.Structure):
    """tdc_epilogue: y = relu?(conv * scale[k] + bias[k] + residual); NULL pointers are skipped."""
    _fields_ = [("scale", C.c_void_p), ("bias", C.c_void_p), ("residual", C.c_void_p), ("relu", C.c_int)]


class TcPlan(C.Structure):
    """tdc_tc_plan: layer-shape facts of the tensor-core variant."""
    _fields_ = [(n, C.c_int) for n in ("C", "K", "R", "S", "mode", "nt", "cb", "nkb", "n_ocb", "hl", "general", "stride", "phase")] + \
               [("weights_bytes", C.c_size_t)]


class DevInfo(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("sm_count", "smem_per_cta", "regs_per_sm", "threads_per_sm")]


class LaunchInfo(C.Structure):
    _fields_ = [("grid_x", C.c_int), ("grid_y", C.c_int), ("threads", C.c_int), ("smem_bytes", C.c_size_t),
                ("regs_per_thread", C.c_int), ("ctas_per_sm", C.c_int)]


# B200 as the selector sees it when no device can be queried (CPU-side tests, table tools).
B200 = DevInfo(148, 232448, 65536, 2048)
STATIC_WORKSPACE_BYTES = 32 << 20   # TDC_STATIC_WORKSPACE_BYTES

_i, _p, _sz = C.c_int, C.c_void_p, C.c_size_t
_PROTOTYPES = {
    "tdc_last_error_string": (C.c_char_p, []),
    "tdc_version": (_i, []),
    "tdc_query_device": (_i, [_i, C.POINTER(DevInfo)]),
    "tdc_core_conv2d_f32": (_i, [_p, _p, _p] + [_i] * 10 + [C.POINTER(Tile), _p]),
    "tdc_conv2d_f32": (_i, [_p, _p, _p, _p] + [_i] * 11 + [C.POINTER(Tile), _p]),
    "tdc_conv2d_epi_f32": (_i, [_p, _p, _p] + [_i] * 10 + [C.POINTER(Epilogue), C.POINTER(Tile), _p]),
    "tdc_tk_block_epi_f32": (_i, [_p] * 5 + [_i] * 12 + [C.POINTER(Epilogue), C.POINTER(Tile), _p, _sz, _p]),
    "tdc_permute_weights": (_i, [_p, _p, _i, _i, _i, _i, _p]),
    "tdc_tc_last_error_string": (C.c_char_p, []),
    "tdc_pool2d_f32": (_i, [_p, _p] + [_i] * 9 + [_p]),
    "tdc_affine_relu_f32": (_i, [_p, _p, _p, _p, _i, _i, _i, C.c_longlong, C.c_longlong, _i, _p]),
    "tdc_tc_plan_make": (_i, [_i] * 5 + [C.POINTER(TcPlan)]),
    "tdc_tc_plan_make_general": (_i, [_i] * 5 + [C.POINTER(TcPlan)]),
    "tdc_tc_plan_make_strided": (_i, [_i] * 8 + [C.POINTER(TcPlan)]),
    "tdc_tc_pick_nt": (_i, [_i, _i, C.c_longlong, _i]),
    "tdc_tc_plan_make_nt": (_i, [_i] * 7 + [C.POINTER(TcPlan)]),
    "tdc_tc_prepare_weights": (_i, [C.POINTER(TcPlan), _p, _i, _p, _p]),
    "tdc_conv2d_tc": (_i, [C.POINTER(TcPlan), _p, _p, _p, _i, _i, _i, C.POINTER(Epilogue), _i, _p]),
    "tdc_conv2d_tc_ranged": (_i, [C.POINTER(TcPlan), _p, _p, _p, _i, _i, _i, C.POINTER(Epilogue), _i, _p, _p, _p]),
    "tdc_tc_check_launch": (_i, [C.POINTER(TcPlan), _i, _i, _i, _i]),
    "tdc_tc_status": (_i, [C.POINTER(_i)]),
    "tdc_select_tile": (_i, [_i] * 9 + [C.POINTER(DevInfo), C.POINTER(Tile)]),
    "tdc_tile_info": (_i, [_i] * 9 + [C.POINTER(Tile), C.POINTER(LaunchInfo)]),
    "tdc_tile_cost": (_i, [_i] * 9 + [C.POINTER(Tile), C.POINTER(DevInfo), C.POINTER(C.c_double),
                                      C.POINTER(C.c_double)]),
    "tdc_tk_block_workspace_bytes": (_sz, [_i] * 11),
    "tdc_tk_block_f32": (_i, [_p] * 6 + [_i] * 13 + [C.POINTER(Tile), _p, _sz, _p]),
    "tdc_tk_block_f32_static": (_i, [_p] * 6 + [_i] * 13 + [C.POINTER(Tile), _p]),
    "tdc_conv_create": (_i, [C.POINTER(_p)] + [_i] * 9 + [_p, _p]),
    "tdc_conv_set_tile": (_i, [_p, C.POINTER(Tile)]),
    "tdc_conv_set_precision": (_i, [_p, _i]),
    "tdc_conv_forward": (_i, [_p, _p, C.POINTER(_p), _p]),
    "tdc_conv_forward_host": (_i, [_p, _p, _p]),
    "tdc_conv_forward_host_async": (_i, [_p, _p, _p, _p]),
    "tdc_conv_destroy": (None, [_p]),
    "tdc_tkconv_create": (_i, [C.POINTER(_p)] + [_i] * 11 + [_p] * 4),
    "tdc_tkconv_set_precision": (_i, [_p, _i]),
    "tdc_tkconv_forward": (_i, [_p, _p, C.POINTER(_p), _p]),
    "tdc_tkconv_forward_host": (_i, [_p, _p, _p]),
    "tdc_tkconv_destroy": (None, [_p]),
}
EXPORTS = tuple(_PROTOTYPES)


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libtdc_b200.so is not built (%s). Run `python ppopp23-tdc_b200/build.py`; "
            "this package has no fallback path." % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _PROTOTYPES.items():
        fn = getattr(lib, name)   # AttributeError here = header and library disagree
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def check(code):
    if code != OK:
        raise TdcError(code, lib.tdc_last_error_string().decode())
