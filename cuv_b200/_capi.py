"""ctypes bindings of ``libcuvdia.so`` (declared in ``include/cuvdia.h``).

The library is the only implementation: if it is missing the import fails, there is no fallback.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcuvdia.so")

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_NOMEM = range(5)
MODE_EXACT, MODE_FAST = 0, 1
T_F32, T_I32, T_U32, T_U8 = range(4)
(RF_ADD, RF_MEAN, RF_ADD_SQUARED, RF_MAX, RF_ARGMAX, RF_ARGMIN, RF_MIN, RF_MULT, RF_LOGADDEXP,
 RF_ADDEXP) = range(10)

# every symbol include/cuvdia.h declares: name -> (restype, argtypes)
_vp, _i, _ll, _f, _c = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_char
SIGNATURES = {
    "cuvdia_error_string": (ctypes.c_char_p, [_i]),
    "cuvdia_last_error_message": (ctypes.c_char_p, []),
    "cuvdia_launch_count": (ctypes.c_ulonglong, []),
    "cuvdia_release_workspaces": (_i, []),
    "cuvdia_plan_create": (_i, [ctypes.POINTER(_vp), _i, _i, _i, _i, _i, ctypes.POINTER(_i)]),
    "cuvdia_plan_destroy": (_i, [_vp]),
    "cuvdia_plan_info": (_i, [_vp, ctypes.POINTER(_i), ctypes.POINTER(_ll)]),
    "cuvdia_plan_offsets_device": (_vp, [_vp]),
    "cuvdia_plan_status": (_i, [_vp, ctypes.POINTER(_i)]),
    "cuvdia_plan_status_clear": (_i, [_vp, _vp]),
    "cuvdia_selftest_bounded_wait": (_i, [_vp, ctypes.c_uint, _vp]),
    "cuvdia_prod_f32": (_i, [_vp, _vp, _vp, _i, _vp, _i, _i, _c, _c, _f, _f, _i, _vp]),
    "cuvdia_prod_bias_sigmoid_sample_f32": (_i, [_vp, _vp, _vp, _i, _vp, _i, _i, _c, _f, _f, _i, _vp, _vp, _i, _vp, _i,
                                                 _vp]),
    "cuvdia_dd2dia_f32": (_i, [_vp, _vp, _vp, _i, _vp, _i, _i, _f, _f, _vp]),
    "cuvdia_avg_diagonals_f32": (_i, [_vp, _vp, _vp, _vp]),
    "cuvdia_reduce_f32": (_i, [_vp, _vp, _ll, _ll, _i, _i, _f, _f, _vp]),
    "cuvdia_reduce": (_i, [_vp, _i, _vp, _i, _ll, _ll, _i, _i, _f, _f, _vp]),
    "cuvdia_reduce_noalloc_f32": (_i, [_vp, _vp, _ll, _ll, _i, _i, _f, _f, _vp]),
    "cuvdia_bias_sigmoid_sample_f32": (_i, [_vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _vp]),
    "cuvdia_bias_sigmoid_sample_sum_f32": (_i, [_vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _vp, _i, _f, _f, _i, _vp]),
    "cuvdia_rbm_cd1_step_f32": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "cuvdia_uniform_f32": (_i, [_vp, _i, _i, _i, _vp, _i, _vp]),
    "cuvdia_rnd_binarize_f32": (_i, [_vp, _i, _i, _i, _vp, _i, _vp]),
    "cuvdia_bias_sigmoid_draw_sum_f32": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _i, _f, _f, _i, _vp, _i, _vp]),
    "cuvdia_rbm_cd1_step_drawn_f32": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "cuvdia_rbm_cd1_step_drawn_allreduce_f32": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp]),
    "cuvdia_rbm_cd1_step_allreduce_f32": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "cuvdia_allreduce_grad": (_i, [_vp, _vp, _ll, _vp, _ll, _vp]),
    "cuvdia_nccl_unique_id": (_i, [ctypes.c_char_p]),
    "cuvdia_nccl_comm_create": (_i, [ctypes.POINTER(_vp), _i, _i, ctypes.c_char_p]),
    "cuvdia_nccl_comm_destroy": (_i, [_vp]),
    "cuvdia_axpby_f32": (_i, [_vp, _vp, _vp, _f, _f, _ll, _vp]),
    "cuvdia_learn_step_weight_decay_f32": (_i, [_vp, _vp, _ll, _f, _f, _vp]),
    "cuvdia_learn_step_weight_decay_momentum_f32": (_i, [_vp, _vp, _vp, _ll, _f, _f, _f, _vp]),
    "cuvdia_binary_f32": (_i, [_vp, _vp, _vp, _i, _f, _f, _ll, _vp]),
    "cuvdia_fill_f32": (_i, [_vp, _f, _ll, _vp]),
    "cuvdia_sequence_f32": (_i, [_vp, _ll, _vp]),
}


class Draw(ctypes.Structure):
    """``cuvdia_draw`` of include/cuvdia.h."""
    _fields_ = [("seed", ctypes.c_ulonglong), ("step", ctypes.c_ulonglong), ("col0", ctypes.c_longlong)]


class RbmCd1Buffers(ctypes.Structure):
    """``cuvdia_rbm_cd1_buffers`` of include/cuvdia.h."""
    _fields_ = [(n, _vp) for n in ("V0", "U_h", "U_v", "b_vis", "c_hid", "H0p", "H0", "V1p", "V1", "H1p", "G_vals",
                                   "gc", "gb")]


class CuvDiaError(RuntimeError):
    """Raised for any non-zero return code; the message is the failed precondition, as the
    ``std::runtime_error`` thrown by CUV's ``cuvAssert`` (tools/cuv_general.cu:45-50)."""

    def __init__(self, code, message):
        super().__init__("%s: %s" % (lib().cuvdia_error_string(code).decode(), message))
        self.code = code


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: build it with `python -m cuv_b200.build` "
                              "(there is no fallback implementation)" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(code):
    if code != OK:
        raise CuvDiaError(code, lib().cuvdia_last_error_message().decode())
