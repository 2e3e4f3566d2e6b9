"""ctypes front end of the CPU oracle (``cuv_host_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``; never by the
product package.  All matrices are float32 numpy arrays in column-major
(Fortran) order, as CUV's ``tensor<float, host_memory_space, column_major>``.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcuv_host_oracle.so")

RF_ADD, RF_MEAN, RF_ADD_SQUARED, RF_MAX, RF_ARGMAX, RF_ARGMIN, RF_MIN, RF_MULT, RF_LOGADDEXP, RF_ADDEXP = range(10)

_f32p = ctypes.POINTER(ctypes.c_float)
_i32p = ctypes.POINTER(ctypes.c_int)


def build(force=False):
    """Compile the oracle with the Makefile beside it (gcc, seconds)."""
    src = os.path.join(_HERE, "cuv_host_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        L.oracle_dia_cell_index.restype = ctypes.c_long
        L.oracle_dia_cell_index.argtypes = [ctypes.c_int] * 5 + [_i32p, ctypes.c_int, ctypes.c_int]
        L.oracle_dia_to_dense.restype = None
        L.oracle_dia_to_dense.argtypes = [_f32p] + [ctypes.c_int] * 5 + [_i32p, _f32p]
        L.oracle_prod_dia.restype = ctypes.c_int
        L.oracle_prod_dia.argtypes = [_f32p, ctypes.c_int, _f32p, _i32p] + [ctypes.c_int] * 5 + [
            _f32p, ctypes.c_int, ctypes.c_int, ctypes.c_char, ctypes.c_float, ctypes.c_float, ctypes.c_int]
        L.oracle_dd2dia.restype = ctypes.c_int
        L.oracle_dd2dia.argtypes = [_f32p, _i32p] + [ctypes.c_int] * 5 + [
            _f32p, ctypes.c_int, _f32p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float,
            ctypes.c_int, ctypes.c_int]
        L.oracle_reduce.restype = ctypes.c_int
        L.oracle_reduce.argtypes = [_f32p, _f32p, ctypes.c_long, ctypes.c_long, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_float, ctypes.c_float, ctypes.c_int]
        L.oracle_bias_sigmoid_sample.restype = None
        L.oracle_avg_diagonals.argtypes = [_f32p, _f32p, _i32p] + [ctypes.c_int] * 5
        L.oracle_reduce_typed.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_long,
                                          ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float]
        L.oracle_bias_sigmoid_sample.argtypes = [_f32p, _f32p, _f32p, _f32p, ctypes.c_long, ctypes.c_long,
                                                 ctypes.c_int]
        L.oracle_learn_step_weight_decay.restype = None
        L.oracle_learn_step_weight_decay.argtypes = [_f32p, _f32p, ctypes.c_long, ctypes.c_float, ctypes.c_float]
        L.oracle_learn_step_weight_decay_momentum.restype = None
        L.oracle_learn_step_weight_decay_momentum.argtypes = [_f32p, _f32p, _f32p, ctypes.c_long, ctypes.c_float,
                                                              ctypes.c_float, ctypes.c_float, ctypes.c_int]
        L.oracle_philox4x32_10.restype = None
        L.oracle_philox4x32_10.argtypes = [ctypes.c_void_p] * 3
        L.oracle_uniform.restype = None
        L.oracle_uniform.argtypes = [_f32p, ctypes.c_long, ctypes.c_long, ctypes.c_long, ctypes.c_ulonglong,
                                     ctypes.c_ulonglong, ctypes.c_longlong, ctypes.c_int]
        _lib = L
    return _lib


def _fp(a):
    return a.ctypes.data_as(_f32p) if a is not None else None


def _ip(a):
    return a.ctypes.data_as(_i32p)


def _colmajor(a, name):
    assert a.dtype == np.float32 and a.ndim == 2 and a.flags.f_contiguous, name + " must be float32 column-major"


class DiaHost:
    """Mirror of ``dia_matrix<float, host_memory_space>`` (basics/dia_matrix.hpp:57-276):
    ``num_dia`` diagonals of ``stride`` floats back to back, int32 offsets in user order."""

    def __init__(self, h, w, offsets, stride=None, row_fact=1, vals=None):
        self.h, self.w, self.rf = int(h), int(w), int(row_fact)
        self.offsets = np.ascontiguousarray(offsets, dtype=np.int32)
        self.nd = int(self.offsets.size)
        self.stride = int(stride) if stride is not None else max(self.h, self.w)
        assert self.rf > 0 and self.stride >= self.h
        if vals is None:
            vals = np.zeros(self.nd * self.stride, dtype=np.float32)
        self.vals = np.ascontiguousarray(vals, dtype=np.float32).reshape(-1)
        assert self.vals.size == self.nd * self.stride

    def cell_index(self, i, j):
        return lib().oracle_dia_cell_index(self.h, self.w, self.rf, self.stride, self.nd, _ip(self.offsets), i, j)

    def to_dense(self):
        d = np.zeros((self.h, self.w), dtype=np.float32, order="F")
        lib().oracle_dia_to_dense(_fp(d), self.h, self.w, self.rf, self.stride, self.nd, _ip(self.offsets),
                                  _fp(self.vals))
        return d

    def valid_mask(self):
        """Boolean [nd, stride] mask of the cells prod/densedense_to_dia may touch
        (row_start <= i < row_start+N per diagonal, matrix_ops/spmv.cu:185-189)."""
        m = np.zeros((self.nd, self.stride), dtype=bool)
        for s, k in enumerate(self.offsets.tolist()):
            r0 = self.rf * max(0, -k)
            n = min(self.h - r0, self.rf * (self.w - max(0, k)))
            if n > 0:
                m[s, r0:r0 + n] = True
        return m

    def nnz(self):
        return int(self.valid_mask().sum())


def prod(C, A, B, transA="n", factAB=1.0, factC=0.0, nthreads=1):
    """C = factC*C + factAB*op(A)*B, in place on C (matrix_ops/spmv.cu:203-220)."""
    _colmajor(B, "B"); _colmajor(C, "C")
    assert B.shape[1] == C.shape[1]
    if transA == "t":
        assert B.shape[0] == A.h and C.shape[0] == A.w
    else:
        assert B.shape[0] == A.w and C.shape[0] == A.h
    rc = lib().oracle_prod_dia(_fp(C), C.shape[0], _fp(A.vals), _ip(A.offsets), A.nd, A.h, A.w, A.stride, A.rf,
                               _fp(B), B.shape[0], B.shape[1], transA.encode(), factAB, factC, nthreads)
    if rc:
        raise RuntimeError("oracle_prod_dia: bad arguments")
    return C


def densedense_to_dia(Cdia, A, B, factAB=1.0, factC=0.0, literal_host=False, nthreads=1):
    """C_dia = factC*C_dia + factAB*(A*B^T restricted to the stored diagonals), in place."""
    _colmajor(A, "A"); _colmajor(B, "B")
    assert A.shape[0] == Cdia.h and B.shape[0] == Cdia.w and A.shape[1] == B.shape[1]
    rc = lib().oracle_dd2dia(_fp(Cdia.vals), _ip(Cdia.offsets), Cdia.nd, Cdia.h, Cdia.w, Cdia.stride, Cdia.rf,
                             _fp(A), A.shape[0], _fp(B), B.shape[0], A.shape[1], factAB, factC,
                             1 if literal_host else 0, nthreads)
    if rc:
        raise RuntimeError("oracle_dd2dia: bad arguments")
    return Cdia


def reduce(dst, src, over_strided, rf=RF_ADD, factNew=1.0, factOld=0.0, nthreads=1):
    """dst = factOld*dst + factNew*rf(src) for a column-major 2-D ``src``:
    ``over_strided`` True sums over columns (one output per row), False sums along
    each column (one output per column)."""
    _colmajor(src, "src")
    n_contig, n_strided = src.shape
    assert dst.dtype == np.float32 and dst.size == (n_contig if over_strided else n_strided)
    rc = lib().oracle_reduce(_fp(dst), _fp(src), n_contig, n_strided, 1 if over_strided else 0, rf,
                             factNew, factOld, nthreads)
    if rc:
        raise RuntimeError("oracle_reduce: bad arguments")
    return dst


def reduce_to_col(dst, src, rf=RF_ADD, factNew=1.0, factOld=0.0, nthreads=1):
    """Column-major src: dst[i] = reduce over j of src[i, j] (matrix_ops_reduce.cu:348-362)."""
    return reduce(dst, src, True, rf, factNew, factOld, nthreads)


def reduce_to_row(dst, src, rf=RF_ADD, factNew=1.0, factOld=0.0, nthreads=1):
    """Column-major src: dst[j] = reduce over i of src[i, j] (matrix_ops_reduce.cu:364-379)."""
    return reduce(dst, src, False, rf, factNew, factOld, nthreads)


def avg_diagonals(dst, A):
    """dst[k] = mean of stored diagonal k over the cells inside the matrix (matrix_ops/diagonals.cu:23-48)."""
    assert dst.dtype == np.float32 and dst.size == A.offsets.size
    if lib().oracle_avg_diagonals(_fp(dst), _fp(A.vals), A.offsets.ctypes.data_as(_i32p), A.offsets.size, A.h, A.w,
                                  A.stride, A.rf):
        raise RuntimeError("oracle_avg_diagonals: row_fact must be 1")
    return dst


TYPE_CODES = {np.dtype(np.float32): 0, np.dtype(np.int32): 1, np.dtype(np.uint32): 2, np.dtype(np.uint8): 3}


def reduce_typed(dst, src, over_strided, rf=RF_ADD, factNew=1.0, factOld=0.0):
    """The reduction between the element types CUV instantiates besides float -> float
    (matrix_ops/matrix_ops_reduce.cu:395-413), with the host loop's semantics: running value in the SOURCE type,
    fold in the DESTINATION type, factors converted to the source type.  ``src`` column-major 2-D, ``dst`` 1-D."""
    _colmajor_any(src)
    n_contig, n_strided = src.shape
    assert dst.size == (n_contig if over_strided else n_strided) and dst.flags.c_contiguous
    rc = lib().oracle_reduce_typed(dst.ctypes.data, TYPE_CODES[dst.dtype], src.ctypes.data, TYPE_CODES[src.dtype],
                                   n_contig, n_strided, 1 if over_strided else 0, rf, factNew, factOld)
    if rc:
        raise RuntimeError("oracle_reduce_typed: pair of types or functor not instantiated by CUV")
    return dst


def _colmajor_any(a):
    assert a.ndim == 2 and a.flags.f_contiguous, "column-major 2-D array expected"


def bias_sigmoid_sample(act, bias=None, u=None, nthreads=1):
    """act <- sigmoid(act + bias[:, None]) in place; returns (act > u) as 0/1 floats if u is given."""
    _colmajor(act, "act")
    sample = None
    if u is not None:
        _colmajor(u, "u")
        sample = np.empty_like(act, order="F")
    lib().oracle_bias_sigmoid_sample(_fp(act), _fp(bias), _fp(u), _fp(sample), act.shape[0], act.shape[1], nthreads)
    return sample


def philox4x32_10(counter, key):
    """The generator's block function: four counter words and two key words -> four output words."""
    c = np.asarray(counter, dtype=np.uint32).copy()
    k = np.asarray(key, dtype=np.uint32).copy()
    out = np.zeros(4, dtype=np.uint32)
    lib().oracle_philox4x32_10(c.ctypes.data, k.ctypes.data, out.ctypes.data)
    return out


def uniform(rows, ncols, seed, step=0, col0=0, which=0):
    """The uniform numbers of draw ``which`` in step ``step`` for the batch columns col0 .. col0 + ncols - 1, as a
    column-major float32 matrix (what the product path's sampling passes draw on the device)."""
    dst = np.empty((rows, ncols), dtype=np.float32, order="F")
    lib().oracle_uniform(_fp(dst), rows, rows, ncols, seed, step, col0, which)
    return dst


def learn_step_weight_decay(W, dW, learnrate, decay=0.0):
    """W = -learnrate*dW + (1 - learnrate*decay)*W in place on flat float32 arrays (tensor_ops/rprop.cu:331-346)."""
    assert W.dtype == np.float32 and dW.dtype == np.float32 and W.size == dW.size
    assert W.flags.c_contiguous or W.flags.f_contiguous
    lib().oracle_learn_step_weight_decay(_fp(W), _fp(dW), W.size, learnrate, decay)
    return W


def learn_step_weight_decay_momentum(W, M, dW, learnrate, momentum_weight=0.9, decay=0.0, device_formula=True):
    """Momentum step in place (tensor_ops/rprop.cu:158-170 device formula, :356-367 host loop)."""
    assert W.dtype == M.dtype == dW.dtype == np.float32 and W.size == dW.size == M.size
    lib().oracle_learn_step_weight_decay_momentum(_fp(W), _fp(M), _fp(dW), W.size, learnrate, momentum_weight, decay,
                                                  1 if device_formula else 0)
    return W
