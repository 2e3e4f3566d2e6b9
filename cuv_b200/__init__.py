"""B200 implementation of CUV's DIA sparse hot path - Python mirror of the reference interface.

The names follow CUV's disabled Python export of the same routines
(``src/cuv_python/export_dia_mat.cpp:212-235``): ``dev_dia_matrix_f``, ``dev_block_descriptor_f``,
``prod``, ``densedense_to_dia``, ``reduce_to_col`` / ``reduce_to_row``.  Every call goes through the C ABI
of ``libcuvdia.so`` (``include/cuvdia.h``); torch only provides device memory and streams.

Dense matrices are CUV's ``tensor<float, dev_memory_space, column_major>``: here a 2-D CUDA torch tensor of
logical shape ``(rows, cols)`` whose rows are contiguous (``stride(0) == 1``); make one with
:func:`colmajor_empty` or :func:`to_device`.
"""
import ctypes

import numpy as np

from . import _capi
from ._capi import (CuvDiaError, MODE_EXACT, MODE_FAST, RF_ADD, RF_MEAN, RF_ADD_SQUARED, RF_MAX, RF_ARGMAX,
                    RF_ARGMIN, RF_MIN, RF_MULT, RF_LOGADDEXP, RF_ADDEXP)

__all__ = ["dev_dia_matrix_f", "host_dia_matrix_f", "filter_factory", "convert", "pull", "save_dia_mat", "load_dia_mat", "dev_block_descriptor_f", "prod", "spmv", "densedense_to_dia", "reduce_to_col",
           "reduce_to_row", "avg_diagonals", "bias_sigmoid_sample", "bias_sigmoid_sample_sum", "prod_bias_sigmoid_sample", "axpby", "learn_step_weight_decay",
           "learn_step_weight_decay_momentum", "colmajor_empty", "to_device", "to_host",
           "launch_count", "plan_status", "raise_if_gave_up", "CuvDiaError", "MODE_EXACT", "MODE_FAST"]


def _torch():
    import torch
    return torch


def _stream():
    return ctypes.c_void_p(_torch().cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def launch_count():
    """Kernels launched by the library so far in this process."""
    return int(_capi.lib().cuvdia_launch_count())


# ---- dense column-major helpers ---------------------------------------------------------------------

def colmajor_empty(rows, cols, device="cuda"):
    torch = _torch()
    return torch.empty((cols, rows), dtype=torch.float32, device=device).t()


def to_device(a, device="cuda"):
    """numpy (any layout) -> column-major CUDA matrix, or 1-D vector."""
    torch = _torch()
    a = np.asarray(a, dtype=np.float32)
    if a.ndim == 1:
        return torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return torch.from_numpy(np.ascontiguousarray(a.T)).to(device).t()


def to_host(t):
    """CUDA matrix -> float32 Fortran-ordered numpy array (or 1-D array)."""
    if t.dim() == 1:
        return t.detach().cpu().numpy()
    return np.asfortranarray(t.detach().cpu().numpy())


def _check_colmajor(t, name):
    torch = _torch()
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32 and t.dim() == 2):
        raise CuvDiaError(_capi.ERR_INVALID, name + " must be a 2-D float32 CUDA tensor")
    if t.shape[0] > 1 and t.stride(0) != 1:
        raise CuvDiaError(_capi.ERR_INVALID, name + " must be column-major (stride(0) == 1)")
    ld = t.stride(1) if t.shape[1] > 1 else t.shape[0]
    if ld < t.shape[0]:
        raise CuvDiaError(_capi.ERR_INVALID, name + " has overlapping columns")
    return int(ld)


# ---- dia_matrix<float, dev_memory_space> -------------------------------------------------------------------

class dev_dia_matrix_f:
    """``dia_matrix<float, dev_memory_space>`` (basics/dia_matrix.hpp:57-276): ``num_dia`` diagonals of
    ``stride`` floats stored back to back in ``vec``; cell (i, j) lives at ``vec[slot(j - i//rf)*stride + i]``;
    ``offsets`` keeps the caller's order.  Owns a plan (device offsets + kernel metadata)."""

    def __init__(self, h, w, offsets, stride=None, row_fact=1, device="cuda"):
        torch = _torch()
        self.h, self.w, self.row_fact = int(h), int(w), int(row_fact)
        self.offsets = np.ascontiguousarray(offsets, dtype=np.int32).reshape(-1)
        self.num_dia = int(self.offsets.size)
        self.stride = int(stride) if stride is not None else max(self.h, self.w)
        self._plan = ctypes.c_void_p()
        with torch.cuda.device(torch.device(device)):
            _capi.check(_capi.lib().cuvdia_plan_create(
                ctypes.byref(self._plan), self.h, self.w, self.num_dia, self.stride, self.row_fact,
                self.offsets.ctypes.data_as(ctypes.POINTER(ctypes.c_int))))
        self.vec = torch.empty(self.num_dia * self.stride, dtype=torch.float32, device=device)   # uninitialised, as CUV
        band, nnz = ctypes.c_int(), ctypes.c_longlong()
        _capi.check(_capi.lib().cuvdia_plan_info(self._plan, ctypes.byref(band), ctypes.byref(nnz)))
        self.is_band, self.nnz = bool(band.value), int(nnz.value)

    def __del__(self):
        plan, self._plan = getattr(self, "_plan", None), None
        if plan:
            try:
                _capi.lib().cuvdia_plan_destroy(plan)
            except Exception:
                pass

    def __len__(self):
        return self.h * self.w

    @property
    def shape(self):
        return (self.h, self.w)

    def dia(self, k):
        """View on the storage of diagonal number ``k`` (dia_matrix.hpp:199-217)."""
        slot = int(np.nonzero(self.offsets == k)[0][-1])
        return self.vec[slot * self.stride:(slot + 1) * self.stride]

    def has(self, i, j):
        return bool(np.any(self.offsets == j - i // self.row_fact))

    def __call__(self, i, j):
        hit = np.nonzero(self.offsets == j - i // self.row_fact)[0]
        return float(self.vec[int(hit[-1]) * self.stride + i]) if hit.size else 0.0

    def set(self, i, j, val):
        hit = np.nonzero(self.offsets == j - i // self.row_fact)[0]
        if hit.size:
            self.vec[int(hit[-1]) * self.stride + i] = val

    def set_vec(self, vals):
        """Copy host values (num_dia*stride floats) into the matrix: the host->device ``convert``
        (convert/convert.cu:71-90)."""
        v = np.ascontiguousarray(vals, dtype=np.float32).reshape(-1)
        if v.size != self.num_dia * self.stride:
            raise CuvDiaError(_capi.ERR_INVALID, "vals.size == num_dia*stride")
        self.vec.copy_(_torch().from_numpy(v))
        return self


class host_dia_matrix_f:
    """``dia_matrix<float, host_memory_space>``: the same container with numpy storage.  It only holds
    data (conversion source/target); there is no host implementation of the products here."""

    def __init__(self, h, w, offsets, stride=None, row_fact=1):
        self.h, self.w, self.row_fact = int(h), int(w), int(row_fact)
        self.offsets = np.ascontiguousarray(offsets, dtype=np.int32).reshape(-1)
        self.num_dia = int(self.offsets.size)
        self.stride = int(stride) if stride is not None else max(self.h, self.w)
        self.vec = np.empty(self.num_dia * self.stride, dtype=np.float32)

    @property
    def shape(self):
        return (self.h, self.w)

    def _slot(self, i, j):
        hit = np.nonzero(self.offsets == j - i // self.row_fact)[0]
        return int(hit[-1]) if hit.size else None

    def has(self, i, j):
        return self._slot(i, j) is not None

    def __call__(self, i, j):
        s = self._slot(i, j)
        return float(self.vec[s * self.stride + i]) if s is not None else 0.0

    def set(self, i, j, val):
        s = self._slot(i, j)
        if s is not None:
            self.vec[s * self.stride + i] = val


_DIA_MAGIC = b"CUVDIA1\0"


def save_dia_mat(mat, filename):
    """Write a DIA matrix (host or device) to a file: the seven fields CUV serialises - width, height,
    num_dia, stride, row_fact, offsets, values (basics/sparse_matrix_io.hpp:59-72), in that order - as a
    little-endian record (8-byte tag, five int32, int32 offsets, float32 values) instead of a Boost archive."""
    vals = mat.vec.detach().cpu().numpy() if isinstance(mat, dev_dia_matrix_f) else mat.vec
    with open(filename, "wb") as f:
        f.write(_DIA_MAGIC)
        np.array([mat.w, mat.h, mat.num_dia, mat.stride, mat.row_fact], dtype="<i4").tofile(f)
        mat.offsets.astype("<i4").tofile(f)
        np.ascontiguousarray(vals, dtype="<f4").tofile(f)


def load_dia_mat(filename, device=None):
    """Read a record written by :func:`save_dia_mat`; returns a host matrix, or a device matrix if
    ``device`` is given (``load`` of src/cuv_python/export_dia_mat.cpp:96-110)."""
    with open(filename, "rb") as f:
        if f.read(8) != _DIA_MAGIC:
            raise CuvDiaError(_capi.ERR_INVALID, "not a DIA matrix record")
        w, h, nd, stride, rf = np.fromfile(f, dtype="<i4", count=5).tolist()
        offsets = np.fromfile(f, dtype="<i4", count=nd)
        vals = np.fromfile(f, dtype="<f4", count=nd * stride)
    if offsets.size != nd or vals.size != nd * stride:
        raise CuvDiaError(_capi.ERR_INVALID, "truncated DIA matrix record")
    host = host_dia_matrix_f(h, w, offsets, stride, rf)
    host.vec[:] = vals
    if device is None:
        return host
    return convert(dev_dia_matrix_f(h, w, offsets, stride, rf, device=device), host)


def convert(dst, src):
    """``cuv::convert`` for the DIA path (convert/convert.cu:42-112): host DIA <-> device DIA (offsets
    and values) and host DIA -> dense (returns a Fortran-ordered numpy matrix when ``dst`` is None)."""
    if isinstance(dst, dev_dia_matrix_f) and isinstance(src, host_dia_matrix_f):
        if (dst.shape, dst.num_dia, dst.stride, dst.row_fact) != (src.shape, src.num_dia, src.stride, src.row_fact) \
                or not np.array_equal(dst.offsets, src.offsets):
            dst.__init__(src.h, src.w, src.offsets, src.stride, src.row_fact, device=dst.vec.device)
        return dst.set_vec(src.vec)
    if isinstance(dst, host_dia_matrix_f) and isinstance(src, dev_dia_matrix_f):
        dst.__init__(src.h, src.w, src.offsets, src.stride, src.row_fact)
        dst.vec[:] = src.vec.detach().cpu().numpy()
        return dst
    if dst is None and isinstance(src, host_dia_matrix_f):
        dense = np.zeros((src.h, src.w), dtype=np.float32, order="F")
        rows = np.arange(src.h)
        for s, o in enumerate(src.offsets.tolist()):
            cols = rows // src.row_fact + o
            ok = (cols >= 0) & (cols < src.w)
            dense[rows[ok], cols[ok]] = src.vec[s * src.stride + rows[ok]]
        return dense
    raise CuvDiaError(_capi.ERR_UNSUPPORTED, "convert: unsupported pair of types")


def pull(mat):
    """Device DIA matrix -> dense host matrix (``pull`` of src/cuv_python/export_dia_mat.cpp:158-167)."""
    return convert(None, convert(host_dia_matrix_f(mat.h, mat.w, mat.offsets, mat.stride, mat.row_fact), mat))


class filter_factory:
    """``filter_factory`` (basics/filter_factory.hpp:6-84): the DIA matrix of a layer of ``fs`` x ``fs`` convolution
    filters between ``input_maps`` and ``output_maps`` images of ``px`` x ``py`` pixels - runs of ``fs`` consecutive
    diagonals one image line apart, one block of ``fs*fs`` diagonals per map distance - and the way back from such a
    matrix to one filter.  Host-side index arithmetic only."""

    def __init__(self, px, py, fs, input_maps, output_maps):
        self.px, self.py, self.fs = int(px), int(py), int(fs)
        self.input_maps, self.output_maps = int(input_maps), int(output_maps)

    def offsets(self):
        """Diagonal numbers in storage order (basics/filter_factory.hpp:58-71)."""
        px, py, fs = self.px, self.py, self.fs
        m, i, j = np.meshgrid(np.arange(self.output_maps + self.input_maps - 1), np.arange(fs), np.arange(fs), indexing="ij")
        shift = -(px + 1) * (fs // 2) - (self.input_maps - 1) * px * py
        return (i * px + j + m * px * py + shift).reshape(-1).astype(np.int32)

    def get_dia(self, device="cuda"):
        """A new device matrix (``device=None``: host matrix) of ``px*py*input_maps`` x ``px*py*output_maps``."""
        h, w = self.px * self.py * self.input_maps, self.px * self.py * self.output_maps
        if device is None:
            return host_dia_matrix_f(h, w, self.offsets(), max(h, w), 1)
        return dev_dia_matrix_f(h, w, self.offsets(), max(h, w), 1, device=device)

    def extract_filter(self, dia, filternumber):
        """The coefficients that column ``filternumber`` receives from each input map, as CUV lays them out: an
        ``(fs*fs, input_maps)`` row-major array filled flat, map after map (basics/filter_factory.hpp:22-41)."""
        host = dia if isinstance(dia, host_dia_matrix_f) else convert(
            host_dia_matrix_f(dia.h, dia.w, dia.offsets, dia.stride, dia.row_fact), dia)
        out = np.zeros(self.fs * self.fs * self.input_maps, dtype=np.float32)
        map_size = host.h // self.input_maps
        for m in range(self.input_maps):
            found = 0
            for i in range(map_size):
                row = i + m * map_size
                if not host.has(row, filternumber):
                    continue
                out[m * self.fs * self.fs + found] = host(row, filternumber)
                found += 1
                if found >= out.size:
                    break
        return out.reshape(self.fs * self.fs, self.input_maps)


class dev_block_descriptor_f:
    """``dev_block_descriptor<float>`` (matrix_ops/densedense_to_sparse.hpp:72-105).  CUV precomputes a
    list of 16x16 tiles here; this implementation needs no tile list, so the descriptor only refers
    to the matrix's plan.  It stays in the interface so calling code is unchanged."""

    def __init__(self, mat):
        self._mat = mat

    def __len__(self):
        # number of 16x16 tiles a stored diagonal crosses is what CUV reports; not needed here
        return 0


# ---- operations --------------------------------------------------------------------------------------

def plan_status(A):
    """The health word of the matrix's plan (blocking): 0, or the code left by a kernel that gave up a bounded
    wait on an asynchronous copy and returned with its output incomplete."""
    st = ctypes.c_int()
    _capi.check(_capi.lib().cuvdia_plan_status(A._plan, ctypes.byref(st)))
    return int(st.value)


def raise_if_gave_up(A):
    """Blocking check after operations on ``A``: waits for the device, and if a kernel of the plan gave up a bounded
    wait, clears the word and raises, as CUV throws from a failed blocking operation (tools/cuv_general.cu:51-61).
    The calls of this module are stream-ordered and do not look at the word themselves unless asked to
    (``check_status=True``), because looking means waiting for the device."""
    _torch().cuda.synchronize()
    st = plan_status(A)
    if st:
        _capi.check(_capi.lib().cuvdia_plan_status_clear(A._plan, _stream()))
        raise CuvDiaError(_capi.ERR_CUDA, "a kernel gave up a bounded wait on an asynchronous copy (status %d): "
                                          "the output is incomplete" % st)


def prod(C, A, B, transA="n", transB="n", factAB=1.0, factC=0.0, mode=MODE_EXACT, check_status=False):
    """C = factC*C + factAB*op(A)*B (matrix_ops/matrix_ops.hpp:118-119, matrix_ops/spmv.cu:221-247).
    ``check_status=True`` makes the call blocking, like CUV's, and raises if a kernel gave up a bounded wait."""
    ldc, ldb = _check_colmajor(C, "C"), _check_colmajor(B, "B")
    if C.shape[1] != B.shape[1]:
        raise CuvDiaError(_capi.ERR_INVALID, "dst.shape()[1] == B.shape()[1]")
    rows_b, rows_c = (A.h, A.w) if transA == "t" else (A.w, A.h)
    if transA in ("n", "t") and (B.shape[0] != rows_b or C.shape[0] != rows_c):
        raise CuvDiaError(_capi.ERR_INVALID, "operand heights match the matrix (spmv.cu:159-160,180-181)")
    _capi.check(_capi.lib().cuvdia_prod_f32(A._plan, _ptr(A.vec), _ptr(B), ldb, _ptr(C), ldc, int(C.shape[1]),
                                            transA.encode(), transB.encode(), factAB, factC, mode, _stream()))
    if check_status:
        raise_if_gave_up(A)
    return C


def prod_bias_sigmoid_sample(C, A, B, transA="n", factAB=1.0, factC=0.0, mode=MODE_EXACT, bias=None, u=None,
                             sample=None):
    """One call for what an RBM/MLP layer does after the product (examples/rbm/base.py:48-54,93-106):
    C <- sigmoid(factC*C + factAB*op(A)*B + bias[:, None]); sample <- (C > u) as 0/1 floats if ``u`` is given.
    Same results as :func:`prod` followed by :func:`bias_sigmoid_sample`."""
    ldc, ldb = _check_colmajor(C, "C"), _check_colmajor(B, "B")
    if C.shape[1] != B.shape[1]:
        raise CuvDiaError(_capi.ERR_INVALID, "dst.shape()[1] == B.shape()[1]")
    rows_b, rows_c = (A.h, A.w) if transA == "t" else (A.w, A.h)
    if transA in ("n", "t") and (B.shape[0] != rows_b or C.shape[0] != rows_c):
        raise CuvDiaError(_capi.ERR_INVALID, "operand heights match the matrix (spmv.cu:159-160,180-181)")
    ldu = lds = 0
    if u is not None:
        ldu = _check_colmajor(u, "u")
        if sample is None:
            sample = colmajor_empty(C.shape[0], C.shape[1], C.device)
        lds = _check_colmajor(sample, "sample")
    _capi.check(_capi.lib().cuvdia_prod_bias_sigmoid_sample_f32(
        A._plan, _ptr(A.vec), _ptr(B), ldb, _ptr(C), ldc, int(C.shape[1]), transA.encode(), factAB, factC, mode,
        _ptr(bias), _ptr(u), ldu, _ptr(sample), lds, _stream()))
    return sample


def spmv(dst, A, v, transA="n", factAv=1.0, factC=0.0, mode=MODE_EXACT, check_status=False):
    """dst = factC*dst + factAv*op(A)*v for one or several vectors packed column-major in 1-D tensors
    (matrix_ops/matrix_ops.hpp:277-278, spmv.cu:248-253)."""
    rows_b, rows_c = (A.h, A.w) if transA == "t" else (A.w, A.h)
    if v.numel() % rows_b or dst.numel() // rows_c != v.numel() // rows_b or dst.numel() % rows_c:
        raise CuvDiaError(_capi.ERR_INVALID, "vector sizes are multiples of the matrix dimensions")
    n = v.numel() // rows_b
    _capi.check(_capi.lib().cuvdia_prod_f32(A._plan, _ptr(A.vec), _ptr(v), rows_b, _ptr(dst), rows_c, n,
                                            transA.encode(), b"n", factAv, factC, mode, _stream()))
    if check_status:
        raise_if_gave_up(A)
    return dst


def densedense_to_dia(C, Cbd, A, B, factAB=1.0, factC=0.0, check_status=False):
    """C_dia = factC*C_dia + factAB*(A*B^T on the stored diagonals)
    (matrix_ops/densedense_to_sparse.hpp:123-130)."""
    lda, ldb = _check_colmajor(A, "A"), _check_colmajor(B, "B")
    if C.w != B.shape[0] or C.h != A.shape[0] or A.shape[1] != B.shape[1]:
        raise CuvDiaError(_capi.ERR_INVALID, "dst.w()==B.shape()[0] && dst.h()==A.shape()[0] && "
                                             "A.shape()[1]==B.shape()[1]")
    _capi.check(_capi.lib().cuvdia_dd2dia_f32(C._plan, _ptr(C.vec), _ptr(A), lda, _ptr(B), ldb, int(A.shape[1]),
                                              factAB, factC, _stream()))
    if check_status:
        raise_if_gave_up(C)
    return C


def avg_diagonals(dst, A):
    """dst[k] = mean over the cells of stored diagonal k that lie inside the matrix (matrix_ops/diagonals.hpp:12,
    host definition matrix_ops/diagonals.cu:23-48)."""
    if dst.numel() != A.num_dia or not dst.is_contiguous():
        raise CuvDiaError(_capi.ERR_INVALID, "dia.num_dia()==dst.size()")
    _capi.check(_capi.lib().cuvdia_avg_diagonals_f32(A._plan, _ptr(A.vec), _ptr(dst), _stream()))
    return dst


def _type_code(t):
    torch = _torch()
    codes = {torch.float32: _capi.T_F32, torch.int32: _capi.T_I32, torch.uint8: _capi.T_U8}
    if hasattr(torch, "uint32"):
        codes[torch.uint32] = _capi.T_U32
    if t.dtype not in codes:
        raise CuvDiaError(_capi.ERR_UNSUPPORTED, "element type %s (float32, int32, uint32, uint8)" % t.dtype)
    return codes[t.dtype]


def _reduce(dst, src, over_first_axis_kept, rf, factNew, factOld):
    if not (src.dim() == 2 and src.is_cuda and dst.is_cuda):
        raise CuvDiaError(_capi.ERR_INVALID, "src must be a 2-D CUDA tensor")
    if src.stride(0) == 1 and (src.shape[1] == 1 or src.stride(1) == src.shape[0]):      # column-major
        n_contig, n_strided, keep_contig = src.shape[0], src.shape[1], over_first_axis_kept
    elif src.stride(1) == 1 and (src.shape[0] == 1 or src.stride(0) == src.shape[1]):    # row-major
        n_contig, n_strided, keep_contig = src.shape[1], src.shape[0], not over_first_axis_kept
    else:
        raise CuvDiaError(_capi.ERR_INVALID, "src must be densely packed")
    if dst.numel() != (n_contig if keep_contig else n_strided) or not dst.is_contiguous():
        raise CuvDiaError(_capi.ERR_INVALID, "main_dim == v.size()")
    _capi.check(_capi.lib().cuvdia_reduce(_ptr(dst), _type_code(dst), _ptr(src), _type_code(src), n_contig, n_strided,
                                          1 if keep_contig else 0, rf, factNew, factOld, _stream()))
    return dst


def reduce_to_col(dst, src, rf=RF_ADD, factNew=1.0, factOld=0.0):
    """dst[i] = factOld*dst[i] + factNew*rf_j(src[i, j]); dst.size == src.shape[0]
    (matrix_ops/matrix_ops.hpp:211-212, matrix_ops_reduce.cu:348-362).  ``src`` / ``dst`` element types: the pairs
    CUV instantiates (float32, int32, uint32, uint8 sources with float32 results; float32 sources with int32, uint32,
    uint8 results; uint8 -> uint8 / uint32), with CUV's semantics for them (running value in the source type)."""
    return _reduce(dst, src, True, rf, factNew, factOld)


def reduce_to_row(dst, src, rf=RF_ADD, factNew=1.0, factOld=0.0):
    """dst[j] = factOld*dst[j] + factNew*rf_i(src[i, j]); dst.size == src.shape[1]
    (matrix_ops/matrix_ops.hpp:227-228, matrix_ops_reduce.cu:364-379)."""
    return _reduce(dst, src, False, rf, factNew, factOld)


def bias_sigmoid_sample(act, bias=None, u=None, sample=None):
    """act <- sigmoid(act + bias[:, None]); sample <- (act > u) as 0/1 floats when ``u`` is given
    (matrix_plus_col + SF_SIGM + rnd_binarize's compare, examples/rbm/base.py:52-54,93-106)."""
    ld = _check_colmajor(act, "act")
    ldu = lds = 0
    if u is not None:
        ldu = _check_colmajor(u, "u")
        if sample is None:
            sample = colmajor_empty(act.shape[0], act.shape[1], act.device)
        lds = _check_colmajor(sample, "sample")
    _capi.check(_capi.lib().cuvdia_bias_sigmoid_sample_f32(_ptr(act), ld, _ptr(bias), _ptr(u), ldu, _ptr(sample),
                                                           lds, int(act.shape[0]), int(act.shape[1]), _stream()))
    return sample


def bias_sigmoid_sample_sum(act, bias, u, sample, sum_dst, sum_of_sample=False, factNew=1.0, factOld=0.0,
                            store_act=True):
    """:func:`bias_sigmoid_sample` that also accumulates ``sum_dst[i] = factOld*sum_dst[i] + factNew*sum_j x[i, j]``
    in the same pass, x being the activation after the logistic or (``sum_of_sample``) the 0/1 sample: the
    ``reduce_to_col`` of the trainer's bias gradients (examples/rbm/base.py:76-83) without a second read of the
    matrix.  ``store_act=False`` leaves ``act`` unwritten."""
    ld = _check_colmajor(act, "act")
    ldu = lds = 0
    if u is not None:
        ldu = _check_colmajor(u, "u")
        lds = _check_colmajor(sample, "sample")
    if sum_dst.numel() != act.shape[0] or not sum_dst.is_contiguous():
        raise CuvDiaError(_capi.ERR_INVALID, "main_dim == v.size()")
    _capi.check(_capi.lib().cuvdia_bias_sigmoid_sample_sum_f32(
        _ptr(act), ld, _ptr(bias), _ptr(u), ldu, _ptr(sample), lds, int(act.shape[0]), int(act.shape[1]),
        _ptr(sum_dst), 1 if sum_of_sample else 0, factNew, factOld, 1 if store_act else 0, _stream()))
    return sample


def fill_rnd_uniform(dst, seed, step=0, col0=0, which=0):
    """dst[i, j] = the uniform number in [0, 1) of element (i, col0 + j) of draw ``which`` in step ``step``
    (``fill_rnd_uniform``, random/random.cu:167-177, as a pure function of its arguments: see
    ``cuvdia_uniform_f32`` in include/cuvdia.h)."""
    import ctypes
    ld = _check_colmajor(dst, "dst")
    d = _capi.Draw(int(seed), int(step), int(col0))
    _capi.check(_capi.lib().cuvdia_uniform_f32(_ptr(dst), ld, int(dst.shape[0]), int(dst.shape[1]), ctypes.byref(d),
                                               int(which), _stream()))
    return dst


def rnd_binarize(act, seed, step=0, col0=0, which=0):
    """act[i, j] = 1 if act[i, j] > u else 0, in place, u the uniform number :func:`fill_rnd_uniform` gives for the same
    arguments (``rnd_binarize``, random/random.cu:86-91,139-156)."""
    import ctypes
    ld = _check_colmajor(act, "act")
    d = _capi.Draw(int(seed), int(step), int(col0))
    _capi.check(_capi.lib().cuvdia_rnd_binarize_f32(_ptr(act), ld, int(act.shape[0]), int(act.shape[1]), ctypes.byref(d),
                                                    int(which), _stream()))
    return act


def bias_sigmoid_draw_sum(act, bias, sample, sum_dst, seed, step=0, col0=0, which=0, sum_of_sample=False, factNew=1.0,
                          factOld=0.0, store_act=True):
    """:func:`bias_sigmoid_sample_sum` with the uniform numbers drawn inside the pass (``rnd_binarize`` fused in,
    random/random.cu:139-156): the bits of that call on ``u = fill_rnd_uniform(..)`` with the same arguments."""
    import ctypes
    ld = _check_colmajor(act, "act")
    lds = _check_colmajor(sample, "sample")
    if sum_dst.numel() != act.shape[0] or not sum_dst.is_contiguous():
        raise CuvDiaError(_capi.ERR_INVALID, "main_dim == v.size()")
    d = _capi.Draw(int(seed), int(step), int(col0))
    _capi.check(_capi.lib().cuvdia_bias_sigmoid_draw_sum_f32(
        _ptr(act), ld, _ptr(bias), _ptr(sample), lds, int(act.shape[0]), int(act.shape[1]), _ptr(sum_dst),
        1 if sum_of_sample else 0, factNew, factOld, 1 if store_act else 0, ctypes.byref(d), int(which), _stream()))
    return sample


def axpby(dst, x, y, a, b):
    """dst = a*x + b*y (apply_binary_functor BF_AXPBY, tensor_ops/tensor_ops.hpp:530-655)."""
    if not (dst.numel() == x.numel() == y.numel()):
        raise CuvDiaError(_capi.ERR_INVALID, "sizes match")
    _capi.check(_capi.lib().cuvdia_axpby_f32(_ptr(dst), _ptr(x), _ptr(y), a, b, dst.numel(), _stream()))
    return dst


def _flat_values(x):
    """The flat float storage of a DIA matrix (its whole value array) or of a tensor."""
    return x.vec if isinstance(x, dev_dia_matrix_f) else x


def learn_step_weight_decay(W, dW, learnrate, decay=0.0, sparsedecay=0.0):
    """W = -learnrate*dW + (1 - learnrate*decay)*W in place (tensor_ops/rprop.hpp:117-128).

    ``W`` and ``dW`` are device tensors or DIA matrices of equal storage size; the update of the sparse
    RBM passes the weight matrix and its gradient (examples/rbm/base.py:72-75).  ``sparsedecay`` is
    accepted and ignored, as in the reference (its L1 term is commented out)."""
    w, g = _flat_values(W), _flat_values(dW)
    if w.numel() != g.numel():
        raise CuvDiaError(_capi.ERR_INVALID, "W.size() == dW.size()")
    _capi.check(_capi.lib().cuvdia_learn_step_weight_decay_f32(_ptr(w), _ptr(g), w.numel(), float(learnrate),
                                                               float(decay), _stream()))
    return W


def learn_step_weight_decay_momentum(W, momentum, dW, learnrate, momentum_weight=0.9, decay=0.0, sparsedecay=0.0):
    """m = momentum_weight*m - learnrate*(dW + decay*W); W += m (tensor_ops/rprop.hpp:130-143, rprop.cu:158-170)."""
    w, m, g = _flat_values(W), _flat_values(momentum), _flat_values(dW)
    if not (w.numel() == g.numel() == m.numel()):
        raise CuvDiaError(_capi.ERR_INVALID, "W.size() == dW.size() == momentum.size()")
    _capi.check(_capi.lib().cuvdia_learn_step_weight_decay_momentum_f32(
        _ptr(w), _ptr(m), _ptr(g), w.numel(), float(learnrate), float(momentum_weight), float(decay), _stream()))
    return W
