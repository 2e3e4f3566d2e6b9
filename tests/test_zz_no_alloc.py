"""The allocation-free reduction entry point, cuvdia_reduce_noalloc_f32.

Who needs it: callers that may not allocate device memory while they run - code living inside a
fixed memory budget that a host application handed out, services that ban allocator calls after
start-up because an allocation can stall the whole device, and callers that could never free what the
library allocated for them.  The ordinary cuvdia_reduce_f32 creates a per-stream workspace with
cudaMalloc the first time a split reduction runs; this variant keeps its partial results in a
4 MiB array inside the library image instead and must give the same answers.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already
executed every other test.  It needs nothing from the other tests and also passes when run alone in
a fresh process (the first call on the device performs the one-time address look-up)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RF_ADD, RF_ARGMAX = 0, 4


def _call(L, name, dst, src, n_contig, n_strided, over_strided, rf, fnew, fold):
    import torch
    fn = getattr(L, name)
    return fn(ctypes.c_void_p(dst.data_ptr()), ctypes.c_void_p(src.data_ptr()), n_contig, n_strided, over_strided,
              rf, fnew, fold, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("n_contig,n_strided,over_strided", [
    (4096, 1024, 1),      # sum over the strided axis: blocks split the lines, partials in the static scratch
    (300000, 24, 0),      # sum along a few long lines: several blocks per line
])
def test_noalloc_matches_allocating_entry_point_twice_in_a_row(n_contig, n_strided, over_strided):
    import torch
    from cuv_b200 import _capi
    L = _capi.lib()
    torch.cuda.set_device(0)
    n_out = n_contig if over_strided else n_strided
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234 + n_contig)
    # two calls in a row on different data and functors: the shared scratch keeps the first call's
    # partial results, which must not leak into the second
    for call, (rf, fnew, fold) in enumerate([(RF_ADD, 0.5, 0.25), (RF_ARGMAX, 1.0, 0.0)]):
        src = torch.rand(n_strided * n_contig, device="cuda", generator=gen) * 2 - 1
        old = torch.rand(n_out, device="cuda", generator=gen)
        want, got = old.clone(), old.clone()
        assert _call(L, "cuvdia_reduce_f32", want, src, n_contig, n_strided, over_strided, rf, fnew, fold) == 0
        rc = _call(L, "cuvdia_reduce_noalloc_f32", got, src, n_contig, n_strided, over_strided, rf, fnew, fold)
        assert rc == 0, L.cuvdia_last_error_message()
        torch.cuda.synchronize()
        if rf == RF_ARGMAX:
            assert torch.equal(got, want), "call %d" % call
        else:
            # same tolerance as the other reduction tests: 1e-4 * sqrt(n_red / 128) relative
            n_red = n_strided if over_strided else n_contig
            tol = 1e-4 * np.sqrt(max(n_red, 128) / 128.0)
            np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), rtol=tol, atol=tol * 1e-2)
            ref = fold * old.double() + fnew * src.double().view(n_strided, n_contig).sum(0 if over_strided else 1)
            np.testing.assert_allclose(got.cpu().numpy(), ref.cpu().numpy(), rtol=tol, atol=tol)


def test_noalloc_refuses_shapes_beyond_its_scratch():
    import torch
    from cuv_b200 import _capi
    L = _capi.lib()
    torch.cuda.set_device(0)
    # 300000 outputs reduced over 64 lines: on a 148-SM B200 the lines are split in two, and two partial
    # results (value + index, 8 bytes) for each of 300000 outputs exceed the 4 MiB array
    n_contig, n_strided = 300000, 64
    src = torch.zeros(n_contig * n_strided, device="cuda")
    dst = torch.zeros(n_contig, device="cuda")
    rc = _call(L, "cuvdia_reduce_noalloc_f32", dst, src, n_contig, n_strided, 1, RF_ADD, 1.0, 0.0)
    assert rc == _capi.ERR_UNSUPPORTED
    msg = L.cuvdia_last_error_message().decode()
    assert "static scratch holds 4194304 bytes" in msg and "cuvdia_reduce_f32" in msg
    assert _call(L, "cuvdia_reduce_f32", dst, src, n_contig, n_strided, 1, RF_ADD, 1.0, 0.0) == 0
    torch.cuda.synchronize()
