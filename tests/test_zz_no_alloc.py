"""GPU test of the allocation-free K1 entry point.

``gtk_k1_select_noalloc`` serves embedders that may not call the CUDA
allocator (a fixed memory budget, or a loop that cannot take the device-wide
synchronisation cudaMalloc implies): its scratch is a static device array
inside the library.  The test calls it through its exported C symbol with
ctypes, twice in a row on changing inputs, and checks selection and residual
against the regular entry point (``gtk_k1_select`` behind ``TopkSelector``)
with the tolerance of the other kernel tests.  It also checks that a size
beyond the stated maximum is refused.  The file is named so that pytest
collects it last.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

GTK_ERR_TOO_LARGE = -4


def _load():
    from gtopkssgd_b200.ops import build
    lib = C.CDLL(build.build())  # the exported C symbols, no Python wrapper in between
    lib.gtk_k1_select_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_uint, C.c_void_p, C.c_void_p,
                                          C.c_int, C.c_void_p]
    lib.gtk_k1_select_noalloc.restype = C.c_int
    lib.gtk_k1_noalloc_max_k.restype = C.c_uint
    lib.gtk_k1_noalloc_scratch_bytes.restype = C.c_ulonglong
    lib.gtk_k1_noalloc_status.argtypes = [C.POINTER(C.c_uint), C.c_int, C.c_void_p]
    lib.gtk_k1_noalloc_status.restype = C.c_int
    return lib


def _check_against_oracle(g, r_before, r_after, out, n, k):
    """Selection and residual against the plain PyTorch statement of the operation."""
    from gtopkssgd_b200.ops import oracle
    from gtopkssgd_b200.ops.select import pairs_to_tensors
    r_ref = r_before.clone()
    idx_ref, val_ref = oracle.compress(g, r_ref, k)
    assert n == idx_ref.numel()
    idx, val = pairs_to_tensors(out, n)
    ref = dict(zip(idx_ref.cpu().tolist(), val_ref.cpu().tolist()))
    got = dict(zip(idx.cpu().tolist(), val.cpu().tolist()))
    assert len(got) == n and set(got) == set(ref)
    for j in ref:
        assert got[j] == pytest.approx(ref[j], rel=1e-6, abs=1e-7)
    assert torch.allclose(r_after, r_ref, rtol=1e-6, atol=1e-7)


def test_noalloc_select_matches_regular_entry_point_twice():
    from gtopkssgd_b200.ops.select import TopkSelector, pairs_to_tensors
    lib = _load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    assert lib.gtk_k1_noalloc_max_k() == 16384
    assert 0 < lib.gtk_k1_noalloc_scratch_bytes() < 2 << 20
    torch.manual_seed(123)
    d, k = 1_000_003, 1000
    ref_sel = TopkSelector(d, k, dev)
    r_ref = torch.zeros(d, device=dev)
    r_new = torch.zeros(d, device=dev)
    out = torch.zeros((k, 2), dtype=torch.int32, device=dev)
    n_out = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    for call in range(2):  # two calls in a row: the second one reuses the shared scratch and the residual
        g = torch.randn(d, device=dev) * (1.0 + call)
        ref_sel.select(g, r_ref, k)
        before = torch.cuda.memory_allocated(dev)
        code = lib.gtk_k1_select_noalloc(g.data_ptr(), r_new.data_ptr(), d, k, out.data_ptr(), n_out.data_ptr(),
                                         1 if call == 0 else 0, stream)
        assert code == 0
        assert torch.cuda.memory_allocated(dev) == before
        torch.cuda.synchronize()
        assert int(n_out.item()) == k
        idx_ref, val_ref = ref_sel.pairs()
        idx, val = pairs_to_tensors(out, k)
        ref = dict(zip(idx_ref.cpu().tolist(), val_ref.cpu().tolist()))
        got = dict(zip(idx.cpu().tolist(), val.cpu().tolist()))
        assert len(got) == k and set(got) == set(ref)
        for j in ref:
            assert got[j] == pytest.approx(ref[j], rel=1e-6, abs=1e-7)
        assert torch.allclose(r_new, r_ref, rtol=1e-6, atol=1e-7)
    st = (C.c_uint * 2)(7, 7)
    assert lib.gtk_k1_noalloc_status(st, 0, stream) == 0 and (st[0], st[1]) == (0, 0)


def test_noalloc_against_the_oracle_with_changing_sizes():
    """Consecutive calls share the scratch and its predicted threshold while (d, k) change between
    them: the largest k the scratch serves, d < k (fewer pairs than asked for come back), a small
    odd size, and back.  Every result is compared with the fp32 PyTorch oracle."""
    lib = _load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    kmax = int(lib.gtk_k1_noalloc_max_k())
    torch.manual_seed(321)
    cases = [(2_000_003, kmax), (2_000_003, kmax), (500, 1000), (4099, 17), (2_000_003, 64), (300_001, 3000),
             (300_001, 3000)]
    resid = {}
    for d, k in cases:
        g = torch.randn(d, device=dev)
        r = resid.setdefault(d, torch.zeros(d, device=dev))
        r_before = r.clone()
        out = torch.zeros((k, 2), dtype=torch.int32, device=dev)
        n_out = torch.zeros(1, dtype=torch.int32, device=dev)
        before = torch.cuda.memory_allocated(dev)
        code = lib.gtk_k1_select_noalloc(g.data_ptr(), r.data_ptr(), d, k, out.data_ptr(), n_out.data_ptr(), 0, stream)
        assert code == 0 and torch.cuda.memory_allocated(dev) == before
        torch.cuda.synchronize()
        n = int(n_out.item())
        assert n == min(k, d)
        _check_against_oracle(g, r_before, r, out, n, k)
    st = (C.c_uint * 2)(7, 7)
    assert lib.gtk_k1_noalloc_status(st, 1, stream) == 0 and (st[0], st[1]) == (0, 0)  # and reset: still works after
    d, k = 100_000, 100
    g, r = torch.randn(d, device=dev), torch.zeros(d, device=dev)
    out = torch.zeros((k, 2), dtype=torch.int32, device=dev)
    n_out = torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.gtk_k1_select_noalloc(g.data_ptr(), r.data_ptr(), d, k, out.data_ptr(), n_out.data_ptr(), 0, stream) == 0
    torch.cuda.synchronize()
    _check_against_oracle(g, torch.zeros(d, device=dev), r, out, int(n_out.item()), k)


def test_noalloc_rejects_misaligned_outputs():
    lib = _load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    d, k = 10000, 10
    g, r = torch.randn(d, device=dev), torch.zeros(d, device=dev)
    out = torch.zeros((k + 1, 2), dtype=torch.int32, device=dev)
    n_out = torch.zeros(2, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert lib.gtk_k1_select_noalloc(g.data_ptr(), r.data_ptr(), d, k, out.data_ptr() + 4, n_out.data_ptr(), 0,
                                     stream) == -1   # pairs need 8-byte alignment
    assert lib.gtk_k1_select_noalloc(g.data_ptr(), r.data_ptr(), d, k, out.data_ptr(), n_out.data_ptr() + 2, 0,
                                     stream) == -1   # the count needs 4-byte alignment
    torch.cuda.synchronize()
    assert float(r.abs().sum()) == 0.0  # nothing was enqueued


def test_noalloc_rejects_sizes_beyond_the_maximum():
    lib = _load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    d = 100000
    k = lib.gtk_k1_noalloc_max_k() + 1
    g = torch.randn(d, device=dev)
    r = torch.zeros(d, device=dev)
    out = torch.zeros((k, 2), dtype=torch.int32, device=dev)
    code = lib.gtk_k1_select_noalloc(g.data_ptr(), r.data_ptr(), d, k, out.data_ptr(), None, 0,
                                     torch.cuda.current_stream(dev).cuda_stream)
    assert code == GTK_ERR_TOO_LARGE
    torch.cuda.synchronize()
    assert float(r.abs().sum()) == 0.0  # nothing was enqueued
