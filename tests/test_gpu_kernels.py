"""GPU numerics tests: every CUDA kernel against the PyTorch fp32 oracle.

The multi-rank exchange kernels are exercised with all P ranks emulated on one
GPU in a single cooperative launch (peer pointers are local pointers), which
runs the full protocol: pushes, flags, epochs, merges, re-selects, broadcast
and residual put-back.
"""
import math

import pytest
import torch

from gtopkssgd_b200.ops import oracle

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")


def _selector(d, k, **kw):
    from gtopkssgd_b200.ops.select import TopkSelector
    return TopkSelector(d, k, DEV, **kw)


def _check_select(sel, g, r_before, k, scale=1.0):
    """Compare the selector's output with the oracle on the same inputs."""
    r_ref = r_before.clone().cpu()
    idx_ref, val_ref = oracle.compress(g.cpu(), r_ref, k, scale)
    idx, val = sel.pairs()
    assert idx.numel() == min(k, g.numel())
    got = dict(zip(idx.cpu().tolist(), val.cpu().tolist()))
    ref = dict(zip(idx_ref.tolist(), val_ref.tolist()))
    assert len(got) == idx.numel(), "duplicate indices in the selection"
    assert set(got) == set(ref)
    for j in ref:
        assert got[j] == pytest.approx(ref[j], rel=1e-6, abs=1e-7)
    return r_ref


@pytest.mark.parametrize("d,k", [(1, 1), (7, 3), (1000, 1), (4099, 17), (100003, 100), (1 << 20, 1048), (3_000_001, 3000)])
def test_k1_select_matches_oracle(d, k):
    torch.manual_seed(d)
    sel = _selector(d, k)
    r = torch.zeros(d, device=DEV)
    for it in range(4):  # call 0: exact path; later calls: predicted threshold
        g = torch.randn(d, device=DEV) * (1.0 + 0.05 * it)
        r_before = r.clone()
        sel.select(g, r, k)
        r_ref = _check_select(sel, g, r_before, k)
        assert torch.allclose(r.cpu(), r_ref, rtol=1e-6, atol=1e-7)
        assert sel.status() == (0, 0)
    assert sel.stats()["n_calls"] == 4


def test_k1_large_vector_dynamic_stream_pass():
    """From 48 M elements on the stream pass hands its work out through a ticket
    counter; compared here against the oracle computed on the device."""
    d, k = 50_000_003, 50_000
    torch.manual_seed(7)
    sel = _selector(d, k)
    r = torch.zeros(d, device=DEV)
    for it in range(3):  # exact path, then predicted thresholds
        g = torch.randn(d, device=DEV)
        r_ref = r.clone()
        idx_ref, val_ref = oracle.compress(g, r_ref, k)
        sel.select(g, r, k)
        idx, val = sel.pairs()
        assert sel.status() == (0, 0) and idx.numel() == k
        order, order_ref = idx.argsort(), idx_ref.argsort()
        assert torch.equal(idx[order], idx_ref[order_ref])
        assert torch.allclose(val[order], val_ref[order_ref], rtol=1e-6, atol=1e-7)
        assert torch.allclose(r, r_ref, rtol=1e-6, atol=1e-7)
        del g, r_ref
    st = sel.stats()  # the residual grows over these calls, so a second exact pass is legitimate
    assert st["n_calls"] == 3 and st["n_fallbacks"] < 3


def test_k1_threshold_prediction_carries_steady_state():
    """With a stationary input distribution only the first call (no threshold
    yet) may take the exact dense path."""
    torch.manual_seed(11)
    d, k = 1 << 20, 1048
    sel = _selector(d, k)
    r = torch.zeros(d, device=DEV)
    for it in range(10):
        g = torch.randn(d, device=DEV) * (1.0 + 0.03 * math.sin(it))
        r.zero_()
        sel.select(g, r, k)
    st = sel.stats()
    assert st["n_calls"] == 10 and st["n_fallbacks"] == 1, st
    assert k <= st["n_cand"] <= sel.cap


def test_k1_unaligned_views_and_scale():
    torch.manual_seed(5)
    d, k = 50001, 50
    big_g = torch.randn(d + 8, device=DEV)
    big_r = torch.zeros(d + 8, device=DEV)
    scale = torch.tensor([0.5], device=DEV)
    for off in (1, 2, 3):
        g, r = big_g[off:off + d], big_r[off:off + d]
        big_r.zero_()
        sel = _selector(d, k)
        for _ in range(2):
            r_before = r.clone()
            sel.select(g, r, k, g_scale=scale)
            r_ref = _check_select(sel, g, r_before, k, 0.5)
            assert torch.allclose(r.cpu(), r_ref, rtol=1e-6, atol=1e-7)
        # nothing outside the view was touched
        assert float(big_r[:off].abs().sum()) == 0.0 and float(big_r[off + d:].abs().sum()) == 0.0


def test_k1_non_finite_entries_are_selected_on_both_paths():
    """NaN and +-Inf count as the largest magnitudes (NaN above Inf), as
    torch.topk(|acc|) of the reference ranks them (compression.py:43): they are
    selected and leave the residual on the exact path (first call) and on the
    predicted-threshold path (later calls) alike."""
    torch.manual_seed(9)
    d, k = 300_000, 300
    sel = _selector(d, k)
    r = torch.zeros(d, device=DEV)
    planted = {0: [(17, float("nan")), (d - 1, float("inf"))],              # call 0: exact path
               2: [(4096, float("-inf")), (123_457, float("nan")), (3, float("nan"))]}  # call 2: predicted threshold
    for it in range(4):
        g = torch.randn(d, device=DEV)
        for j, v in planted.get(it, []):
            g[j] = v
        r_before = r.clone()
        sel.select(g, r, k)
        idx, val = sel.pairs()
        assert sel.status() == (0, 0) and idx.numel() == k
        got = dict(zip(idx.cpu().tolist(), val.cpu().tolist()))
        assert len(got) == k
        bad = planted.get(it, [])
        for j, v in bad:
            assert j in got, "call %d: non-finite entry %d not selected" % (it, j)
            assert (math.isnan(v) and math.isnan(got[j])) or got[j] == v
            assert float(r[j]) == 0.0
        # the finite rest: the k - len(bad) largest finite magnitudes, residual = acc off the selection
        acc = (g + r_before).cpu()
        finite = acc.clone()
        for j, _ in bad:
            finite[j] = 0.0
        top = set(torch.topk(finite.abs(), k - len(bad)).indices.tolist())
        assert set(got) - {j for j, _ in bad} == top
        keep = torch.ones(d, dtype=torch.bool)
        keep[list(got)] = False
        assert torch.equal(r.cpu()[keep], acc[keep])
        assert torch.isfinite(r).all()
        if it == 2:
            assert sel.stats()["fallback"] == 0, "call 2 was meant to run on the predicted threshold"


def test_k1_scale_jump_and_ties():
    """A 5x scale jump overflows or starves the candidate list: the exact path
    must take over; repeated values must still give exactly k entries."""
    torch.manual_seed(6)
    d, k = 200000, 200
    sel = _selector(d, k)
    r = torch.zeros(d, device=DEV)
    for scale in (1.0, 1.0, 5.0, 0.2, 1.0):
        g = torch.randn(d, device=DEV) * scale
        r.zero_()
        sel.select(g, r, k)
        _check_select(sel, g, torch.zeros(d, device=DEV), k)
    g = torch.ones(d, device=DEV)  # all tied
    r.zero_()
    sel.select(g, r, k)
    idx, val = sel.pairs()
    assert idx.numel() == k and idx.unique().numel() == k and torch.all(val == 1.0)
    assert float(r.sum()) == d - k
    g = torch.zeros(d, device=DEV)  # all zero
    r.zero_()
    sel.select(g, r, k)
    idx, val = sel.pairs()
    assert idx.numel() == k and torch.all(val == 0)


def test_k1_density_one():
    d = 1000
    sel = _selector(d, d)
    g = torch.randn(d, device=DEV)
    r = torch.zeros(d, device=DEV)
    sel.select(g, r, d)
    idx, val = sel.pairs()
    assert idx.numel() == d and float(r.abs().sum()) == 0.0
    assert torch.equal(val[torch.argsort(idx)], g)


def _pairs_tensor(idx, val, cap):
    from gtopkssgd_b200.ops.select import tensors_to_pairs
    out = torch.zeros((cap, 2), dtype=torch.int32, device=DEV)
    tensors_to_pairs(idx.to(DEV), val.to(DEV), out)
    return out


@pytest.mark.parametrize("momentum,nesterov,wd,damp", [(0.9, False, 1e-4, 0.0), (0.9, True, 5e-4, 0.0),
                                                      (0.0, False, 0.0, 0.0), (0.5, False, 0.0, 0.1)])
def test_k3_sparse_plus_dense_equals_reference_sgd(momentum, nesterov, wd, damp):
    from gtopkssgd_b200.ops.sgd import SgdHyper, sgd_dense, sgd_sparse
    torch.manual_seed(7)
    d, k, P = 100003, 101, 4
    p = torch.randn(d, device=DEV)
    buf = torch.zeros(d, device=DEV)
    p_ref, buf_ref = p.cpu().clone(), buf.cpu().clone()
    h = SgdHyper(lr=0.1, momentum=momentum, dampening=damp, weight_decay=wd, nesterov=nesterov)
    for step in range(3):
        idx = torch.randperm(d)[:k]
        val = torch.randn(k)
        pairs = _pairs_tensor(idx, val, k)
        counts = torch.tensor([k], dtype=torch.int32, device=DEV)
        sgd_dense(p, buf, h, first_step=(step == 0))
        sgd_sparse(p, buf, pairs, counts, 1, k, h, first_step=(step == 0), scale=1.0 / P)
        dense = oracle.scatter_average((idx, val), d, P)
        oracle.sgd_step(p_ref, buf_ref, dense, 0.1, momentum, damp, wd, nesterov, first_step=(step == 0))
    assert torch.allclose(p.cpu(), p_ref, rtol=1e-5, atol=1e-6)
    if momentum:
        assert torch.allclose(buf.cpu(), buf_ref, rtol=1e-5, atol=1e-6)


def test_k3_dense_mode_and_scatter():
    from gtopkssgd_b200.ops.sgd import SgdHyper, scatter_dense, sgd_dense, sgd_sparse
    torch.manual_seed(8)
    d, P = 70001, 8
    p = torch.randn(d + 1, device=DEV)[1:]  # unaligned view
    buf = torch.zeros(d + 1, device=DEV)[1:]
    g = torch.randn(d + 1, device=DEV)[1:]
    coef = torch.tensor([0.25], device=DEV)
    p_ref, buf_ref = p.cpu().clone(), buf.cpu().clone()
    h = SgdHyper(lr=0.05, momentum=0.9, weight_decay=1e-4)
    sgd_dense(p, buf, h, True, g=g, scale=1.0 / P, coef=coef)
    oracle.sgd_step(p_ref, buf_ref, g.cpu() * (0.25 / P), 0.05, 0.9, 0.0, 1e-4, False, True)
    assert torch.allclose(p.cpu(), p_ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(buf.cpu(), buf_ref, rtol=1e-5, atol=1e-6)
    # atomic mode with repeated indices over two segments
    k = 64
    idx = torch.randint(0, 100, (2 * k,))
    val = torch.randn(2 * k)
    pairs = _pairs_tensor(idx, val, 2 * k)
    counts = torch.tensor([k, k - 3], dtype=torch.int32, device=DEV)
    dense = torch.empty(d, device=DEV)
    scatter_dense(dense, pairs, counts, 2, k, 0.5, use_atomics=True)
    ref = torch.zeros(d)
    ref.index_add_(0, idx[:k], val[:k] * 0.5)
    ref.index_add_(0, idx[k:2 * k - 3], val[k:2 * k - 3] * 0.5)
    assert torch.allclose(dense.cpu(), ref, atol=1e-6)
    q = torch.zeros(d, device=DEV)
    sgd_sparse(q, None, pairs, counts, 2, k, SgdHyper(lr=1.0), False, 0.5, use_atomics=True)
    assert torch.allclose(q.cpu(), -ref, atol=1e-6)


def test_k4_clip_norm():
    from gtopkssgd_b200.ops.clip import ClipNorm
    torch.manual_seed(9)
    d = 1_000_003
    x = torch.randn(d + 1, device=DEV)[1:]
    c = ClipNorm(DEV)
    c.add_dense(x)
    coef = c.finalize(0.25)
    norm = float(x.double().norm())
    assert c.last_norm() == pytest.approx(norm, rel=1e-5)
    assert float(coef) == pytest.approx(0.25 / (norm + 1e-6), rel=1e-5)
    # sparse pairs, scaled by 1/P, no clipping needed -> coef 1; accumulator was cleared
    k = 1000
    val = torch.randn(k) * 1e-3
    pairs = _pairs_tensor(torch.arange(k), val, k)
    counts = torch.tensor([k], dtype=torch.int32, device=DEV)
    c.add_pairs(pairs, counts, 1, k)
    coef = c.finalize(400.0, scale=0.125)
    assert float(coef) == 1.0
    assert c.last_norm() == pytest.approx(float(val.double().norm()) / 8, rel=1e-5)


def _emulated_world(P, d, k, mode="gtopk"):
    from gtopkssgd_b200.ops import exchange as ex
    with_ag = mode != "gtopk"
    regions = ex.SymmetricRegion.create_emulated(P, ex.region_bytes(k, with_ag), DEV)
    ranks = []
    for r in range(P):
        sel = _selector(d, k)
        resid = torch.zeros(d, device=DEV)
        ranks.append(ex.ExchangeRank(r, P, d, k, sel, resid, regions[r], with_allgather=with_ag,
                                     reselect=(mode == "topk2")))
    desc = torch.cat([r.desc for r in ranks])
    return ranks, desc


def _read_gout(rank, parity):
    from gtopkssgd_b200.ops.select import pairs_to_tensors
    n = int(rank.n_global.item())
    off = rank.layout[2] + parity * rank.kcap * 8
    raw = rank.region.tensor()[off:off + n * 8].view(torch.int32).view(n, 2)
    return pairs_to_tensors(raw, n)


@pytest.mark.parametrize("P", [2, 4, 8])
@pytest.mark.parametrize("d,k,nctas", [(4096, 8, 1), (50000, 50, 1), (300000, 3000, 4), (2_000_000, 20000, 8),
                                       (2_000_000, 20000, 12)])  # 1 CTA; clusters of 4 and 8; software barrier
def test_k2_gtopk_exchange_emulated(P, d, k, nctas):
    from gtopkssgd_b200.ops import exchange as ex
    torch.manual_seed(100 * P + k)
    ranks, desc = _emulated_world(P, d, k)
    res_ref = [torch.zeros(d) for _ in range(P)]
    for epoch in (1, 2, 3):  # both parities, flag reuse
        grads = [torch.randn(d, device=DEV) for _ in range(P)]
        for r, g in zip(ranks, grads):
            r.selector.select(g, r.resid, k)
        ex.launch_gtopk(ranks, desc, 0, P, k, nctas=nctas, limit_ms=2000)
        torch.cuda.synchronize()
        for r in ranks:
            assert r.status() == (0, 0)
        glob, _ = oracle.simulate_gtopk_step([g.cpu() for g in grads], res_ref, k)
        ref = dict(zip(glob[0].tolist(), glob[1].tolist()))
        for r in ranks:
            gi, gv = _read_gout(r, r.last_parity())
            got = dict(zip(gi.cpu().tolist(), gv.cpu().tolist()))
            assert len(got) == gi.numel()
            assert set(got) == set(ref), "rank %d" % r.rank
            for j in ref:
                assert got[j] == pytest.approx(ref[j], rel=1e-5, abs=1e-6)
            assert torch.allclose(r.resid.cpu(), res_ref[r.rank], rtol=1e-5, atol=1e-6)
            assert r.region.guards_intact(), "a store landed outside the slots of rank %d" % r.rank


@pytest.mark.parametrize("nctas", [1, 4, 12])
def test_k2_reselect_when_the_threshold_prediction_misses(nctas):
    """The re-select of a tree round reads its first two radix digits from histograms built on the
    fly around a predicted threshold digit (this rank's own k-th magnitude, then the previous round's
    threshold).  Ranks whose gradients differ in scale by orders of magnitude put the union's
    threshold far outside that window, so the counting sweep has to take over; tiny and huge ranks
    alternate so that both receivers and senders of every round are affected."""
    from gtopkssgd_b200.ops import exchange as ex
    P, d, k = 4, 300_000, 3000
    torch.manual_seed(4242 + nctas)
    ranks, desc = _emulated_world(P, d, k)
    res_ref = [torch.zeros(d) for _ in range(P)]
    scales = [1.0, 3.0e3, 1.0e-3, 5.0e1]
    for epoch in range(3):
        grads = [torch.randn(d, device=DEV) * scales[(r + epoch) % P] for r in range(P)]
        for r, g in zip(ranks, grads):
            r.selector.select(g, r.resid, k)
        ex.launch_gtopk(ranks, desc, 0, P, k, nctas=nctas, limit_ms=2000)
        torch.cuda.synchronize()
        assert all(r.status() == (0, 0) for r in ranks)
        glob, _ = oracle.simulate_gtopk_step([g.cpu() for g in grads], res_ref, k)
        ref = dict(zip(glob[0].tolist(), glob[1].tolist()))
        for r in ranks:
            gi, gv = _read_gout(r, r.last_parity())
            got = dict(zip(gi.cpu().tolist(), gv.cpu().tolist()))
            assert set(got) == set(ref), "rank %d epoch %d" % (r.rank, epoch)
            for j in ref:
                assert got[j] == pytest.approx(ref[j], rel=1e-5, abs=1e-9)
            assert torch.allclose(r.resid.cpu(), res_ref[r.rank], rtol=1e-5, atol=1e-9)


def test_region_guard_bands_detect_a_stray_write():
    """The canary bands around a peer-visible region are checked by reading
    them back; an ordinary torch write into the band (inside the same
    allocation) must be noticed."""
    from gtopkssgd_b200.ops import exchange as ex
    regions = ex.SymmetricRegion.create_emulated(2, ex.region_bytes(64, True), DEV)
    assert all(r.guards_intact() for r in regions)
    assert regions[0].tensor().numel() == regions[0].nbytes
    regions[0].tensor().fill_(7)              # the whole usable region may be written
    assert regions[0].guards_intact()
    regions[1]._owner[ex.GUARD_BYTES + regions[1].nbytes + 3] = 0   # first band byte range after the region
    assert not regions[1].guards_intact() and regions[0].guards_intact()


@pytest.mark.parametrize("mode", ["topk", "topk2"])
@pytest.mark.parametrize("P", [2, 3, 4])  # the all-gather modes need no power-of-two world
def test_k2t_allgather_emulated(P, mode):
    from gtopkssgd_b200.ops import exchange as ex
    from gtopkssgd_b200.ops.select import pairs_to_tensors
    torch.manual_seed(P)
    d, k = 200000, 500
    ranks, desc = _emulated_world(P, d, k, mode)
    seg_counts = torch.zeros(P * ex.MAX_PEERS, dtype=torch.int32, device=DEV)
    res_ref = [torch.zeros(d) for _ in range(P)]
    for epoch in (1, 2):
        grads = [torch.randn(d, device=DEV) for _ in range(P)]
        for r, g in zip(ranks, grads):
            r.selector.select(g, r.resid, k)
        ex.launch_allgather(ranks, desc, seg_counts, 0, P, k, reselect=(mode == "topk2"), nctas=2,
                            limit_ms=2000)
        torch.cuda.synchronize()
        local = [oracle.compress(g.cpu(), rr, k) for g, rr in zip(grads, res_ref)]
        for r in ranks:
            assert r.status() == (0, 0)
            counts = seg_counts[r.rank * ex.MAX_PEERS:r.rank * ex.MAX_PEERS + P].cpu().tolist()
            assert counts == [k] * P
            assert r.last_parity() == epoch & 1
            base = r.layout[1] + r.last_parity() * ex.MAX_PEERS * k * 8
            for q in range(P):
                raw = r.region.tensor()[base + q * k * 8: base + (q + 1) * k * 8].view(torch.int32).view(k, 2)
                qi, qv = pairs_to_tensors(raw, k)
                assert set(qi.cpu().tolist()) == set(local[q][0].tolist())
        if mode == "topk2":
            gi_ref, gv_ref = oracle.topk2_reselect(local, k)
            ref = dict(zip(gi_ref.tolist(), gv_ref.tolist()))
            for rr, loc in zip(res_ref, local):
                oracle.put_back(rr, loc, gi_ref)
            for r in ranks:
                gi, gv = _read_gout(r, r.last_parity())
                got = dict(zip(gi.cpu().tolist(), gv.cpu().tolist()))
                assert set(got) == set(ref)
                for j in ref:
                    assert got[j] == pytest.approx(ref[j], rel=1e-5, abs=1e-6)
                assert torch.allclose(r.resid.cpu(), res_ref[r.rank], rtol=1e-5, atol=1e-6)


def test_k2_bounded_wait_reports_timeout():
    """A receiver whose partner never sends must give up after the limit and
    report a status; the context stays usable.  Rank 0 of a 2-rank world is
    launched alone (its partner's kernel is simply not launched)."""
    from gtopkssgd_b200.ops import exchange as ex
    d, k = 10000, 10
    ranks, desc = _emulated_world(2, d, k)
    g = torch.randn(d, device=DEV)
    ranks[0].selector.select(g, ranks[0].resid, k)
    ex.launch_gtopk(ranks[:1], ranks[0].desc, 0, 2, k, nctas=2, limit_ms=50)
    torch.cuda.synchronize()
    status, where = ranks[0].status()
    assert status == 1 and 210 <= where < 220
    assert int(ranks[0].n_global.item()) == 0  # an empty global set: the consumer applies nothing
    assert int(ranks[0].epoch.item()) == 1     # the aborted call did not advance the counter
    # a failed exchange stays failed: the next call returns at once (no second wait), still empty
    import time
    ranks[0].n_global.fill_(123)
    t0 = time.time()
    ex.launch_gtopk(ranks[:1], ranks[0].desc, 0, 2, k, nctas=2, limit_ms=5000)
    ranks[0].mirror_status()
    torch.cuda.synchronize()
    assert time.time() - t0 < 2.0
    assert int(ranks[0].n_global.item()) == 0 and ranks[0].status()[0] == 1
    assert ranks[0].failed_on_host_mirror()[0] == 1  # what the host sees without synchronising
    # the host clears the failure (all ranks together); the device is healthy and a complete exchange works
    ranks[0].clear_failure()
    assert ranks[0].status() == (0, 0)
    for r in ranks:
        r.selector.select(torch.randn(d, device=DEV), r.resid, k)
    ex.launch_gtopk(ranks, desc, 0, 2, k, nctas=1, limit_ms=2000)
    torch.cuda.synchronize()
    assert all(r.status() == (0, 0) for r in ranks)
    assert [int(r.epoch.item()) for r in ranks] == [2, 2]
    assert int(ranks[1].n_global.item()) == k
