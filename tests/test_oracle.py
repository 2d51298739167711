"""CPU tests of the PyTorch oracle: the semantics every kernel is held to."""
import numpy as np
import pytest
import torch

from gtopkssgd_b200.ops import oracle


def brute_force_tree(sets, k):
    """Independent restatement of the recursive-doubling merge with numpy
    dictionaries (no shared code with the oracle)."""
    sets = [dict(zip(i.tolist(), v.tolist())) for i, v in sets]
    P = len(sets)
    step = 1
    while step < P:
        for i in range(0, P, 2 * step):
            a, b = sets[i], sets[i + step]
            merged = dict(a)
            for j, v in b.items():
                merged[j] = np.float32(np.float32(merged.get(j, 0.0)) + np.float32(v)) if j in merged else v
            items = sorted(merged.items(), key=lambda kv: -abs(kv[1]))[:k]
            sets[i] = dict(items)
        step *= 2
    return sets[0]


@pytest.mark.parametrize("P", [1, 2, 4, 8])
def test_tree_matches_brute_force(P):
    torch.manual_seed(P)
    d, k = 5000, 37
    sets = []
    for r in range(P):
        g = torch.randn(d)
        idx, val = oracle.compress(g, torch.zeros(d), k)
        sets.append((idx, val))
    gi, gv = oracle.gtopk_tree(sets, k)
    ref = brute_force_tree(sets, k)
    assert gi.numel() <= k
    assert set(gi.tolist()) == set(ref.keys())
    for j, v in zip(gi.tolist(), gv.tolist()):
        assert abs(v - ref[j]) <= 1e-6 * max(1.0, abs(v))


def test_compress_residual_semantics():
    torch.manual_seed(0)
    d, k = 1000, 10
    g, r = torch.randn(d), torch.randn(d) * 0.1
    acc = g + r
    idx, val = oracle.compress(g, r, k)
    assert idx.numel() == k
    assert torch.equal(val, acc[idx])
    assert torch.all(r[idx] == 0)
    mask = torch.ones(d, dtype=torch.bool)
    mask[idx] = False
    assert torch.equal(r[mask], acc[mask])
    assert acc.abs()[mask].max() <= val.abs().min()


def test_put_back_by_index_membership():
    r = torch.zeros(10)
    local = (torch.tensor([1, 3, 5]), torch.tensor([1.0, -2.0, 3.0]))
    oracle.put_back(r, local, torch.tensor([3, 7]))
    assert r.tolist() == [0, 1.0, 0, 0, 0, 3.0, 0, 0, 0, 0]


def test_mass_conservation_two_ranks():
    """sum_p (g_p + r_prev_p) = scatter(global) + sum_p r_new_p, except for
    values truncated inside the tree (none at P=2 when the union fits)."""
    torch.manual_seed(1)
    d, k = 64, 64  # k = d: nothing is ever truncated
    grads = [torch.randn(d) for _ in range(2)]
    res = [torch.zeros(d) for _ in range(2)]
    total = grads[0] + grads[1]
    glob, _ = oracle.simulate_gtopk_step(grads, res, k)
    dense = torch.zeros(d)
    dense[glob[0]] = glob[1]
    assert torch.allclose(dense + res[0] + res[1], total, atol=1e-6)


def test_power_of_two_only():
    with pytest.raises(ValueError):
        oracle.tree_rounds(6)


def test_sgd_matches_torch_optim():
    torch.manual_seed(2)
    p = torch.randn(100)
    q = p.clone().requires_grad_(True)
    opt = torch.optim.SGD([q], lr=0.1, momentum=0.9, weight_decay=1e-4)
    buf = torch.zeros(100)
    for step in range(3):
        g = torch.randn(100)
        q.grad = g.clone()
        opt.step()
        oracle.sgd_step(p, buf, g, 0.1, 0.9, 0.0, 1e-4, False, first_step=(step == 0))
    assert torch.allclose(p, q.detach(), atol=1e-6)


def test_topk2_is_topk_of_sum():
    torch.manual_seed(3)
    d, k, P = 2000, 20, 4
    sets = [oracle.compress(torch.randn(d), torch.zeros(d), k) for _ in range(P)]
    dense = oracle.topk_allgather_sum(sets, d)
    gi, gv = oracle.topk2_reselect(sets, k)
    _, ref = torch.topk(dense.abs(), k)
    assert set(gi.tolist()) == set(ref.tolist())
    assert torch.allclose(dense[gi], gv, atol=1e-6)


# ---- property tests (hypothesis): invariants of one gTop-k exchange for random sizes and worlds
from hypothesis import given, settings as hsettings, strategies as hst  # noqa: E402


@hsettings(max_examples=60, deadline=None)
@given(logp=hst.integers(0, 3), d=hst.integers(8, 300), kfrac=hst.floats(0.01, 1.0), seed=hst.integers(0, 10 ** 6))
def test_exchange_invariants(logp, d, kfrac, seed):
    P = 1 << logp
    k = max(int(d * kfrac), 1)
    g = torch.Generator().manual_seed(seed)
    grads = [torch.randn(d, generator=g) for _ in range(P)]
    res_prev = [torch.randn(d, generator=g) * 0.1 for _ in range(P)]
    res = [r.clone() for r in res_prev]
    (gi, gv), local = oracle.simulate_gtopk_step(grads, res, k)
    # the global set: at most k entries, each index once, drawn from the union of the local selections
    assert gi.numel() <= k and gi.unique().numel() == gi.numel()
    union = torch.cat([l[0] for l in local]).unique()
    assert torch.isin(gi, union).all()
    in_global = torch.zeros(d, dtype=torch.bool)
    in_global[gi] = True
    for p in range(P):
        acc = grads[p] + res_prev[p]
        li, lv = local[p]
        assert li.numel() == min(k, d) and torch.equal(lv, acc[li])
        # local selection = the k largest magnitudes of acc
        kth = acc.abs().topk(min(k, d)).values.min()
        mask = torch.zeros(d, dtype=torch.bool)
        mask[li] = True
        assert (acc.abs()[mask] >= kth).all() and (acc.abs()[~mask] <= kth).all()
        # residual: 0 exactly where the entry was selected locally AND its index is in the global set
        gone = mask & in_global
        assert torch.equal(res[p][gone], torch.zeros(int(gone.sum())))
        assert torch.equal(res[p][~gone], acc[~gone])
    # a global value is the sum of the contributions that survived the tree; with k >= d nothing is cut
    if k >= d:
        dense = torch.zeros(d)
        dense[gi] = gv
        assert torch.allclose(dense, sum(gr + rp for gr, rp in zip(grads, res_prev)), atol=1e-5)
    if P == 1:
        assert set(gi.tolist()) == set(local[0][0].tolist())


@hsettings(max_examples=30, deadline=None)
@given(logp=hst.integers(1, 3), d=hst.integers(16, 200), seed=hst.integers(0, 10 ** 6))
def test_identical_workers_agree_with_local_topk(logp, d, seed):
    """All ranks hold the same gradient: the tree keeps exactly the local
    selection and every value is P times the local one."""
    P, k = 1 << logp, max(d // 8, 1)
    g = torch.randn(d, generator=torch.Generator().manual_seed(seed))
    res = [torch.zeros(d) for _ in range(P)]
    (gi, gv), local = oracle.simulate_gtopk_step([g.clone() for _ in range(P)], res, k)
    order, lorder = gi.argsort(), local[0][0].argsort()
    assert torch.equal(gi[order], local[0][0][lorder])
    assert torch.allclose(gv[order], P * local[0][1][lorder])
    for r in res:  # nothing selected locally was dropped globally: the residual holds only unselected entries
        assert torch.equal(r[gi], torch.zeros(gi.numel()))


@hsettings(max_examples=40, deadline=None)
@given(P=hst.integers(1, 6), d=hst.integers(8, 200), kfrac=hst.floats(0.02, 0.6), seed=hst.integers(0, 10 ** 6))
def test_allgather_modes_invariants(P, d, kfrac, seed):
    """'topk' is the dense sum of the P local selections; 'topk2' keeps the k
    largest magnitudes of that sum (any world size)."""
    k = max(int(d * kfrac), 1)
    g = torch.Generator().manual_seed(seed)
    local = [oracle.compress(torch.randn(d, generator=g), torch.zeros(d), k) for _ in range(P)]
    dense = oracle.topk_allgather_sum(local, d)
    ref = torch.zeros(d)
    for idx, val in local:
        ref[idx] += val
    assert torch.allclose(dense, ref, atol=1e-6)
    gi, gv = oracle.topk2_reselect(local, k)
    assert gi.numel() <= k and gi.unique().numel() == gi.numel()
    assert torch.allclose(gv, dense[gi], atol=1e-5)
    nz = int((dense != 0).sum())
    if nz > k:  # nothing outside the selection beats anything inside it
        outside = dense.abs().clone()
        outside[gi] = 0
        assert outside.max() <= gv.abs().min() + 1e-6
