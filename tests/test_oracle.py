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
