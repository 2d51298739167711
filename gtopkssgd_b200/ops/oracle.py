"""Plain PyTorch statement of every sparse-gradient operation.

This module is three things at once: the numerics oracle that the CUDA kernels
are tested against, the implementation used on CPU tensors (the gloo fallback
path), and an executable description of the reference semantics:

* compression.py:32-57  -- residual add, magnitude top-k, residual write-back
* compression.py:66-75  -- put-back of "selected locally, not globally" values
* allreducer.py:71-163  -- the recursive-doubling gTop-k tree
* allreducer.py:29-64, 461-473 -- Top-k all-gather and its re-selecting variant
* distributed_optimizer.py:105-143 -- weight decay + momentum/nesterov SGD

All functions work on 1-D fp32 tensors of any device and allocate freely; none
of them is meant to be fast.
"""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple

import torch

Pairs = Tuple[torch.Tensor, torch.Tensor]  # (int64 indices, fp32 values)


def num_selected(numel: int, density: float) -> int:
    """k = max(int(d * rho), 1), as in compression.py:39."""
    return max(int(numel * density), 1)


def compress(g: torch.Tensor, r: torch.Tensor, k: int, scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """acc = scale*g + r; returns the k largest-magnitude (idx, acc[idx]) and
    leaves r = acc off the selection, 0 on it (in place)."""
    acc = torch.addcmul(r, g, torch.as_tensor(scale, dtype=g.dtype, device=g.device)) if scale != 1.0 else g + r
    k = min(k, acc.numel())
    _, idx = torch.topk(acc.abs(), k, sorted=False)
    val = acc[idx].clone()
    r.copy_(acc)
    r[idx] = 0.0
    return idx, val


def merge_select(a: Pairs, b: Pairs, k: int) -> Pairs:
    """Union of two sparse sets with values summed on shared indices, cut to
    the k largest magnitudes (one tree node of allreducer.py:117-131; a shared
    index appears once)."""
    idx = torch.cat([a[0], b[0]])
    val = torch.cat([a[1], b[1]])
    uniq, inv = torch.unique(idx, return_inverse=True)
    sums = torch.zeros(uniq.numel(), dtype=val.dtype, device=val.device).index_add_(0, inv, val)
    if uniq.numel() > k:
        _, top = torch.topk(sums.abs(), k, sorted=False)
        uniq, sums = uniq[top], sums[top]
    return uniq, sums


def tree_rounds(world: int) -> int:
    if world < 1 or world & (world - 1):
        raise ValueError("gTop-k needs a power-of-two number of workers, got %d" % world)
    return int(math.log2(world))


def gtopk_tree(sets: Sequence[Pairs], k: int) -> Pairs:
    """Global set that rank 0 holds after log2(P) rounds: round r merges rank
    i + 2^r into rank i for i = 0 mod 2^(r+1)."""
    sets = list(sets)
    world = len(sets)
    for r in range(tree_rounds(world)):
        step = 1 << r
        for i in range(0, world, 2 * step):
            sets[i] = merge_select(sets[i], sets[i + step], k)
    return sets[0]


def topk_allgather_sum(sets: Sequence[Pairs], numel: int) -> torch.Tensor:
    """Dense sum of the P sparse vectors ('topk' mode)."""
    out = torch.zeros(numel, dtype=sets[0][1].dtype, device=sets[0][1].device)
    for idx, val in sets:
        out.index_add_(0, idx, val)
    return out


def topk2_reselect(sets: Sequence[Pairs], k: int) -> Pairs:
    """'topk2': sum all P selections (in rank order), keep the k largest sums."""
    acc = sets[0]
    for s in sets[1:]:
        acc = merge_select(acc, s, 1 << 62)
    if acc[0].numel() > k:
        _, top = torch.topk(acc[1].abs(), k, sorted=False)
        acc = (acc[0][top], acc[1][top])
    return acc


def put_back(r: torch.Tensor, local: Pairs, global_idx: torch.Tensor) -> None:
    """Entries selected locally whose index is not in the global set return to
    the residual; membership is by index only."""
    keep = ~torch.isin(local[0], global_idx)
    r[local[0][keep]] += local[1][keep]


def scatter_average(pairs: Pairs, numel: int, world: int) -> torch.Tensor:
    out = torch.zeros(numel, dtype=pairs[1].dtype, device=pairs[1].device)
    out[pairs[0]] = pairs[1]
    return out / world


def sgd_step(p: torch.Tensor, buf: torch.Tensor | None, g: torch.Tensor, lr: float, momentum: float = 0.0,
             dampening: float = 0.0, weight_decay: float = 0.0, nesterov: bool = False,
             first_step: bool = False) -> None:
    """In-place momentum SGD exactly as distributed_optimizer.py:105-143: decay
    is added to the (already averaged, sparsified) gradient, the first step
    sets buf = d_p."""
    d_p = g + weight_decay * p if weight_decay != 0 else g.clone()
    if momentum != 0:
        assert buf is not None
        if first_step:
            buf.mul_(momentum).add_(d_p)
        else:
            buf.mul_(momentum).add_(d_p, alpha=1 - dampening)
        d_p = d_p.add(buf, alpha=momentum) if nesterov else buf
    p.add_(d_p, alpha=-lr)


def clip_coef(total_norm: float, max_norm: float) -> float:
    c = max_norm / (total_norm + 1e-6)
    return c if c < 1 else 1.0


def simulate_gtopk_step(grads: List[torch.Tensor], residuals: List[torch.Tensor], k: int) -> Tuple[Pairs, List[Pairs]]:
    """One full gTop-k exchange for P simulated ranks: compress each rank,
    run the tree, put back.  Returns the global set and the local selections;
    residuals are updated in place."""
    local = [compress(g, r, k) for g, r in zip(grads, residuals)]
    glob = gtopk_tree(local, k)
    for r, loc in zip(residuals, local):
        put_back(r, loc, glob[0])
    return glob, local
