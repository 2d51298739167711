"""One checked exchange on the real transport, compared with the oracle.

``exchange_selfcheck(optimizer)`` runs the select + exchange of every merged
group once more on whatever the gradient buffers hold, gathers every rank's
local selection through the CPU process group and recomputes on the host what
the reference's algorithm gives for them (``ops/oracle.py``: the
recursive-doubling tree of allreducer.py:71-163 for gTop-k, the re-selected sum
of allreducer.py:467-473 for 'topk2', the plain sum of allreducer.py:461-466
for 'topk'), then compares: the global index set, its values, that every rank
holds the same set, this rank's own top-k selection (as a property: nothing
left out is larger than anything taken, so ties at the k-th magnitude may fall
either way), and this rank's residual after the put-back
(compression.py:66-75).  It is meant for the end of a
benchmark or a smoke run on real GPUs, where the unit tests' emulated ranks do
not reach: collective (every rank calls it), synchronising, and it advances
the exchange state like one more iteration without a parameter update.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from ..ops import oracle
from ..ops.select import pairs_to_tensors
from . import comm


def _max_rel_err(got: dict, ref: dict) -> float:
    err = 0.0
    for j, v in ref.items():
        g = got.get(j)
        if g is None:
            return float("inf")
        err = max(err, abs(g - v) / max(abs(v), 1e-12))
    return err


def exchange_selfcheck(optimizer, rtol: float = 1e-5) -> dict:
    a = optimizer._allreducer
    world, rank = a.size(), a.rank()
    out = {"ok": True, "mode": a.mode, "world": world, "groups": []}
    if a.mode == "none" or world < 2:
        out["skipped"] = "nothing to exchange"
        return out
    density = a.get_current_density()
    for eng in a.engines:
        k = min(oracle.num_selected(eng.param_numel, density), eng.max_k)
        g = eng.grad.clone()
        r_before = eng.resid.clone()
        eng.reduce(density, None)
        if eng.is_cuda:
            torch.cuda.synchronize()
        status = eng.rank_ctx.status() if getattr(eng, "rank_ctx", None) is not None else (0, 0)
        li, lv = eng.selector.pairs()
        res = eng.result
        live = res.live_pairs()
        segs = []
        for s in range(res.nseg):
            n = int(res.counts[s])
            si, sv = pairs_to_tensors(live[s * res.seg_stride:(s + 1) * res.seg_stride], n)
            segs.append((si.cpu(), sv.cpu()))
        mine = {"local": (li.cpu(), lv.cpu()), "segs": segs, "status": status}
        everyone: List[dict] = [None] * world
        dist.all_gather_object(everyone, mine, group=comm.cpu_group())
        local_sets = [e["local"] for e in everyone]
        row = {"k": k, "status": [list(e["status"]) for e in everyone]}
        # what the reference's algorithm gives for these P local selections
        if a.mode == "gtopk":
            ref_i, ref_v = oracle.gtopk_tree(local_sets, k)
        elif a.mode == "topk2":
            ref_i, ref_v = oracle.topk2_reselect(local_sets, k)
        else:
            dense = oracle.topk_allgather_sum(local_sets, eng.numel)
            ref_i = dense.nonzero().flatten()
            ref_v = dense[ref_i]
        ref = dict(zip(ref_i.tolist(), ref_v.tolist()))
        if a.mode == "topk":
            acc = torch.zeros(eng.numel)
            for si, sv in segs:
                acc.index_add_(0, si, sv)
            gi = acc.nonzero().flatten()
            got = dict(zip(gi.tolist(), acc[gi].tolist()))
            same_everywhere = True
        else:
            gi, gv = segs[0]
            got = dict(zip(gi.tolist(), gv.tolist()))
            row["n_global"] = len(got)
            same_everywhere = all(set(e["segs"][0][0].tolist()) == set(got) for e in everyone)
        row["index_sets_equal"] = set(got) == set(ref)
        if not row["index_sets_equal"]:
            # what kind of difference: entries that no rank selected in this call can only come from a
            # receive slot that was read before (all of) this call's data had landed in it
            union = set()
            for li_, _ in local_sets:
                union.update(li_.tolist())
            extra, missing = set(got) - set(ref), set(ref) - set(got)
            row["n_extra"], row["n_missing"] = len(extra), len(missing)
            row["n_extra_not_in_any_local_selection"] = len(extra - union)
            # entries of equal magnitude at the k-th place may be chosen either way by a tree node
            row["tie_swap"] = sorted(abs(got[j]) for j in extra) == sorted(abs(ref[j]) for j in missing)
        common = {j: v for j, v in ref.items() if j in got}
        row["max_rel_err"] = _max_rel_err(got, common) if (row["index_sets_equal"] or row.get("tie_swap")) \
            else float("inf")
        row["all_ranks_same_set"] = bool(same_everywhere)
        # this rank's own select and residual.  A top-k selection is right when it has min(k, d) distinct
        # entries, carries acc = g + r at them, and no entry left out is larger in magnitude than one taken
        # (entries EQUAL to the k-th magnitude may be chosen either way: which of them torch.topk would
        # have picked is not part of the semantics); non-finite entries count as the largest.
        acc = g + r_before
        mag = torch.nan_to_num(acc.abs(), nan=float("inf"))
        taken = torch.zeros(acc.numel(), dtype=torch.bool, device=acc.device)
        li_d = li.to(acc.device)
        taken[li_d] = True
        n_taken = int(taken.sum())
        min_in = float(mag[taken].min()) if n_taken else float("inf")
        max_out = float(mag[~taken].max()) if n_taken < acc.numel() else 0.0
        vals_ok = bool(torch.equal(torch.nan_to_num(acc[li_d]), torch.nan_to_num(lv.to(acc.device))))
        row_sel = n_taken == li.numel() == min(k, acc.numel()) and min_in >= max_out and vals_ok
        row["ties_at_kth_on_rank_%d" % rank] = int((mag == min_in).sum()) if n_taken else 0
        r_exp = torch.where(taken, torch.zeros_like(acc), acc)
        if a.mode != "topk":
            # against the global set this rank actually holds (checked against the oracle's above)
            oracle.put_back(r_exp, (li_d, lv.to(acc.device)), segs[0][0].to(r_exp.device))
        row_res = bool(torch.allclose(eng.resid, r_exp, rtol=1e-5, atol=1e-7, equal_nan=True))
        flags = torch.tensor([int(row_sel), int(row_res)], dtype=torch.int32)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN, group=comm.cpu_group())
        row["select_ok_all_ranks"], row["residual_ok_all_ranks"] = bool(flags[0]), bool(flags[1])
        row["ok"] = bool((row["index_sets_equal"] or row.get("tie_swap")) and row["max_rel_err"] <= rtol
                         and row["all_ranks_same_set"]
                         and row["select_ok_all_ranks"] and row["residual_ok_all_ranks"]
                         and all(s == [0, 0] for s in row["status"]))
        out["groups"].append(row)
        out["ok"] = out["ok"] and row["ok"]
    g0 = out["groups"][0]
    out["k"] = g0["k"]
    out["max_rel_err"] = max(r["max_rel_err"] for r in out["groups"])
    return out
