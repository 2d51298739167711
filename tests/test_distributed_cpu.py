"""Multi-process CPU tests over gloo: the plumbing config (ResNet-20, two
workers, gTop-k density 0.001, momentum SGD with residuals) against a
single-process simulation built from the oracle, plus host-side fault
injection."""
import pytest
import torch

from gtopkssgd_b200.ops import oracle
from gtopkssgd_b200.utils.launch import spawn_ranks

import _workers


def replay_and_check(traces, density, compressor, rtol=1e-5, atol=1e-6):
    """Teacher-forced replay: every iteration the oracle gets the gradients the
    workers actually produced and must reproduce their parameters and
    residuals, merged group by merged group.  (Comparing free-running
    trajectories instead would be chaotic: one flipped top-k entry changes every
    later gradient.)"""
    world = len(traces)
    total = traces[0]["p0"].numel()
    # (start, span in the flat buffer, parameter count): k follows the parameter count, the alignment
    # gaps inside a span hold zeros and never win
    groups = [tuple(g) if len(g) == 3 else (g[0], g[1], g[1])
              for g in (traces[0].get("groups") or [(0, traces[0]["numel"])])]
    res = [torch.zeros(total) for _ in range(world)]
    bufs = [torch.zeros(total) for _ in range(world)]
    params = [t["p0"].clone() for t in traces]
    for it in range(len(traces[0]["grads"])):
        dense = torch.zeros(total)
        for start, numel, nparam in groups:
            sl = slice(start, start + numel)
            k = oracle.num_selected(nparam, density)
            grads = [t["grads"][it][sl] for t in traces]
            rs = [r[sl] for r in res]  # views: updated in place
            if compressor == "gtopk":
                glob, _ = oracle.simulate_gtopk_step(grads, rs, k)
                dense[sl] = oracle.scatter_average(glob, numel, world)
            elif compressor == "topk":
                local = [oracle.compress(g, r, k) for g, r in zip(grads, rs)]
                dense[sl] = oracle.topk_allgather_sum(local, numel) / world
            elif compressor == "topk2":
                local = [oracle.compress(g, r, k) for g, r in zip(grads, rs)]
                gi, gv = oracle.topk2_reselect(local, k)
                for r, loc in zip(rs, local):
                    oracle.put_back(r, loc, gi)
                dense[sl] = oracle.scatter_average((gi, gv), numel, world)
            else:
                # dense mode reduces in place inside the hook: the recorded buffer already holds the sum
                assert all(torch.equal(grads[0], g) for g in grads[1:])
                dense[sl] = grads[0] / world
        for r in range(world):
            lr = traces[r]["lrs"][it] if "lrs" in traces[r] else 0.1
            oracle.sgd_step(params[r], bufs[r], dense, lr, 0.9, 0.0, 1e-4, False, first_step=(it == 0))
            got = traces[r]["params"][it]
            for start, numel, _ in groups:  # padding between groups is not compared
                sl = slice(start, start + numel)
                assert torch.allclose(got[sl], params[r][sl], rtol=rtol, atol=atol), \
                    (it, r, start, float((got[sl] - params[r][sl]).abs().max()))
                if compressor != "none":
                    assert torch.allclose(traces[r]["resid"][it][sl], res[r][sl], rtol=rtol, atol=atol), (it, r, start)
            params[r] = got.clone()  # teacher forcing
    for r in range(1, world):  # replicas stay identical
        assert torch.equal(traces[0]["params"][-1], traces[r]["params"][-1])


@pytest.mark.parametrize("compressor", ["gtopk", "topk", "topk2", "none"])
def test_resnet20_two_workers_gloo_matches_oracle(compressor):
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 2, args=(3, 0.001, compressor), timeout_s=600)
    replay_and_check(traces, 0.001, compressor)


def test_two_workers_three_merge_groups_gloo():
    """Merge threshold of 100 000 elements: ResNet-20 splits into three groups,
    each selected and exchanged on its own."""
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 2, args=(3, 0.001, "gtopk", "cpu", 100000), timeout_s=600)
    assert len(traces[0]["groups"]) == 3
    replay_and_check(traces, 0.001, "gtopk")


def test_four_workers_gtopk_gloo():
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 4, args=(2, 0.001, "gtopk"), timeout_s=600)
    replay_and_check(traces, 0.001, "gtopk")


@pytest.mark.parametrize("mode", ["exit", "stall"])
def test_missing_peer_raises_and_calls_err_handler(mode):
    out = spawn_ranks(_workers.failing_peer_worker, 2, args=(mode,), timeout_s=240, allow_failures=True)
    status0, res0 = out[0]
    assert status0 == "ok", res0
    assert res0[0] == "timeout", res0
    assert res0[1] < 60
    assert res0[2] == [(1, 0)]  # err_handler(new world size, my rank)


def test_orderly_departure_is_seen_on_the_host_before_the_next_launch():
    out = spawn_ranks(_workers.leaving_peer_worker, 2, timeout_s=240)
    assert out[1] == "left"
    kind, seconds, calls, msg = out[0]
    assert kind == "left-detected" and seconds < 2.0  # far below the 30 s wait limit
    assert calls == [(1, 0)] and "[1]" in msg


def test_trainer_saves_state_when_a_peer_leaves(tmp_path):
    out = spawn_ranks(_workers.interrupted_trainer_worker, 2, args=(str(tmp_path),), timeout_s=300)
    assert out[1] == {"finished": True}
    r0 = out[0]
    assert "left the job" in r0["error"], r0
    assert len(r0["files"]) == 1 and r0["iter"] == 2
    assert {"epoch", "iter", "optimizer", "residuals", "state"} <= set(r0["keys"]) and r0["n_resid"] > 0


@pytest.mark.parametrize("compressor", ["topk", "topk2"])
def test_three_workers_allgather_modes(compressor):
    """The all-gather modes have no tree and run on any world size."""
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 3, args=(2, 0.001, compressor), timeout_s=600)
    replay_and_check(traces, 0.001, compressor)


def test_three_workers_gtopk_is_refused():
    out = spawn_ranks(_workers.gtopk_world3_worker, 3, timeout_s=120)
    assert all("power-of-two" in o for o in out), out


@pytest.mark.parametrize("world,compressor,leaver", [(4, "topk2", 3), (4, "gtopk", 1), (2, "gtopk", 0)])
def test_planned_departure_shrinks_the_job(world, compressor, leaver):
    """A rank announces its departure; every survivor drops it at the same
    iteration, the process group is re-formed and training continues.  With
    three workers left gTop-k (power-of-two tree) continues as topk2."""
    total, leave_iter = 12, 3
    out = spawn_ranks(_workers.elastic_worker, world, args=(compressor, leaver, leave_iter, total), timeout_s=300)
    at = out[leaver]["left_at"]
    assert at == 6                                   # announced at 3, check points every 2: (3 // 2 + 2) * 2
    assert out[leaver]["iters"] == at                # the leaver took part in iterations 0 .. at-1
    survivors = [r for r in range(world) if r != leaver]
    for new_rank, r in enumerate(survivors):
        o = out[r]
        assert o["iters"] == total and o["calls"] == [(world - 1, new_rank)]
        assert [h[1] for h in o["hist"]] == [world] * at + [world - 1] * (total - at)
        assert o["hist"][-1][2] == new_rank
        expected_mode = compressor if (world - 1) & (world - 2) == 0 or compressor != "gtopk" else "topk2"
        assert o["hist"][-1][3] == expected_mode
        assert torch.isfinite(o["params"]).all()
    for r in survivors[1:]:                          # the replicas stay identical after the shrink
        assert torch.equal(out[survivors[0]]["params"], out[r]["params"])
    assert not torch.equal(out[leaver]["params"], out[survivors[0]]["params"])


def test_elastic_training_driver(tmp_path):
    out = spawn_ranks(_workers.elastic_trainer_worker, 2, args=(str(tmp_path),), timeout_s=300)
    assert out[1]["iters"] == 6 and out[1]["nworkers"] == 2          # asked after iteration 1 (train_iter 2): effective at 6
    assert out[0]["iters"] == 10 and out[0]["nworkers"] == 1 and out[0]["world_now"] == 1
    assert out[0]["loss"] == out[0]["loss"]


def test_validation_longer_than_the_wait_limit_does_not_time_out(tmp_path):
    """Rank 0 validates for 4 s at every epoch boundary while the exchange's wait limit is 1.5 s: the
    other rank meets it at a host barrier instead of running into a bounded wait."""
    out = spawn_ranks(_workers.slow_validation_worker, 2, args=(str(tmp_path),), timeout_s=300)
    assert out[0]["validations"] >= 2
    assert out[0]["iters"] == out[1]["iters"] and out[0]["iters"] >= 6
    assert out[0]["epoch"] == out[1]["epoch"] >= 2


@pytest.mark.parametrize("world,compressor", [(2, "gtopk"), (4, "gtopk"), (3, "topk2"), (2, "topk")])
def test_exchange_selfcheck_on_gloo_ranks(world, compressor):
    """The checked exchange that the benchmark runs on real GPUs, here over the gloo fallback."""
    out = spawn_ranks(_workers.selfcheck_worker, world, args=(compressor,), timeout_s=300)
    for o in out:
        assert o["ok"], o
        assert len(o["groups"]) >= 2 and o["max_rel_err"] <= 1e-5
        assert all(g["index_sets_equal"] and g["residual_ok_all_ranks"] and g["select_ok_all_ranks"] for g in o["groups"])


def test_topk_allgather_with_half_precision_wire_values():
    import numpy as np
    out = spawn_ranks(_workers.fp16_wire_worker, 2, timeout_s=120)
    want_v = np.concatenate([((np.arange(4, dtype=np.float32) + 1.0) * (1.0 + r) / 3.0).astype(np.float16) for r in range(2)])
    want_i = np.concatenate([np.arange(4) + 10 * r for r in range(2)]).astype(np.uint32)
    for o in out:
        assert o["v"].dtype == np.float16 and np.array_equal(o["v"], want_v) and np.array_equal(o["i"], want_i)
