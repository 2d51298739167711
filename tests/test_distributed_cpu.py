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
    residuals.  (Comparing free-running trajectories instead would be
    chaotic: one flipped top-k entry changes every later gradient.)"""
    world = len(traces)
    numel = traces[0]["numel"]
    total = traces[0]["p0"].numel()
    k = oracle.num_selected(numel, density)
    res = [torch.zeros(numel) for _ in range(world)]
    bufs = [torch.zeros(numel) for _ in range(world)]
    params = [t["p0"][:numel].clone() for t in traces]
    assert total - numel < 64  # one group: only tail padding
    for it in range(len(traces[0]["grads"])):
        grads = [t["grads"][it][:numel] for t in traces]
        if compressor == "gtopk":
            glob, _ = oracle.simulate_gtopk_step(grads, res, k)
            dense = oracle.scatter_average(glob, numel, world)
        elif compressor == "topk":
            local = [oracle.compress(g, r, k) for g, r in zip(grads, res)]
            dense = oracle.topk_allgather_sum(local, numel) / world
        elif compressor == "topk2":
            local = [oracle.compress(g, r, k) for g, r in zip(grads, res)]
            gi, gv = oracle.topk2_reselect(local, k)
            for r, loc in zip(res, local):
                oracle.put_back(r, loc, gi)
            dense = oracle.scatter_average((gi, gv), numel, world)
        else:
            # dense mode reduces in place inside the hook: the recorded buffer already holds the sum
            assert all(torch.equal(grads[0], g) for g in grads[1:])
            dense = grads[0] / world
        for r in range(world):
            lr = traces[r]["lrs"][it] if "lrs" in traces[r] else 0.1
            oracle.sgd_step(params[r], bufs[r], dense, lr, 0.9, 0.0, 1e-4, False, first_step=(it == 0))
            got = traces[r]["params"][it][:numel]
            assert torch.allclose(got, params[r], rtol=rtol, atol=atol), (it, r, float((got - params[r]).abs().max()))
            if compressor != "none":
                assert torch.allclose(traces[r]["resid"][it][:numel], res[r], rtol=rtol, atol=atol), (it, r)
            params[r] = got.clone()  # teacher forcing
    for r in range(1, world):  # replicas stay identical
        assert torch.equal(traces[0]["params"][-1], traces[r]["params"][-1])


@pytest.mark.parametrize("compressor", ["gtopk", "topk", "topk2", "none"])
def test_resnet20_two_workers_gloo_matches_oracle(compressor):
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 2, args=(3, 0.001, compressor), timeout_s=600)
    replay_and_check(traces, 0.001, compressor)


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
