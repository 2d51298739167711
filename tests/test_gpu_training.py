"""GPU end-to-end tests: the DistributedOptimizer on CUDA (fused select,
fused sparse SGD step, side stream) replayed against the oracle, on one GPU
and -- when the box has them -- on 2 and 4 GPUs through the peer-store
exchange kernel over CUDA IPC."""
import pytest
import torch

import _workers
from test_distributed_cpu import replay_and_check
from gtopkssgd_b200.ops import oracle
from gtopkssgd_b200.utils.launch import spawn_ranks

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("compressor", ["gtopk", "none"])
def test_single_gpu_training_matches_oracle(compressor):
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 1, args=(4, 0.001, compressor, "cuda"), timeout_s=300)
    replay_and_check(traces, 0.001, compressor, rtol=1e-4, atol=1e-5)


def test_single_gpu_three_merge_groups_overlap_backward():
    """Three merged groups: the select of a finished group runs on the side
    stream while backward continues."""
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 1, args=(4, 0.001, "gtopk", "cuda", 100000), timeout_s=300)
    assert len(traces[0]["groups"]) == 3
    replay_and_check(traces, 0.001, "gtopk", rtol=1e-4, atol=1e-5)


@pytest.mark.multigpu
def test_two_gpu_three_merge_groups():
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 2, args=(4, 0.001, "gtopk", "cuda", 100000), timeout_s=300,
                         env={"NCCL_NVLS_ENABLE": "0"})
    replay_and_check(traces, 0.001, "gtopk", rtol=1e-4, atol=1e-5)


@pytest.mark.multigpu
@pytest.mark.parametrize("compressor", ["gtopk", "topk", "topk2", "none"])
def test_two_gpu_training_matches_oracle(compressor):
    env = {"NCCL_NVLS_ENABLE": "0"}
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 2, args=(4, 0.001, compressor, "cuda"), timeout_s=300,
                         env=env)
    replay_and_check(traces, 0.001, compressor, rtol=1e-4, atol=1e-5)


@pytest.mark.multigpu
@pytest.mark.parametrize("compressor", ["gtopk", "topk2"])
def test_two_gpu_staged_transport_matches_oracle(compressor):
    """Ranks without GPU peer access (several hosts) exchange through the host
    and gloo; forced here on one host."""
    env = {"NCCL_NVLS_ENABLE": "0", "GTOPK_TRANSPORT": "staged"}
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 2, args=(4, 0.001, compressor, "cuda"), timeout_s=300,
                         env=env)
    replay_and_check(traces, 0.001, compressor, rtol=1e-4, atol=1e-5)


@pytest.mark.multigpu
def test_four_gpu_gtopk_matches_oracle():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 4, args=(3, 0.001, "gtopk", "cuda"), timeout_s=300,
                         env={"NCCL_NVLS_ENABLE": "0"})
    replay_and_check(traces, 0.001, "gtopk", rtol=1e-4, atol=1e-5)


@pytest.mark.multigpu
def test_eight_gpu_gtopk_matches_oracle():
    if torch.cuda.device_count() < 8:
        pytest.skip("needs 8 GPUs")
    traces = spawn_ranks(_workers.resnet20_gtopk_worker, 8, args=(3, 0.001, "gtopk", "cuda"), timeout_s=300,
                         env={"NCCL_NVLS_ENABLE": "0"})
    replay_and_check(traces, 0.001, "gtopk", rtol=1e-4, atol=1e-5)


def _check_real_peer_exchange(out, world, d, k, epochs):
    res_ref = [torch.zeros(d) for _ in range(world)]
    for e in range(epochs):
        # the same Philox stream as in the workers (seed-determined, whatever the device index)
        grads = [torch.randn(d, device="cuda:0", generator=torch.Generator(device="cuda:0").manual_seed(1000 * e + r)).cpu()
                 for r in range(world)]
        glob, local = oracle.simulate_gtopk_step(grads, res_ref, k)
        ref = dict(zip(glob[0].tolist(), glob[1].tolist()))
        for r in range(world):
            ep = out[r]["epochs"][e]
            assert tuple(ep["status"]) == (0, 0) and ep["guards"], (e, r, ep["status"])
            assert set(ep["local"][0].tolist()) == set(local[r][0].tolist()), "epoch %d rank %d: local selection" % (e, r)
            got = dict(zip(ep["global"][0].tolist(), ep["global"][1].tolist()))
            assert len(got) == k and set(got) == set(ref), \
                "epoch %d rank %d: %d extra, %d missing in the global set" % (e, r, len(set(got) - set(ref)), len(set(ref) - set(got)))
            for j, v in ref.items():
                assert got[j] == pytest.approx(v, rel=1e-5, abs=1e-6)
            assert torch.allclose(ep["resid"], res_ref[r], rtol=1e-5, atol=1e-6)


@pytest.mark.multigpu
@pytest.mark.parametrize("d,k,nctas", [(1_000_000, 1000, 1), (1_000_000, 5000, 4), (2_000_000, 14000, 16),
                                       (2_000_000, 20000, 24)])  # one CTA; clusters of 4 and 16; software barrier
def test_exchange_kernel_between_real_gpus_matches_oracle(d, k, nctas):
    """The multi-CTA forms of the exchange over NVLink peers: what the emulated single-GPU tests cannot
    see is whether a partner's flag can overtake data still in flight from other SMs."""
    world = 4 if torch.cuda.device_count() >= 4 else 2
    epochs = 6
    out = spawn_ranks(_workers.real_peer_exchange_worker, world, args=(d, k, nctas, epochs), timeout_s=300,
                      env={"NCCL_NVLS_ENABLE": "0"})
    _check_real_peer_exchange(out, world, d, k, epochs)


@pytest.mark.multigpu
@pytest.mark.parametrize("nctas", [1, 8])
def test_allgather_reselect_kernel_between_real_gpus_matches_oracle(nctas):
    """'topk2' over NVLink peers with one and with several CTAs per rank: every rank pushes its pairs into
    every peer's all-gather slots, merges the P lists in rank order and re-selects."""
    world = 4 if torch.cuda.device_count() >= 4 else 2
    d, k, epochs = 1_000_000, 4000, 4
    out = spawn_ranks(_workers.real_peer_exchange_worker, world, args=(d, k, nctas, epochs, "topk2"), timeout_s=300,
                      env={"NCCL_NVLS_ENABLE": "0"})
    res_ref = [torch.zeros(d) for _ in range(world)]
    for e in range(epochs):
        grads = [torch.randn(d, device="cuda:0", generator=torch.Generator(device="cuda:0").manual_seed(1000 * e + r)).cpu()
                 for r in range(world)]
        local = [oracle.compress(g, r, k) for g, r in zip(grads, res_ref)]
        gi_ref, gv_ref = oracle.topk2_reselect(local, k)
        for r, loc in zip(res_ref, local):
            oracle.put_back(r, loc, gi_ref)
        ref = dict(zip(gi_ref.tolist(), gv_ref.tolist()))
        for r in range(world):
            ep = out[r]["epochs"][e]
            assert tuple(ep["status"]) == (0, 0) and ep["guards"]
            got = dict(zip(ep["global"][0].tolist(), ep["global"][1].tolist()))
            assert len(got) == k and set(got) == set(ref), "epoch %d rank %d" % (e, r)
            for j, v in ref.items():
                assert got[j] == pytest.approx(v, rel=1e-5, abs=1e-6)
            assert torch.allclose(ep["resid"], res_ref[r], rtol=1e-5, atol=1e-6)


@pytest.mark.multigpu
def test_exchange_kernel_between_eight_gpus_matches_oracle():
    if torch.cuda.device_count() < 8:
        pytest.skip("needs 8 GPUs")
    d, k, epochs = 2_000_000, 14000, 4
    out = spawn_ranks(_workers.real_peer_exchange_worker, 8, args=(d, k, 16, epochs), timeout_s=300,
                      env={"NCCL_NVLS_ENABLE": "0"})
    _check_real_peer_exchange(out, 8, d, k, epochs)


def test_single_gpu_cuda_graph_step_matches_oracle():
    traces = spawn_ranks(_workers.graphed_step_worker, 1, args=(7, "gtopk"), timeout_s=300)
    assert traces[0]["graphs"] == 1
    replay_and_check(traces, 0.001, "gtopk", rtol=1e-4, atol=1e-5)


@pytest.mark.multigpu
@pytest.mark.parametrize("compressor,graphs", [("gtopk", 1), ("none", 0)])
def test_two_gpu_cuda_graph_step_matches_oracle(compressor, graphs):
    """gTop-k iterations are captured (peer-store exchange inside the graph);
    dense multi-GPU iterations stay eager by design."""
    traces = spawn_ranks(_workers.graphed_step_worker, 2, args=(7, compressor), timeout_s=240,
                         env={"NCCL_NVLS_ENABLE": "0"})
    assert traces[0]["graphs"] == graphs
    replay_and_check(traces, 0.001, compressor, rtol=1e-4, atol=1e-5)


def test_graft_smoke():
    import __graft_entry__ as g
    g.smoke()


def test_prefetched_batches_train_like_host_batches():
    """DLTrainer.prefetch copies a pinned batch on a side stream.  The consumer
    sees exactly the host data (also while the compute stream is busy), and
    ``train_step`` takes the handle in the eager and the CUDA-graph path: the
    first step, which depends only on the initial weights and the batch, gives
    the same loss as with the host batch."""
    import torch
    from gtopkssgd_b200.trainer.dl_trainer import DLTrainer, PrefetchedBatch

    def trainer(graph):
        torch.manual_seed(0)
        return DLTrainer(0, 1, dist=False, ngpus=1, batch_size=8, data_dir="synthetic", dataset="cifar10",
                         dnn="resnet20", lr=0.1, nworkers=1, device=torch.device("cuda", 0), synthetic_train_size=64,
                         cuda_graph=graph)

    g = torch.Generator().manual_seed(1)
    batches = [(torch.randn(8, 3, 32, 32, generator=g).pin_memory(),
                torch.randint(0, 10, (8,), generator=g).pin_memory()) for _ in range(6)]
    t = trainer(False)
    busy = torch.randn(4096, 4096, device="cuda")
    for b in batches * 3:
        h = t.prefetch(b)
        assert isinstance(h, PrefetchedBatch) and t.prefetch(h) is h
        busy = busy @ busy * 1e-4          # keeps the compute stream occupied while the copy runs
        x, y, _, _ = t._to_device(h)
        assert torch.equal(x.cpu(), b[0]) and torch.equal(y.cpu(), b[1])

    for graph in (False, True):
        first = {}
        for prefetch in (False, True):
            t = trainer(graph)
            nxt, losses = None, []
            for i, b in enumerate(batches):
                if prefetch:
                    cur = nxt if nxt is not None else t.prefetch(b)
                    nxt = t.prefetch(batches[i + 1]) if i + 1 < len(batches) else None
                else:
                    cur = b
                t.train_step(data=cur)
                losses.append(t.loss)
            assert all(l == l and l < 1e3 for l in losses)
            first[prefetch] = losses[0]
        assert abs(first[False] - first[True]) < 1e-4, first


@pytest.mark.multigpu
@pytest.mark.parametrize("leaver", [0, 1])
def test_two_gpu_planned_departure(leaver):
    """One of two GPU ranks announces its departure (between iterations,
    nothing in flight); the other closes its peer mappings, leaves the NCCL
    group and trains on alone from the agreed iteration."""
    total = 12
    out = spawn_ranks(_workers.elastic_worker, 2, args=("gtopk", leaver, 3, total, "cuda"), timeout_s=300,
                      env={"NCCL_NVLS_ENABLE": "0"})
    other = 1 - leaver
    at = out[leaver]["left_at"]
    assert at == 6 and out[leaver]["iters"] == at
    o = out[other]
    assert o["iters"] == total and o["calls"] == [(1, 0)]
    assert [h[1] for h in o["hist"]] == [2] * at + [1] * (total - at)
    import torch
    assert torch.isfinite(o["params"]).all() and not torch.equal(o["params"], out[leaver]["params"])
