"""The reference arm's plumbing, checked without a GPU.

* the reference's own ``gtopk_sparse_allreduce`` / ``topk_sparse_allreduce``
  (``allreducer.py:29-163``), run unmodified over the mpi4py stand-in on gloo
  ranks, give what ``ops/oracle.py`` gives: this pins the oracle (and so every
  kernel tested against it) to the reference's code, not to a reading of it;
* ``baseline/ref_arm.py`` drives the reference's trainer, optimizer wrapper and
  communication thread end to end (dry run on CPU) and prints the bench line.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "allreducer.py")),
                                reason="baseline/_ref (copy of the reference tree) is not present")


def _torchrun(nproc, script, args, port, timeout=600):
    env = dict(os.environ)
    env.pop("PYTHONPATH", None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
           "--master-addr", "127.0.0.1", "--master-port", str(port), script] + [str(a) for a in args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


def test_manifest_matches_copy():
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import setup_ref
        assert setup_ref.verify(REF)
    finally:
        sys.path.pop(0)


@pytest.mark.parametrize("world", [2, 4])
def test_reference_algorithms_match_oracle(tmp_path, world):
    from gtopkssgd_b200.ops import oracle
    d, k = 4000, 64
    r = _torchrun(world, os.path.join(ROOT, "tests", "_ref_worker.py"), [str(tmp_path), d, k], 29610 + world)
    assert r.returncode == 0, r.stderr[-3000:]
    sets = []
    for rank in range(world):
        sets.append((torch.from_numpy(np.load(tmp_path / ("in_idx_%d.npy" % rank))),
                     torch.from_numpy(np.load(tmp_path / ("in_val_%d.npy" % rank)))))
    gi, gv = oracle.gtopk_tree(sets, k)
    want = dict(zip(gi.tolist(), gv.tolist()))
    for rank in range(world):
        idx = np.load(tmp_path / ("g_idx_%d.npy" % rank))
        val = np.load(tmp_path / ("g_val_%d.npy" % rank))
        assert len(idx) == k and set(idx.tolist()) == set(want), "rank %d: global index set differs" % rank
        for i, v in zip(idx.tolist(), val.tolist()):
            assert abs(v - want[i]) <= 1e-5 * max(1.0, abs(want[i]))
        # included = positions of the local selection whose index is in the global set
        inc = np.load(tmp_path / ("g_inc_%d.npy" % rank))
        local_idx = sets[rank][0].numpy()
        assert set(local_idx[inc].tolist()) == set(local_idx.tolist()) & set(want)
        resid_ref = torch.zeros(d)
        keep = np.ones(k, dtype=bool)
        keep[inc] = False
        resid_ref[sets[rank][0][keep]] += sets[rank][1][keep]
        resid = torch.zeros(d)
        oracle.put_back(resid, sets[rank], gi)
        assert torch.equal(resid, resid_ref)
        # all-gather variant: P*k pairs in rank order
        ti = np.load(tmp_path / ("t_idx_%d.npy" % rank))
        tv = np.load(tmp_path / ("t_val_%d.npy" % rank))
        dense = torch.zeros(d).index_add_(0, torch.from_numpy(ti), torch.from_numpy(tv))
        assert torch.allclose(dense, oracle.topk_allgather_sum(sets, d), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("compressor", ["gtopk", "none"])
def test_ref_arm_dry_run_two_ranks(compressor):
    r = _torchrun(2, os.path.join(ROOT, "baseline", "ref_arm.py"),
                  ["--cpu-dry-run", "--gpus", 2, "--model", "resnet20", "--steps", 3, "--warmup", 3,
                   "--compressor", compressor], 29620 + len(compressor))
    assert r.returncode == 0, r.stderr[-3000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and out["n_gpus"] == 2 and out["value"] > 0
    assert out["config"]["source_matches_manifest"] is True
    assert out["e2e"]["h2d_bytes_per_step"] == 32 * 3 * 32 * 32 * 4 + 32 * 8
    if compressor == "gtopk":
        assert out["comm_ms_per_iter"]["exchange_ms"] > 0 and out["comm_ms_per_iter"]["select_ms"] > 0


def test_bench_reference_flag_hands_over(tmp_path):
    """bench.py --impl reference replaces itself with the reference arm (which needs a GPU for a number)."""
    env = dict(os.environ)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--model", "resnet20",
                        "--steps", "3"], capture_output=True, text=True, timeout=300, env=env, cwd=str(tmp_path))
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["impl"] == "reference"
    if not torch.cuda.is_available():
        assert "CUDA" in out.get("error", "")
