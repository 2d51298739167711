"""Child of tests/test_reference_arm_cpu.py: one rank that calls the reference's own
``gtopk_sparse_allreduce`` / ``topk_sparse_allreduce`` over the mpi4py stand-in and
saves what it got.  Run under torchrun; argv: out_dir d k."""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") not in (ROOT, HERE)]
sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))

import numpy as np  # noqa: E402

if not hasattr(np, "int"):
    np.int = int
import torch  # noqa: E402
from mpi4py import MPI  # noqa: E402

import allreducer as ref_ar  # noqa: E402

out_dir, d, k = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
comm = MPI.COMM_WORLD
rank, world = comm.rank, comm.size
assert os.path.abspath(ref_ar.__file__).startswith(os.path.join(ROOT, "baseline", "_ref"))
g = torch.Generator().manual_seed(77 + rank)
dense = torch.randn(d, generator=g)
# ranks share part of their support so that shared indices get summed
idx = torch.topk(dense.abs(), k).indices.numpy().astype(np.int64)
val = dense.numpy()[idx].astype(np.float32)
np.save(os.path.join(out_dir, "in_idx_%d.npy" % rank), idx)
np.save(os.path.join(out_dir, "in_val_%d.npy" % rank), val.copy())
storage = {}
for rep in range(2):  # twice: the second call reuses the cached receive buffer
    values, indexes, included = ref_ar.gtopk_sparse_allreduce(comm, val.copy(), storage=storage, indexes=idx.copy())
np.save(os.path.join(out_dir, "g_idx_%d.npy" % rank), np.asarray(indexes).astype(np.int64))
np.save(os.path.join(out_dir, "g_val_%d.npy" % rank), np.asarray(values).astype(np.float32))
np.save(os.path.join(out_dir, "g_inc_%d.npy" % rank), np.asarray(included).astype(np.int64))
tv, ti, _ = ref_ar.topk_sparse_allreduce(comm, val.copy(), {}, indexes=idx.astype(np.uint32))
np.save(os.path.join(out_dir, "t_idx_%d.npy" % rank), np.asarray(ti).astype(np.int64))
np.save(os.path.join(out_dir, "t_val_%d.npy" % rank), np.asarray(tv).astype(np.float32))
dense_sum = ref_ar.dense_allreduce(comm, np.full(8, float(rank + 1), dtype=np.float32))
assert np.allclose(dense_sum, world * (world + 1) / 2), dense_sum
assert comm.bcast(rank * 10 + 3) == 3
comm.Barrier()
MPI.Finalize()
