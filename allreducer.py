"""Same import name as the reference module (AllReducer and the sparse / dense
all-reduce functions).  ``python allreducer.py`` runs the sparse all-reduce
micro-benchmark."""
from gtopkssgd_b200.parallel.allreducer import (MESSAGE, AllReducer, GTopkTimeout, SparseResult,  # noqa: F401
                                                 _default_err_callback)
from gtopkssgd_b200.parallel.compat import (THRESHOLD, benchmark_gtopk_sparse_allreduce, dense_allreduce,  # noqa: F401
                                             force_insert_item, gtopk_sparse_allreduce, topk, topk_sparse_allreduce)

if __name__ == "__main__":
    benchmark_gtopk_sparse_allreduce()
