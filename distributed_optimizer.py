"""Same import name as the reference module: ``import distributed_optimizer as dopt``."""
from gtopkssgd_b200.parallel.distributed_optimizer import (DistributedOptimizer, _DistributedOptimizer,  # noqa: F401
                                                            rank, size)
