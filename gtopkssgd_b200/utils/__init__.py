"""Small host-side helpers (paths, ids, numpy top-k, timers, clock sampling)."""
from .misc import create_path, gen_random_id, topk, force_insert_item, update_fontsize, autolabel  # noqa: F401
from .timing import CudaTimer, PhaseTimers  # noqa: F401
