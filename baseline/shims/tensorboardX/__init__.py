"""Stand-in for ``tensorboardX`` (absent from this image): ``SummaryWriter``
forwards to ``torch.utils.tensorboard`` when that imports, else swallows calls."""
try:
    from torch.utils.tensorboard import SummaryWriter  # noqa: F401
except Exception:  # pragma: no cover - tensorboard missing
    class SummaryWriter:
        def __init__(self, *a, **k):
            pass

        def __getattr__(self, name):
            return lambda *a, **k: None
