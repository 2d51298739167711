"""Stand-in for the ``mpi4py`` package (absent from this image): only the
``MPI`` sub-module, with the subset of calls that the reference makes."""
from . import MPI  # noqa: F401

__version__ = "0.0-torchdist"
