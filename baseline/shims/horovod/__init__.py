"""Stand-in for the ``horovod`` package (absent from this image); see ``horovod.torch``."""
__version__ = "0.0-torchdist"
