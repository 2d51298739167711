"""Stand-in for ``h5py`` (absent from this image) so that the reference's
``datasets.py`` imports; opening a file is an error, the benchmark feeds
synthetic batches."""


class File:
    def __init__(self, *a, **k):
        raise RuntimeError("h5py is not installed in this image; the reference arm runs on synthetic batches only")
