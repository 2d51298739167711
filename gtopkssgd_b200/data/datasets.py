"""ImageNet from one HDF5 file (reference: datasets.py:8-36): datasets
``train_img`` / ``val_img`` (uint8 N x 224 x 224 x 3) and ``train_labels`` /
``val_labels`` (int16), opened read-only in SWMR mode."""
from __future__ import annotations

import numpy as np
import torch


class DatasetHDF5(torch.utils.data.Dataset):
    def __init__(self, hdf5fn, t, transform=None, target_transform=None):
        try:
            import h5py
        except ImportError as exc:  # optional dependency
            raise ImportError("the ImageNet HDF5 reader needs h5py; use --data-dir synthetic otherwise") from exc
        self.hf = h5py.File(hdf5fn, "r", libver="latest", swmr=True)
        self.t = t
        self.d = self.hf["%s_img" % t]
        self.dlabel = self.hf["%s_labels" % t][...]
        self.n_images = self.d.shape[0]
        self.transform, self.target_transform = transform, target_transform

    def __len__(self):
        return self.n_images

    def __getitem__(self, index):
        img, target = self.d[index, ...], np.int64(self.dlabel[index])
        if self.transform is not None:
            img = self.transform(img)
        if self.target_transform is not None:
            target = self.target_transform(target)
        return img, target
