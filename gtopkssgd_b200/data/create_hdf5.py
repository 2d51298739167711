"""Convert an ImageNet folder tree into the single HDF5 file that
``DatasetHDF5`` reads (reference: scripts/create_hdf5.py, scripts/test_read_hdf5.py).

    python -m gtopkssgd_b200.data.create_hdf5 --root /data/imagenet --out imagenet-shuffled.hdf5
    python -m gtopkssgd_b200.data.create_hdf5 --inspect imagenet-shuffled.hdf5 [--save-sample sample.png]

Layout written: ``train_img`` / ``val_img`` uint8 [N, 224, 224, 3] (shorter
side resized to 256, centre crop 224, training set shuffled once) and
``train_labels`` / ``val_labels`` int16.  Class ids follow the sorted order of
the sub-directory names under ``train/``.  Needs h5py and Pillow.
"""
from __future__ import annotations

import argparse
import os
import random

import numpy as np

SIZE = 224


def list_images(split_dir, class_to_id):
    items = []
    for cls in sorted(os.listdir(split_dir)):
        d = os.path.join(split_dir, cls)
        if os.path.isdir(d) and cls in class_to_id:
            items += [(os.path.join(d, f), class_to_id[cls]) for f in sorted(os.listdir(d))
                      if f.lower().endswith((".jpeg", ".jpg", ".png"))]
    return items


def load_image(path):
    from PIL import Image
    img = Image.open(path).convert("RGB")
    w, h = img.size
    s = 256.0 / min(w, h)
    img = img.resize((max(SIZE, int(round(w * s))), max(SIZE, int(round(h * s)))), Image.BILINEAR)
    w, h = img.size
    left, top = (w - SIZE) // 2, (h - SIZE) // 2
    return np.asarray(img.crop((left, top, left + SIZE, top + SIZE)), dtype=np.uint8)


def convert(root, out, limit=None, seed=0):
    import h5py
    classes = sorted(d for d in os.listdir(os.path.join(root, "train")) if os.path.isdir(os.path.join(root, "train", d)))
    class_to_id = {c: i for i, c in enumerate(classes)}
    with h5py.File(out, "w", libver="latest") as hf:
        for split in ("train", "val"):
            items = list_images(os.path.join(root, split), class_to_id)
            if split == "train":
                random.Random(seed).shuffle(items)
            if limit:
                items = items[:limit]
            imgs = hf.create_dataset("%s_img" % split, (len(items), SIZE, SIZE, 3), dtype=np.uint8,
                                     chunks=(1, SIZE, SIZE, 3))
            hf.create_dataset("%s_labels" % split, data=np.array([y for _, y in items], dtype=np.int16))
            for i, (path, _) in enumerate(items):
                imgs[i] = load_image(path)
                if i % 10000 == 0:
                    print("%s: %d / %d" % (split, i, len(items)), flush=True)
    return out


def inspect(path, save_sample=None, index=0):
    import h5py
    with h5py.File(path, "r") as hf:
        for key in hf:
            print(key, hf[key].shape, hf[key].dtype)
        if save_sample:
            from PIL import Image
            Image.fromarray(hf["train_img"][index]).save(save_sample)
            print("label:", int(hf["train_labels"][index]), "->", save_sample)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--root", type=str, help="folder with train/<class>/*.JPEG and val/<class>/*.JPEG")
    ap.add_argument("--out", type=str, default="imagenet-shuffled.hdf5")
    ap.add_argument("--limit", type=int, default=None, help="images per split (for a quick sample file)")
    ap.add_argument("--inspect", type=str, default=None)
    ap.add_argument("--save-sample", type=str, default=None)
    args = ap.parse_args(argv)
    if args.inspect:
        inspect(args.inspect, args.save_sample)
    else:
        convert(args.root, args.out, args.limit)


if __name__ == "__main__":
    main()
