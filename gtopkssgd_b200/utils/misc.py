"""Helpers with the names of the reference's utils.py:7-39 (Python 3)."""
from __future__ import annotations

import hashlib
import os
import time
from typing import Dict, List, Tuple

import numpy as np


def gen_random_id() -> str:
    return hashlib.sha256(("%r-%d" % (time.time(), os.getpid())).encode()).hexdigest()


def create_path(relative_path: str, base: str | None = None) -> str:
    """mkdir -p; relative paths are taken from the working directory."""
    path = relative_path if os.path.isabs(relative_path) else os.path.join(base or os.getcwd(), relative_path)
    os.makedirs(path, exist_ok=True)
    return path


def topk(tensor: np.ndarray, k: int) -> Tuple[np.ndarray, np.ndarray]:
    """Indices and values of the k largest magnitudes, ascending by magnitude."""
    order = np.argpartition(np.abs(tensor), -k)[-k:]
    order = order[np.argsort(np.abs(tensor[order]), kind="stable")]
    return order, tensor[order]


def force_insert_item(d: Dict[str, List], key: str, val) -> None:
    d.setdefault(key, []).append(val)


def update_fontsize(ax, fontsize: float = 12.0) -> None:
    items = [ax.title, ax.xaxis.label, ax.yaxis.label] + ax.get_xticklabels() + ax.get_yticklabels()
    for item in items:
        item.set_fontsize(fontsize)


def autolabel(rects, ax, label, rotation: int = 90) -> None:
    for rect in rects:
        top = rect.get_y() + rect.get_height()
        ax.text(rect.get_x() + rect.get_width() / 2.0, 1.03 * top, label, ha="center", va="bottom", rotation=rotation)
