"""Run-wide switches and the shared logger.

Mirrors the module constants of the reference's settings.py:6-35 (same names,
same default PREFIX string, same log line format) so that log directories and
log parsers written for the reference keep working.  Every switch can also be
set through an environment variable ``GTOPK_<NAME>``.
"""
from __future__ import annotations

import logging
import os
import socket


def _env_flag(name: str, default: bool) -> bool:
    raw = os.environ.get("GTOPK_" + name)
    if raw is None:
        return default
    return raw.strip().lower() not in ("0", "false", "no", "")


DEBUG = _env_flag("DEBUG", False)
SPARSE = _env_flag("SPARSE", False)
WARMUP = _env_flag("WARMUP", True)
DELAY_COMM = int(os.environ.get("GTOPK_DELAY_COMM", "1"))
TENSORBOARD = _env_flag("TENSORBOARD", True)
PROFILING_NORM = _env_flag("PROFILING_NORM", False)
# Pin the density to --density from epoch 0 on (the reference uses 0.004 in
# epoch 0 whatever --density says, allreducer.py:226-230).
PIN_DENSITY = _env_flag("PIN_DENSITY", False)
# Merge threshold in elements; a group closes once it holds this many
# (allreducer.py:26: 640 Mi elements, i.e. the whole model is one group).
THRESHOLD = int(os.environ.get("GTOPK_THRESHOLD", str(640 * 1024 * 1024)))
# NVTX ranges around every phase of the gradient path (select, exchange,
# update) and around each training step, for timeline tools.
NVTX = _env_flag("NVTX", False)
# Limit of every device-side wait, in milliseconds.
WAIT_LIMIT_MS = float(os.environ.get("GTOPK_WAIT_LIMIT_MS", "20000"))

# How CUDA ranks exchange their sparse sets: "p2p" = peer stores over NVLink inside the exchange
# kernels (all ranks on one host with peer access), "staged" = device -> host -> gloo -> device (ranks on
# several hosts, or no peer access), "auto" = p2p where possible.
TRANSPORT = os.environ.get("GTOPK_TRANSPORT", "auto").lower()
# Host watchdog on the device work of an iteration, multi-GPU runs only: seconds
# after which a still-running iteration is reported (0 = twice the device wait
# limit plus 30 s; negative = no watchdog).
WATCHDOG_S = float(os.environ.get("GTOPK_WATCHDOG_S", "0"))

PREFIX = ("compression" if SPARSE else "baseline") + ("-gwarmup" if WARMUP else "")
PREFIX += "-dc%d" % DELAY_COMM + "-model-ijcai2019"

hostname = socket.gethostname()
logger = logging.getLogger(hostname)
logger.setLevel(logging.DEBUG if DEBUG else logging.INFO)
formatter = logging.Formatter("%(asctime)s [%(filename)s:%(lineno)d] %(levelname)s %(message)s")
if not logger.handlers:
    _h = logging.StreamHandler()
    _h.setFormatter(formatter)
    logger.addHandler(_h)
logger.propagate = False


def add_file_handler(path: str) -> logging.Handler:
    """Per-rank log file in the same line format."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    h = logging.FileHandler(path)
    h.setFormatter(formatter)
    logger.addHandler(h)
    return h
