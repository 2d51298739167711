"""Markdown tables from benchmark output.

    python -m gtopkssgd_b200.analysis.bench_report --runs 1=out/n1 2=out/n2 4=out/n4 8=out/n8

Each ``N=DIR`` names a directory of JSON lines written by ``bench.py`` at N GPUs:
``ours_<model>.json`` and ``ref_<model>.json`` (``bench.py --impl reference``),
optionally ``refdense_<model>.json`` (``--impl reference --compressor none``),
``ours_eager_*``, ``oursdense_bucketed_*``, ``oursdense_onebucket_*``,
``ours_multigroup_*``; plus ``allreduce.json`` (``bench_allreduce --json``) and
``ref_allreduce.json`` (``baseline/ref_allreduce_bench.py --json``) for the
sparse all-reduce grid.  Prints the throughput table with the ratio of the two
arms, weak-scaling efficiencies, the like-for-like table and the
micro-benchmark tables.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict, List, Optional

MODELS = ("resnet50", "vgg16", "lstm", "resnet20")
VARIANTS = ("ours", "ours_eager", "oursdense_bucketed", "oursdense_onebucket", "ours_multigroup", "ref", "refdense")


def load_line(path: str) -> Optional[dict]:
    """Last JSON line of a bench output file, or None if there is no measurement in it."""
    try:
        with open(path) as fh:
            lines = [l for l in fh.read().splitlines() if l.strip().startswith("{")]
        j = json.loads(lines[-1])
        return j if "value" in j else None
    except (OSError, IndexError, ValueError):
        return None


class Runs:
    def __init__(self, dirs: Dict[int, List[str]]):
        self.dirs = dirs

    def get(self, n: int, name: str) -> Optional[dict]:
        for d in self.dirs.get(n, []):
            j = load_line(os.path.join(d, name + ".json"))
            if j:
                return j
        return None

    def file(self, n: int, name: str) -> Optional[str]:
        for d in self.dirs.get(n, []):
            p = os.path.join(d, name)
            if os.path.exists(p):
                return p
        return None


def _f(j, key, fmt="%.0f"):
    return (fmt % j[key]) if j else "—"


def _e2e(j):
    return ("%.0f" % j["e2e"]["value"]) if j and j.get("e2e") else "—"


def throughput_table(runs: Runs) -> str:
    out = ["| model | N | ours samples/s | ms/step | ours e2e | reference gTop-k samples/s | ms/step | reference e2e | "
           "ours ÷ reference (e2e) | reference dense | ours: select / exchange (of which wait) ms | "
           "reference: select / exchange ms |", "|" + "---|" * 12]
    for m in MODELS:
        for n in sorted(runs.dirs):
            o, r, rd = runs.get(n, "ours_" + m), runs.get(n, "ref_" + m), runs.get(n, "refdense_" + m)
            if not o and not r:
                continue
            ratio = "—"
            if o and r and o.get("e2e") and r.get("e2e"):
                ratio = "**%.2f×**" % (o["e2e"]["value"] / r["e2e"]["value"])
            co = (o or {}).get("comm_ms_per_iter") or {}
            cr = (r or {}).get("comm_ms_per_iter") or {}
            cs = "%.3f / %.3f (%.3f)" % (co.get("select_ms", 0), co.get("exchange_ms", 0),
                                         co.get("exchange_wait_ms", 0)) if co else "—"
            crs = "%.2f / %.2f" % (cr.get("select_ms", 0), cr.get("exchange_ms", 0)) if cr else "—"
            out.append("| %s | %d | %s | %s | %s | %s | %s | %s | %s | %s | %s | %s |" % (
                m, n, _f(o, "value"), _f(o, "ms_per_step", "%.2f"), _e2e(o), _f(r, "value"),
                _f(r, "ms_per_step", "%.2f"), _e2e(r), ratio, _f(rd, "value"), cs, crs))
    return "\n".join(out)


def efficiencies(runs: Runs) -> Dict[str, Dict[int, float]]:
    """{arm_model: {N: per-GPU throughput at N / at 1}} for every arm that has an N = 1 line."""
    out: Dict[str, Dict[int, float]] = {}
    for arm in ("ours", "ref"):
        for m in MODELS:
            base = runs.get(1, "%s_%s" % (arm, m)) if 1 in runs.dirs else None
            if not base:
                continue
            for n in sorted(runs.dirs):
                j = runs.get(n, "%s_%s" % (arm, m))
                if j and n > 1:
                    out.setdefault("%s_%s" % (arm, m), {})[n] = (j["value"] / n) / base["value"]
    return out


def like_for_like_table(runs: Runs) -> str:
    rows = []
    for n in sorted(runs.dirs, reverse=True):
        for m in MODELS:
            vals = [runs.get(n, "%s_%s" % (v, m)) for v in VARIANTS]
            if sum(v is not None for v in vals) < 3:
                continue
            rows.append("| %s | %d | " % (m, n) + " | ".join(
                ("%.0f (%.2f ms)" % (v["value"], v["ms_per_step"])) if v else "—" for v in vals) + " |")
    if not rows:
        return ""
    head = ["| model | N | gTop-k graph | gTop-k eager | dense NCCL eager, 8 M-element buckets | dense NCCL eager, "
            "one bucket | gTop-k graph, 8 M-element merge groups | reference gTop-k | reference dense |",
            "|" + "---|" * 9]
    return "\n".join(head + rows)


def micro_table(ours_json: str, ref_json: Optional[str]) -> str:
    with open(ours_json) as fh:
        rows = json.load(fh)["rows"]
    ref = {}
    if ref_json and os.path.exists(ref_json):
        with open(ref_json) as fh:
            ref = {(r["d"], r["rho"]): r for r in json.load(fh)["rows"]}
    out = ["| d | ρ | k | K1 | K2 isolated / steady | ours K1+K2 isolated / steady | dense NCCL isolated / steady | "
           "reference select + exchange | ours vs NCCL (steady) | ours vs reference | K2 steady ÷ NVLink wire time |",
           "|" + "---|" * 11]
    for r in rows:
        rr = ref.get((r["d"], r["rho"]))
        k2c = r.get("k2_chain_ms", r.get("k2_ms", 0.0))
        steady = r["k1_ms"] + k2c
        nccl = r.get("dense_nccl_chain_ms", r.get("dense_nccl_ms", 0.0))
        out.append("| %.1f M | %g | %d | %.3f | %.3f / %.3f | %.3f / %.3f | %.3f / %.3f | %s | %.2f× | %s | %.3f |" % (
            r["d"] / 1e6, r["rho"], r["k"], r["k1_ms"], r.get("k2_ms", 0.0), k2c, r["ours_ms"], steady,
            r.get("dense_nccl_ms", 0.0), nccl,
            ("%.2f + %.2f" % (rr["select_ms"], rr["exchange_ms"])) if rr else "—", nccl / steady if steady else 0.0,
            ("%.0f×" % (rr["total_ms"] / r["ours_ms"])) if rr else "—",
            (r.get("nvlink_roofline_ms", 0.0) / k2c) if k2c else 0.0))
    return "\n".join(out)


def report(runs: Runs) -> str:
    parts = [throughput_table(runs), ""]
    for name, d in efficiencies(runs).items():
        parts.append("%s weak-scaling efficiency: %s" % (name, ", ".join("%d: %.1f %%" % (n, 100 * v)
                                                                            for n, v in sorted(d.items()))))
    lfl = like_for_like_table(runs)
    if lfl:
        parts += ["", lfl]
    for n in sorted(runs.dirs):
        a = runs.file(n, "allreduce.json")
        if a:
            parts += ["", "**P = %d** (ms per call)" % n, "", micro_table(a, runs.file(n, "ref_allreduce.json"))]
    return "\n".join(parts) + "\n"


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--runs", nargs="+", required=True, metavar="N=DIR[,DIR...]",
                    help="directories of bench output per GPU count (first directory that has a file wins)")
    args = ap.parse_args(argv)
    dirs: Dict[int, List[str]] = {}
    for spec in args.runs:
        n, _, paths = spec.partition("=")
        dirs[int(n)] = [p for p in paths.split(",") if p]
    print(report(Runs(dirs)), end="")


if __name__ == "__main__":
    main()
