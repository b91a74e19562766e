"""Command line: ``python -m dfccl_b200.simulator -f config.json``.

Same contract as the reference's ``python simulator.py -f cfg.json``
(simulator/simulator.py:724-752): ``num_process`` worker processes each run
``total_rounds`` rounds and the deadlock ratio over all of them is printed.
Workers get distinct seeds derived from the config seed so that more
processes mean more samples, not repeated ones.
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
from typing import Optional, Tuple

from .model import parse_config, run_rounds


def _worker(args) -> Tuple[int, int]:
    cfg, idx = args
    w = parse_config(cfg)
    seed = None if w.seed is None else w.seed + 7919 * idx
    return run_rounds(w, seed=seed)


def run_config(cfg: dict, processes: Optional[int] = None) -> Tuple[int, int]:
    """Run a config dict; returns ``(deadlocked_rounds, total_rounds)``."""
    n = processes if processes is not None else int(cfg.get("num_process", 1))
    if n <= 1:
        return _worker((cfg, 0))
    with mp.get_context("fork").Pool(n) as pool:
        parts = pool.map(_worker, [(cfg, i) for i in range(n)])
    return sum(p[0] for p in parts), sum(p[1] for p in parts)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Collective-issue-order deadlock simulator")
    ap.add_argument("-f", "--file", required=True, help="JSON config (see simulator/configs)")
    ap.add_argument("--processes", type=int, default=None)
    a = ap.parse_args(argv)
    with open(a.file) as fh:
        cfg = json.load(fh)
    bad, total = run_config(cfg, a.processes)
    print(f"#Deadlock round / rounds: {bad} / {total}, ratio: {bad / max(total, 1):.4f}")
    return 0
