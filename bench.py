#!/usr/bin/env python3
"""Benchmark entry: ``python bench.py --gpus 1 --steps K --warmup W``.

Prints one JSON line (see freetoken_b200/benchmark.py for the method).  The
engine is single-GPU: for ``--gpus N`` with N > 1 it says so and exits with 2.
``--impl reference`` reports that the reference cannot be installed here.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from freetoken_b200.benchmark import main  # noqa: E402

if __name__ == "__main__":
    raise SystemExit(main())
