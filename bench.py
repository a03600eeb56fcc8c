#!/usr/bin/env python3
"""Benchmark entry: ``python bench.py --gpus 1 --steps K --warmup W``.

Prints one JSON line (see freetoken_b200/benchmark.py for the method).  The
engine is single-GPU: for ``--gpus N`` with N > 1 it says so and exits with 2.
``--impl reference`` reports that the reference cannot be installed here.
``--design fazinex`` runs, instead of the default workload, the Fazinex decoder beside the
MiniMax-M3 decoder at equal size (freetoken_b200/design_bench.py); ``--design tonapel`` does the
same for the Tonapel decoder (freetoken_b200/tonapel_bench.py), ``--design nirelix`` runs the Nirelix
decoder beside the Tonapel decoder at equal size (freetoken_b200/nirelix_bench.py), ``--design mezapel``
the Mezapel decoder beside the MiniMax-M3 decoder at equal size (freetoken_b200/mezapel_bench.py).
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from freetoken_b200.benchmark import main  # noqa: E402

if __name__ == "__main__":
    raise SystemExit(main())
