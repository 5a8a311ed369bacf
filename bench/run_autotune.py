#!/usr/bin/env python
"""End-to-end autotuning on one box: fit the fabric (or read ``--fabric-json``), let the tuner
pick mesh shape, dataflow and slice count for a GPT block, optionally with measured GEMM times.
Counterpart of runautotune.sh, which runs Autotuner.py for GPT-3 (96 heads) and Megatron (160)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from meshslice_b200.autotuner import main

if __name__ == "__main__":
    main()
