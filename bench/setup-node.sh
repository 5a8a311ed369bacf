#!/bin/sh
# Prepares one 8-GPU node for the benchmarks (the counterpart of the reference's setup-tpupod.sh,
# which installs jax[tpu] and copies the scripts to every pod worker): build the native extension
# in-tree for sm_100a, build the network simulator, run the CPU tests, show what the node has.
set -e
cd "$(dirname "$0")/.."
python -m meshslice_b200.build
make -C meshslice_b200/csrc/netsim netsim
python -m pytest tests -q -m "not gpu" -x
if command -v nvidia-smi >/dev/null 2>&1; then
  nvidia-smi --query-gpu=index,name,memory.total,clocks.max.sm --format=csv
  nvidia-smi topo -m || true
fi
