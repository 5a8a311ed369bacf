#!/bin/bash
# Runs the transformer-block benchmark for the four algorithms on one mesh shape of this box
# (counterpart of runexp.sh, which fans the same four runs out over a TPU pod).
# usage: bench/runexp.sh NROW NCOL
NROW=${1:-2}; NCOL=${2:-4}; N=$((NROW*NCOL))
for alg in collective wang meshflow summa; do
  python -m torch.distributed.run --nnodes=1 --nproc-per-node $N --master-addr 127.0.0.1 --master-port 29600 \
    bench/BenchTransformer.py --alg $alg --nrows $NROW --ncols $NCOL --nheads 32 --batchsize 32
done
