#!/bin/bash
# Slice-count sweep of the transformer-block benchmark (counterpart of runksplittune.sh).
# usage: bench/runksplittune.sh NROW NCOL
NROW=${1:-2}; NCOL=${2:-4}; N=$((NROW*NCOL))
for k in 1 2 4 8; do
  python -m torch.distributed.run --nnodes=1 --nproc-per-node $N --master-addr 127.0.0.1 --master-port 29601 \
    bench/BenchTransformer.py --alg meshflow --nrows $NROW --ncols $NCOL --nheads 32 --batchsize 32 --ksplit $k $k $k $k
done
