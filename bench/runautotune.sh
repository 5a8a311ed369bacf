#!/bin/bash
# Autotunes GPT-3 (96 heads) and Megatron (160 heads) blocks for 8 GPUs (counterpart of
# runautotune.sh).  Pass a fabric file fitted by BenchCollectives2D as $1 to use measured constants.
F=${1:+--fabric-json $1}
python bench/run_autotune.py --nrows 2 --ncols 4 --batchsize 32 --nheads 96 --sweep $F > gpt3_8.log
python bench/run_autotune.py --nrows 2 --ncols 4 --batchsize 32 --nheads 160 --sweep $F > megatron_8.log
