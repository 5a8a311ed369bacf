#!/bin/sh
# Regression runs with recorded outputs (the counterpart of the reference's
# tests/testsuite_default_rdmaNic.py, which diffs simulator and per-node output against *.gold
# files).  The simulation is deterministic, so the outputs must match byte for byte.
#   run_gold.sh <netsim binary> [--update]
set -e
BIN=${1:?usage: run_gold.sh <netsim binary> [--update]}
HERE=$(cd "$(dirname "$0")" && pwd)
UPDATE=$2
fail=0
run() {
  name=$1; shift
  out=$("$BIN" "$@" 2>&1) || { echo "gold $name: netsim exited with an error"; echo "$out"; fail=1; return; }
  if [ "$UPDATE" = "--update" ]; then
    printf '%s\n' "$out" > "$HERE/gold/$name.gold"
  elif [ "$out" != "$(cat "$HERE/gold/$name.gold")" ]; then
    echo "gold $name: output differs from gold/$name.gold"
    printf '%s\n' "$out" | diff "$HERE/gold/$name.gold" - || true
    fail=1
  fi
}
C="$HERE/configs"
run msg_2nodes          --config "$C/sst_torus.ini" --scenario rdma-msg --nodes 2 --bytes 400
run imb_2nodes          --config "$C/sst_torus.ini" --scenario imb --nodes 2 --bytes 1 --repeat 10
run imb_4nodes_torus    --config "$C/sst_torus.ini" --scenario imb --nodes 4 --topology torus:2x2 --bytes 4096 --repeat 3
run incast_v2_8nodes    --config "$C/sst_torus.ini" --scenario rdma-incast-v2 --nodes 8 --topology torus:2x2x2 --bytes 3000
run write_hbm           --config "$C/sst_torus_hbm.ini" --scenario rdma-write --nodes 2 --bytes 100000
run sendrecv_nvswitch   --config "$C/b200_nvswitch.ini" --scenario rdma-sendrecv --bytes 1048576
run barrier_16nodes     --scenario barrier --nodes 16 --topology torus:4x4 --repeat 5
[ "$fail" = 0 ] && [ "$UPDATE" != "--update" ] && echo "netsim gold runs match"
exit $fail
