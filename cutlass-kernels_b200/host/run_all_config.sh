#!/usr/bin/bash
# Sweep of the FMHA driver over head sizes and precisions, shaped like the reference's
# src/fmha-pipeline/compile_run_all_config.sh:3-61 (batch 4, sequence 4096, dim 2048).  The reference
# recompiles for every tile-size / macro combination; here one library holds every kernel, so the sweep is
# over run-time arguments only.
#
#   run_all_config.sh            FLOP runs (1000 iterations each)
#   run_all_config.sh verify     a reference-checked run before every FLOP run
#   run_all_config.sh verify-all reference-checked runs only, with the score dump and the row statistics checked too
# Extra arguments after the mode are passed to every run (e.g. --causal=true).
HEADSIZES=( 64 128 256 )
PRECS=( 1 2 3 )          # 1 fp16, 2 e4m3, 3 bf16 (bf16 is an addition to the reference's list)
MODE=$1
shift
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
BIN="$HERE/../bin/fmha_forward"
if [[ ! -x "$BIN" ]]; then echo "build first: make -C $HERE/.."; exit 1; fi
STATUS=0
for PREC in "${PRECS[@]}"; do
for HEAD in "${HEADSIZES[@]}"; do
  if [[ $MODE == "verify" || $MODE == "verify-all" ]]; then
    VA=; if [[ $MODE == "verify-all" ]]; then VA="--verify-all=true"; fi
    "$BIN" --batch-size=4 --seq-length=4096 --dim-size=2048 --iterations=1 --head-size=$HEAD --reference-check=true $VA --prec-type=$PREC "$@" || STATUS=1
  fi
  if [[ $MODE != "verify-all" ]]; then
    echo "FLOP RUN BEGIN"
    echo "PREC=$PREC, HEAD=$HEAD"
    "$BIN" --batch-size=4 --seq-length=4096 --dim-size=2048 --iterations=1000 --head-size=$HEAD --reference-check=false --prec-type=$PREC "$@" || STATUS=1
    echo "FLOP RUN END"
  fi
done
done
exit $STATUS
