#!/bin/bash
# Collective sweeps for the baseline table: this library, stock NCCL and the reference build, same harness
# (coll_bench), only LD_PRELOAD and the PICCL_* variables change.
#   benchmarks/run_sweeps.sh N OUTDIR [quick|lean|focus]
# quick: fewer iterations and smaller maxima; lean: additionally every second size and a reduced set of variants
# (what fits a few minutes on 8 GPUs); focus: what AUTO and the in-switch path (NVLS) do for all five collectives against stock NCCL
# and the ring, nothing else.
# Writes OUTDIR/sweep_<N>.csv (all rows) .  Reference rows are only produced for configurations in which the
# reference is valid (fp32/int32, allreduce all algorithms, allgather RING/K_RING/PRD/PRM with k a power that
# fits, reduce RING, broadcast RING/K_RING in place); its stubs and unsafe configurations are not run.
N=${1:-2}; OUT=${2:-results}; QUICK=${3:-}
HERE="$(cd "$(dirname "$0")/.." && pwd)"; cd "$HERE"
CB=piccl_b200/lib/coll_bench; OURS=piccl_b200/lib/piccl.so; REF=baseline/_ref/piccl.so
mkdir -p "$OUT"; CSV="$OUT/sweep_$N.csv"; echo "# coll,label,dtype,op,ranks,bytes,iters,time_us,algbw_GBs,busbw_GBs,check" > "$CSV"
IS=1000; IL=100; [ -n "$QUICK" ] && { IS=200; IL=20; }
STEP=2; AR_MIN=8; LEAN=""; [ "$QUICK" = "lean" ] && { STEP=4; AR_MIN=16; LEAN=1; }
run() {  # label preload coll algo k dtype min max extra...
  local label=$1 pre=$2 coll=$3 algo=$4 k=$5 dt=$6 min=$7 max=$8; shift 8
  local up; up=$(echo "$coll" | tr a-z A-Z)
  local extra_env=(); while [ $# -gt 0 ] && [[ "$1" == [A-Z]*=* ]]; do extra_env+=("$1"); shift; done   # leading VAR=VALUE words: environment
  env "${extra_env[@]}" ${pre:+LD_PRELOAD=$pre} ${algo:+PICCL_${up}_ALGO=$algo} ${k:+PICCL_${up}_K=$k} timeout 300 $CB --gpus $N --coll $coll --dtype $dt --min $min --max $max \
      --check --label "$label" --iters-small $IS --iters-large $IL --step $STEP "$@" 2>/dev/null | grep -E "^(allreduce|allgather|reduce_scatter|reduce|broadcast)," >> "$CSV"
}
if [ "$QUICK" = "focus" ]; then
  IS=200; IL=20; STEP=4
  for dt in float bf16; do
    run nccl "" allreduce "" "" $dt 65536 1073741824
    run ours-AUTO-k-1 $OURS allreduce AUTO "" $dt 65536 1073741824
    run ours-NVLS-k-1 $OURS allreduce NVLS "" $dt 65536 1073741824
    run ours-RING-k-1 $OURS allreduce RING "" $dt 65536 1073741824
  done
  for coll in allgather reduce_scatter broadcast reduce; do
    run nccl "" $coll "" "" float 1024 268435456
    run ours-AUTO-k-1 $OURS $coll AUTO "" float 1024 268435456
    run ours-NVLS-k-1 $OURS $coll NVLS "" float 65536 268435456
    run ours-RING-k-1 $OURS $coll RING "" float 1024 268435456
  done
  echo "rows: $(wc -l < "$CSV")"; exit 0
fi
KS="2 4"; [ "$N" -ge 8 ] && KS="2 4 8"
AR_MAX=1073741824; BLK_MAX=268435456; [ "$QUICK" = "quick" ] && { AR_MAX=268435456; BLK_MAX=67108864; }
if [ -n "$LEAN" ]; then
  # ---- reduced set
  run nccl "" allreduce "" "" float $AR_MIN $AR_MAX
  for spec in "RING -" "PRD -" "PRM 2" "PRM $N" "K_RING 4" "DIRECT -"; do set -- $spec; k=$2; [ "$k" = "-" ] && k=""; run ours-$1-k${k:--1} $OURS allreduce $1 "$k" float $AR_MIN $AR_MAX; done
  if [ -f $REF ]; then run ref-RING $REF allreduce RING "" float $AR_MIN $AR_MAX; run ref-PRD $REF allreduce PRD "" float $AR_MIN $AR_MAX; run ref-PRM-k$N $REF allreduce PRM $N float $AR_MIN $AR_MAX; fi
  run nccl "" allreduce "" "" bf16 $AR_MIN $AR_MAX
  for spec in "RING -" "PRD -" "PRM $N" "DIRECT -"; do set -- $spec; k=$2; [ "$k" = "-" ] && k=""; run ours-$1-k${k:--1} $OURS allreduce $1 "$k" bf16 $AR_MIN $AR_MAX; done
  for coll in allgather reduce_scatter reduce broadcast; do
    run nccl "" $coll "" "" float 1024 $BLK_MAX
    run ours-RING-k-1 $OURS $coll RING "" float 1024 $BLK_MAX
    run ours-PRD-k-1 $OURS $coll PRD "" float 1024 $BLK_MAX
    run ours-PRM-k2 $OURS $coll PRM 2 float 1024 $BLK_MAX
    run ours-DIRECT-k-1 $OURS $coll DIRECT "" float 1024 $BLK_MAX
    run nccl "" $coll "" "" bf16 1024 $BLK_MAX
    run ours-RING-k-1 $OURS $coll RING "" bf16 1024 $BLK_MAX
  done
  if [ -f $REF ]; then
    run ref-RING $REF allgather RING "" float 1024 $BLK_MAX
    run ref-PRD $REF allgather PRD "" float 1024 $BLK_MAX
    run ref-RING $REF reduce RING "" float 1024 $BLK_MAX
    run ref-RING $REF broadcast RING "" float 1024 $BLK_MAX --in-place
  fi
  echo "rows: $(wc -l < "$CSV")"; exit 0
fi
# ---- allreduce, fp32 and bf16
for dt in float bf16; do
  run nccl "" allreduce "" "" $dt 8 $AR_MAX
  run ours-AUTO-k-1 $OURS allreduce AUTO "" $dt 8 $AR_MAX
  run ours-NVLS-k-1 $OURS allreduce NVLS "" $dt 8 $AR_MAX
  run ours-RING-k-1 $OURS allreduce RING "" $dt 8 $AR_MAX
  run ours-PRD-k-1 $OURS allreduce PRD "" $dt 8 $AR_MAX
  run ours-DIRECT-k-1 $OURS allreduce DIRECT "" $dt 8 $AR_MAX
  for k in $KS; do run ours-PRM-k$k $OURS allreduce PRM $k $dt 8 $AR_MAX; done
  for k in 2 4; do [ $((N % k)) -eq 0 ] && [ $k -lt $N ] && run ours-K_RING-k$k $OURS allreduce K_RING $k $dt 8 $AR_MAX; done
done
if [ -f $REF ]; then
  run ref-RING $REF allreduce RING "" float 8 $AR_MAX
  run ref-PRD $REF allreduce PRD "" float 8 $AR_MAX
  for k in $KS; do run ref-PRM-k$k $REF allreduce PRM $k float 8 $AR_MAX; done
  for k in 2 4; do [ $((N % k)) -eq 0 ] && [ $k -lt $N ] && run ref-K_RING-k$k $REF allreduce K_RING $k float 8 $AR_MAX; done
fi
# ---- the other collectives (per-rank block sizes)
for coll in allgather reduce_scatter reduce broadcast; do
  for dt in float bf16 int32; do
    run nccl "" $coll "" "" $dt 1024 $BLK_MAX
    run ours-AUTO-k-1 $OURS $coll AUTO "" $dt 1024 $BLK_MAX
    run ours-NVLS-k-1 $OURS $coll NVLS "" $dt 1024 $BLK_MAX
    run ours-RING-k-1 $OURS $coll RING "" $dt 1024 $BLK_MAX
    run ours-PRD-k-1 $OURS $coll PRD "" $dt 1024 $BLK_MAX
    run ours-PRM-k2 $OURS $coll PRM 2 $dt 1024 $BLK_MAX
    run ours-DIRECT-k-1 $OURS $coll DIRECT "" $dt 1024 $BLK_MAX
    [ $((N % 2)) -eq 0 ] && [ 2 -lt $N ] && run ours-K_RING-k2 $OURS $coll K_RING 2 $dt 1024 $BLK_MAX
  done
done
# reduce with max (root 0): fp32 takes the peer-to-peer schedules (the switch has no fp32 max), bf16 may go through the switch
for dt in float bf16 int32; do
  run nccl-max "" reduce "" "" $dt 1024 $BLK_MAX --op max
  run ours-AUTO-max $OURS reduce AUTO "" $dt 1024 $BLK_MAX --op max
  run ours-RING-max $OURS reduce RING "" $dt 1024 $BLK_MAX --op max
done
if [ -f $REF ]; then
  # only where the reference is valid: all-gather RING / K_RING / PRD / PRM with a radix that divides the rank count a whole number
  # of times, reduce RING, broadcast RING / K_RING in place; fp32 and int32 (it has no half types)
  for dt in float int32; do
    run ref-RING $REF allgather RING "" $dt 1024 $BLK_MAX
    run ref-PRD $REF allgather PRD "" $dt 1024 $BLK_MAX
    run ref-PRM-k2 $REF allgather PRM 2 $dt 1024 $BLK_MAX
    [ $((N % 2)) -eq 0 ] && [ 2 -lt $N ] && run ref-K_RING-k2 $REF allgather K_RING 2 $dt 1024 $BLK_MAX
    run ref-RING $REF reduce RING "" $dt 1024 $BLK_MAX
    run ref-RING-max $REF reduce RING "" $dt 1024 $BLK_MAX --op max
    run ref-RING $REF broadcast RING "" $dt 1024 $BLK_MAX --in-place
    [ $((N % 2)) -eq 0 ] && [ 2 -lt $N ] && run ref-K_RING-k2 $REF broadcast K_RING 2 $dt 1024 $BLK_MAX --in-place
  done
fi
echo "rows: $(wc -l < "$CSV")"
