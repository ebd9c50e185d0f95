#!/usr/bin/env bash
# The sweeps of the benchmark configurations on N GPUs of one box:
#   bash bench/run_sweeps.sh N [OUT_DIR] [TUNING_FILE]
#   A. all-reduce, 1 KB - 1 GB, fp32 and bf16, every algorithm at its automatic channel count
#      (every configuration checked first: float64 host sum up to 16 MB, NCCL above);
#   B. all-reduce channel sweep (1 / 2 / 4 / 8 / 16 / 32 channels) at 256 KB, 16 MB and 512 MB;
#   C. all-gather and reduce-scatter, 1 KB - 1 GB, fp32 and bf16.
# SWEEP_QUICK=1 takes every fourth size (1 KB, 4 KB, ... 1 GB), 10 iterations and fp32 only for C: a third of the
# box time, for large worlds.
# Rows go to OUT_DIR/sweep_{N}gpu_{allreduce,channels,shards}.json; the winners of A and C are merged
# into TUNING_FILE (default: the table shipped with the package), which the selector reads.
# The reference's counterpart is tests/run_algo_comparison.sh + tests/bench_algo_comparison.py.
set -u
N=${1:?number of GPUs}
OUT=${2:-bench/results}
TUNING=${3:-pccl_b200/dsl/algorithms/tuning_b200.json}
HERE=$(cd "$(dirname "$0")/.." && pwd)
mkdir -p "$OUT"
RUN="python -m torch.distributed.run --nnodes=1 --nproc-per-node $N --master-addr 127.0.0.1"
export PCCL_VALIDATE=${PCCL_VALIDATE:-0}          # templates are validated by the test-suite; saves W compilations per plan
export PCCL_TUNING_FILE=/nonexistent              # "auto" rows must not follow an older table while a new one is measured
ALGOS=auto,ll,push,ring,rhd,tree,oneshot,twoshot,nvls,nvls_kernel,hybrid
SIZES=""; ITERS=20; SHARD_DTYPES=fp32,bf16
if [ "${SWEEP_QUICK:-0}" = "1" ]; then
  SIZES="--sizes 1K,4K,16K,64K,256K,1M,4M,16M,64M,256M,1G"; ITERS=10; SHARD_DTYPES=fp32
fi
$RUN --master-port 29601 "$HERE/bench/collective_sweep.py" --collectives allreduce --dtypes fp32,bf16 \
    --min-bytes 1K --max-bytes 1G $SIZES --algos $ALGOS --channels auto --iters $ITERS --check \
    --out "$OUT/sweep_${N}gpu_allreduce.json" --write-tuning "$TUNING" > "$OUT/sweep_${N}gpu_allreduce.log" 2>&1
$RUN --master-port 29602 "$HERE/bench/collective_sweep.py" --collectives allreduce --dtypes fp32 \
    --min-bytes 256K --max-bytes 512M --sizes 256K,16M,512M --algos ring,twoshot,nvls --channels 1,2,4,8,16,32 --iters 10 \
    --out "$OUT/sweep_${N}gpu_channels.json" > "$OUT/sweep_${N}gpu_channels.log" 2>&1
$RUN --master-port 29603 "$HERE/bench/collective_sweep.py" --collectives allgather,reduce_scatter --dtypes $SHARD_DTYPES \
    --min-bytes 1K --max-bytes 1G $SIZES --algos auto,ll,push,ring,twoshot,nvls --channels auto --iters $ITERS \
    --out "$OUT/sweep_${N}gpu_shards.json" --write-tuning "$TUNING" > "$OUT/sweep_${N}gpu_shards.log" 2>&1
grep -c '^{' "$OUT"/sweep_${N}gpu_*.log
