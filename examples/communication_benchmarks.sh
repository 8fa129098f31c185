#!/usr/bin/env bash
# Collective sweep on one node: every compressed collective of this library against native NCCL, per codec.
#   GPUS=8 examples/communication_benchmarks.sh            # writes sweep_<GPUS>gpu.json and prints the table
# Variables: GPUS (2), CODECS, MIN_MIB (1), MAX_MIB (1024), ITERS (30), WARMUP (20), THRESHOLD (0 = compress every size),
# AUTOTUNE (1: one-/two-shot and NCCL/multimem chosen from times measured at first use; 0: selector heuristics), OUT.
# Role of the reference's examples/benchmarks_scripts/communication_benchmarks.sh:17-132 (sizes doubling from 1 MB,
# 20 warm-up and 30 timed iterations, one policy per codec); the per-depth loop of that script has no counterpart
# because these collectives are single kernels, not a staged pipeline with a depth.
set -euo pipefail
here=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
root=$(cd "$here/.." && pwd)
gpus=${GPUS:-2}
codecs=${CODECS:-sdp4bit,sdp4bit_sr,mxfp8,taco,zfp8}
out=${OUT:-sweep_${gpus}gpu.json}
port=${MASTER_PORT:-29562}
extra=()
[[ "${AUTOTUNE:-1}" == 0 ]] && extra+=(--no-autotune)
cd "$root"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$gpus" --master-addr 127.0.0.1 --master-port "$port" \
  -m coccl_b200.bench_collectives --min-mib "${MIN_MIB:-1}" --max-mib "${MAX_MIB:-1024}" --codecs "$codecs" \
  --iters "${ITERS:-30}" --warmup "${WARMUP:-20}" --threshold "${THRESHOLD:-0}" --out "$out" "${extra[@]}"
python -m coccl_b200.bench_collectives --table "$out"
