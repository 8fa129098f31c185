#!/usr/bin/env bash
# 3-D parallel GPT pre-training with compressed collectives, one process per GPU.
#   examples/train_gpt.sh <model> [nnodes] [gpus-per-node] [node-rank]       e.g.  examples/train_gpt.sh gpt-6.7b 1 8 0
# <model>: gpt-2.7b | gpt-6.7b | gpt-13b | qwen2.5-7b | qwen3-8b | llama3-8b | qwen3-30b-a3b (with EP) | ... (python -m coccl_b200.pretrain -h);
# HF_MODEL=<directory> starts from a Hugging Face checkpoint of the Llama / Qwen family instead.
# Variables: TP (2), PP (2), EP (1), VIRTUAL_STAGES (1), GLOBAL_BATCH (0 = 8 sequences per data-parallel rank),
# MICRO_BATCH (2), STEPS (1000), LR (3e-4), DATA (flat token file; empty = synthetic ids), SAVE (checkpoint directory,
# resumed when it already holds one), SAVE_INTERVAL (500), MASTER_ADDR (127.0.0.1), MASTER_PORT (29500),
# COCCL_ENABLE (1; 0 = native NCCL everywhere), COCCL_CONFIG_FILE (default: the shipped training policy).
# Role of the reference's examples/training_scripts/train_qwen_coccl.sh:60-131, which exports the same two COCCL_*
# variables and starts an external Megatron trainer; here the trainer is coccl_b200.pretrain.
set -euo pipefail
model=${1:?usage: $0 <model> [nnodes] [gpus-per-node] [node-rank]}
nnodes=${2:-1}
gpus=${3:-8}
node_rank=${4:-0}
here=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
root=$(cd "$here/.." && pwd)
export COCCL_ENABLE=${COCCL_ENABLE:-1}
export COCCL_CONFIG_FILE=${COCCL_CONFIG_FILE:-$root/coccl_b200/configs/training.toml}
"$root/coccl_b200/lib/coccl-config-check" --nodes "$nnodes" --devices-per-node "$gpus" "$COCCL_CONFIG_FILE" >/dev/null
args=(--model "$model" --tp "${TP:-2}" --pp "${PP:-2}" --ep "${EP:-1}" --virtual-stages "${VIRTUAL_STAGES:-1}"
      --global-batch "${GLOBAL_BATCH:-0}" --micro-batch "${MICRO_BATCH:-2}" --steps "${STEPS:-1000}" --lr "${LR:-3e-4}"
      --log-interval "${LOG_INTERVAL:-10}")
[[ -n "${DATA:-}" ]] && args+=(--data "$DATA")
[[ -n "${HF_MODEL:-}" ]] && args+=(--hf-model "$HF_MODEL")
[[ -n "${SAVE:-}" ]] && args+=(--save "$SAVE" --save-interval "${SAVE_INTERVAL:-500}" --resume)
cd "$root"
exec python -m torch.distributed.run --nnodes "$nnodes" --nproc-per-node "$gpus" --node-rank "$node_rank" \
  --master-addr "${MASTER_ADDR:-127.0.0.1}" --master-port "${MASTER_PORT:-29500}" -m coccl_b200.pretrain "${args[@]}"
