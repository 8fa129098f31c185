#!/usr/bin/env bash
# Run an unmodified NCCL program (a C program, or PyTorch with its bundled NCCL) on the drop-in library.
#   examples/preload.sh [policy.toml] -- <command> [args...]
# The library exports the nccl* entry points, serves the calls the policy selects with its own compressed kernels and
# forwards everything else to the NCCL it finds (COCCL_NCCL_LIBRARY overrides the search). Role of the LD_PRELOAD lines of
# the reference's launcher (examples/training_scripts/train_qwen_coccl.sh:78-82).
set -euo pipefail
here=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
root=$(cd "$here/.." && pwd)
policy=$root/coccl_b200/configs/normal-sdp4bit.toml
if [[ "${1:-}" != "--" ]]; then policy=$1; shift; fi
[[ "${1:-}" == "--" ]] || { echo "usage: $0 [policy.toml] -- <command> [args...]" >&2; exit 2; }
shift
"$root/coccl_b200/lib/coccl-config-check" "$policy" >/dev/null
export COCCL_ENABLE=${COCCL_ENABLE:-1}
export COCCL_CONFIG_FILE=$policy
export LD_PRELOAD="$root/coccl_b200/lib/libcoccl_nccl.so${LD_PRELOAD:+:$LD_PRELOAD}"
exec "$@"
