#!/usr/bin/env bash
# Build everything in-tree for sm_100a and run the host-only checks.
#   examples/build.sh            library, plugins, drop-in NCCL library, config checker, host test runner
#   examples/build.sh --torch    also the torch.distributed backend
# Role of the reference's examples/build_scripts/build.sh:1-45 (make of the library, the plugins and the perf programs).
set -euo pipefail
here=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
root=$(cd "$here/.." && pwd)
cd "$root"
python -m coccl_b200._build "$@"
"$root/coccl_b200/lib/coccl_host_tests"
for policy in "$root"/coccl_b200/configs/*.toml; do
  "$root/coccl_b200/lib/coccl-config-check" "$policy" >/dev/null
  echo "policy ok: ${policy#$root/}"
done
