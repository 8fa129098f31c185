#!/usr/bin/env bash
# Builds the example codec into OUT (default: examples/plugin/out) and checks a policy file that uses it.
#   examples/plugin/build.sh [OUT]
# A plugin needs the SDK header tree only (coccl_b200/csrc/include); it does not link against the library.
set -euo pipefail
here=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
root=$(cd "$here/../.." && pwd)
out=${1:-$here/out}
mkdir -p "$out"
nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 -Xcompiler -fPIC -shared \
  -I"$root/coccl_b200/csrc/include" "$here/bf16cast_plugin.cu" -o "$out/libbf16cast.so"
sed "s|^library_path = .*|library_path = \"$out\"|" "$here/bf16cast.toml" > "$out/bf16cast.toml"
"$root/coccl_b200/lib/coccl-config-check" --nodes 1 --devices-per-node 8 "$out/bf16cast.toml"
echo "built $out/libbf16cast.so; run a program with COCCL_ENABLE=1 COCCL_CONFIG_FILE=$out/bf16cast.toml"
