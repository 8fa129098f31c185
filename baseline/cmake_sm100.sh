#!/usr/bin/env bash
# cmake front end for the reference's dietGPU plugin build (dietgpu/Makefile:20-30 of the reference):
# the plugin Makefile hard-codes COCCL_CUDA_ARCHITECTURES=80 and its vendored glog asks for a CMake
# policy level that current CMake releases refuse. This wrapper changes the two arguments on the
# command line and leaves the reference's sources as they are.
args=()
configure=0
for a in "$@"; do
  case "$a" in
    -DCOCCL_CUDA_ARCHITECTURES=*) args+=("-DCOCCL_CUDA_ARCHITECTURES=${COCCL_REF_CUDA_ARCH:-100}"); configure=1 ;;
    *) args+=("$a") ;;
  esac
done
if [[ $configure == 1 ]]; then args+=("-DCMAKE_POLICY_VERSION_MINIMUM=3.5"); fi
exec cmake "${args[@]}"
