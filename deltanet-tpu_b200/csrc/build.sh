#!/bin/bash
# Builds the C-ABI shared library for sm_100a next to the Python package.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/../deltanet_b200/libdeltanet_b200.so"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
"$NVCC" -std=c++17 -O3 -lineinfo -gencode arch=compute_100a,code=sm_100a \
  --expt-extended-lambda -Xcompiler -fPIC -shared ${DN_PTXAS_V:+-Xptxas -v} ${DN_EXTRA_FLAGS:-} \
  "$HERE"/dn_api.cu "$HERE"/dn_prepass_fwd.cu "$HERE"/dn_state.cu "$HERE"/dn_prepass_bwd.cu \
  "$HERE"/dn_decode.cu "$HERE"/dn_misc.cu "$HERE"/dn_umma_selftest.cu "$HERE"/dn_state_tc.cu "$HERE"/dn_prepass_fwd_tc.cu "$HERE"/dn_prepass_bwd_tc.cu "$HERE"/dn_noalloc.cu -o "${DN_OUT:-$OUT}"
echo "built ${DN_OUT:-$OUT}"
