#!/bin/bash
# Builds the optional XLA FFI shim (dn_ffi.cc) next to the Python package, where jaxlib is installed.
# Exits 0 without building anything when `import jax.ffi` fails: the C-ABI library does not need it.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
PY="${PYTHON:-python}"
INC="$("$PY" -c 'import jax.ffi; print(jax.ffi.include_dir())' 2>/dev/null)" || { echo "jax.ffi not importable: XLA FFI shim not built"; exit 0; }
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
"$NVCC" -std=c++17 -O2 -Xcompiler -fPIC -shared -I"$INC" "$HERE/dn_ffi.cc" \
  -L"$HERE/../deltanet_b200" -ldeltanet_b200 -Xlinker -rpath -Xlinker '$ORIGIN' \
  -o "$HERE/../deltanet_b200/libdeltanet_b200_ffi.so"
echo "built $HERE/../deltanet_b200/libdeltanet_b200_ffi.so"
