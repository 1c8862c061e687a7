#!/bin/bash
# Builds the C-ABI shared library for sm_100a next to the Python package (see Makefile).
# DN_OUT=<path> writes the library elsewhere; DN_EXTRA_FLAGS / DN_PTXAS_V=1 are passed to nvcc
# (a different flag set needs its own object directory: DN_OBJDIR=<dir>).
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
make -C "$HERE" -j"$(nproc)" ${DN_OUT:+OUT="$DN_OUT"} ${DN_OBJDIR:+OBJDIR="$DN_OBJDIR"}
