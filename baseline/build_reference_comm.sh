#!/bin/bash
# Builds the reference's intranode communication extension (stream_ep_cpp: csrc/stream_ep.cpp,
# csrc/kernels/runtime.cu, csrc/kernels/intranode.cu) UNMODIFIED for sm_100 into baseline/_ref, with the
# reference's own -DDISABLE_NVSHMEM switch (its setup.py turns the internode sources off when the
# nvidia.nvshmem module cannot be imported; here the module is hidden behind an empty `nvidia` package
# because its internode.cu needs <infiniband/mlx5dv.h>, which this image does not have).
# Usage: baseline/build_reference_comm.sh /path/to/reference     (no GPU needed)
set -euo pipefail
REF=${1:?usage: build_reference_comm.sh /path/to/reference}
HERE=$(cd "$(dirname "$0")" && pwd)
WORK=$(mktemp -d /tmp/streamep_ref_build.XXXXXX)
cp -r "$REF"/. "$WORK"/src
mkdir -p "$WORK/shim/nvidia" && : > "$WORK/shim/nvidia/__init__.py"
cd "$WORK/src"
# The stock build passes -rdc=true to nvcc but, with NVSHMEM off, its setup.py has no device-link step: the shared
# object it produces is left with unresolved __cudaRegisterLinkedBinary_* symbols and cannot be imported.  (The
# reference's other switch, DISABLE_SM90_FEATURES=1, avoids -rdc but does not compile: intranode.cu(595) and 70 more
# errors.)  So the objects of the stock build are device-linked here and the library is linked again; the sources and
# their compile flags stay exactly the reference's.
export TORCH_CUDA_ARCH_LIST=10.0 DISABLE_AGGRESSIVE_PTX_INSTRS=1 MAX_JOBS=${MAX_JOBS:-8}
export CXX=/usr/bin/g++ CC=/usr/bin/gcc
PYTHONPATH="$WORK/shim${PYTHONPATH:+:$PYTHONPATH}" python setup.py build_ext --build-lib "$HERE/_ref" 2>&1 | grep -v "warning #\|^ *\^\|^$\|Remark\|declared but never" | tail -60
OBJ=$(find "$WORK/src/build" -name "*.o" | sort)
SO=$(ls "$HERE"/_ref/stream_ep_cpp*.so)
TORCH_LIB=$(python -c "import torch, os; print(os.path.join(os.path.dirname(torch.__file__), 'lib'))")
nvcc -dlink -gencode=arch=compute_100,code=sm_100 $(echo "$OBJ" | grep -v stream_ep.o) -o "$WORK/dlink.o" --compiler-options -fPIC
/usr/bin/g++ -shared $OBJ "$WORK/dlink.o" -L"$TORCH_LIB" -L/usr/local/cuda/lib64 -L/usr/local/cuda/lib64/stubs -lc10 -ltorch -ltorch_cpu \
    -ltorch_python -lcudart -lcudadevrt -lc10_cuda -ltorch_cuda -lcuda -o "$SO"
cp -r "$WORK/src/stream_ep" "$WORK/src/tests" "$HERE/_ref/" 2>/dev/null || true
ls -la "$HERE/_ref"
