#!/bin/sh
# Builds the pybind11 module sparseops_backend (host C++ above the C ABI), in-tree next to this
# script.  It links libspx_b200.so from its own directory ($ORIGIN).
set -e
cd "$(dirname "$0")"
CXX=${SPX_CXX:-g++}
PYINC=$(python3 -m pybind11 --includes)
EXT=$(python3-config --extension-suffix)
exec $CXX -std=c++17 -O2 -fPIC -shared -fvisibility=hidden -Wall -Wno-unused-function \
    -I../include -Icsrc/host $PYINC \
    -o sparseops_backend$EXT csrc/host/bindings.cpp csrc/host/ellpack.cpp csrc/host/onnx_reader.cpp \
    csrc/host/sparse_onnx.cpp csrc/host/rbm.cpp \
    -L. -lspx_b200 -Wl,-rpath,'$ORIGIN' -lpthread
