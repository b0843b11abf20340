#!/bin/sh
# Builds libspx_b200.so (CUDA kernels + C ABI) for sm_100a, in-tree next to this script.
# No fast-math: sigmoid/tanh must stay within a few ulp of the C library, and only explicit
# fmaf() calls may fuse (-fmad=false) so that accumulation chains match the reference bit for bit.
set -e
cd "$(dirname "$0")"
NVCC=${NVCC:-nvcc}
$NVCC -std=c++17 -O3 -lineinfo -gencode arch=compute_100a,code=sm_100a -fmad=false \
    -Xcompiler -fPIC -shared -I../include -Icsrc/cuda \
    ${SPX_PTXAS_V:+-Xptxas -v} \
    -o libspx_b200.so csrc/cuda/abi.cu csrc/cuda/comm.cu csrc/cuda/spmm.cu csrc/cuda/spmv.cu \
    csrc/cuda/conv.cu csrc/cuda/pool.cu csrc/cuda/eltwise.cu csrc/cuda/encode.cu -ldl
# bench equipment, not part of the product library: the L2 -> SM gather bandwidth probe bench.py loads
$NVCC -std=c++17 -O3 -lineinfo -gencode arch=compute_100a,code=sm_100a -Xcompiler -fPIC -shared \
    -o libspx_bench_probe.so csrc/bench/l2_gather_probe.cu
