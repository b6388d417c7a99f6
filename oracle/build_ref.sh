#!/bin/bash
# Builds the reference's own CUDA extension (module name flash_moba_cuda) for sm_100 from its
# sources WHERE THEY LIE in a reference checkout, trimmed to the translation units that the bf16
# causal configurations of head dims 64, 128 and 256 use; nothing of the reference is copied.  Test
# infrastructure: the result (oracle/_ref/flash_moba_cuda.so, git-ignored) is only loaded by
# oracle/ref_cuda.py for parity checks and for timing the reference's kernels beside this
# library's.  The other instantiations that the reference's dispatch names stay undefined; the
# loader opens the module with lazy binding, so they are only missed if called.
#
#   bash oracle/build_ref.sh /path/to/reference [jobs]
#
# Objects are kept in oracle/_ref/obj/ (git-ignored, and left out of GPU-box snapshots) so that a
# rerun only compiles what is missing.
# Needs nvcc, the PyTorch headers of the running interpreter and a CUTLASS 3.x / 4.x header tree
# (the reference's csrc/cutlass submodule; when that is empty, the tree that ships inside the
# flashinfer package is used).
set -e
REF=${1:?usage: build_ref.sh /path/to/reference [jobs]}
JOBS=${2:-8}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$HERE/_ref
mkdir -p "$OUT/obj"
PY=${PYTHON:-python}
TORCH_INC=$($PY -c "from torch.utils import cpp_extension as c; print(' '.join('-I'+p for p in c.include_paths()))" 2>/dev/null)
TORCH_LIB=$($PY -c "import torch, os; print(os.path.join(os.path.dirname(torch.__file__), 'lib'))")
PY_INC=$($PY -c "import sysconfig; print(sysconfig.get_paths()['include'])")
ABI=$($PY -c "import torch; print(int(torch._C._GLIBCXX_USE_CXX11_ABI))")
CUTLASS=$REF/csrc/cutlass/include
if [ ! -d "$CUTLASS/cute" ]; then
  CUTLASS=$($PY -c "import flashinfer, os; print(os.path.join(os.path.dirname(flashinfer.__file__), 'data/cutlass/include'))")
fi
INC="-I$REF/csrc/flash_moba -I$REF/csrc/flash_moba/src -I$REF/csrc/flash_topk -I$REF/csrc/flash_topk/src -I$CUTLASS $TORCH_INC -I$PY_INC"
DEFS="-DTORCH_EXTENSION_NAME=flash_moba_cuda -DTORCH_API_INCLUDE_EXTENSION_H -D_GLIBCXX_USE_CXX11_ABI=$ABI"
NVCC_FLAGS="-O3 -std=c++17 -U__CUDA_NO_HALF_OPERATORS__ -U__CUDA_NO_HALF_CONVERSIONS__ -U__CUDA_NO_HALF2_OPERATORS__ -U__CUDA_NO_BFLOAT16_CONVERSIONS__ --expt-relaxed-constexpr --expt-extended-lambda --use_fast_math -gencode arch=compute_100,code=sm_100 -Xcompiler -fPIC"
SRCS="
csrc/flash_moba_binding.cpp
csrc/flash_moba/flash_moba_api.cpp
csrc/flash_topk/flash_topk_api.cpp
csrc/flash_topk/src/varlen_sort.cu
csrc/flash_moba/src/flash_moba_fwd_hdim128_bf16_causal_sm80.cu
csrc/flash_moba/src/flash_moba_bwd_hdim128_bf16_causal_sm80.cu
csrc/flash_topk/src/flash_topk16_hdim128_bf16_causal_sm80.cu
csrc/flash_moba/src/flash_moba_fwd_hdim64_bf16_causal_sm80.cu
csrc/flash_moba/src/flash_moba_bwd_hdim64_bf16_causal_sm80.cu
csrc/flash_topk/src/flash_topk16_hdim64_bf16_causal_sm80.cu
csrc/flash_moba/src/flash_moba_fwd_hdim256_bf16_causal_sm80.cu
csrc/flash_moba/src/flash_moba_bwd_hdim256_bf16_causal_sm80.cu
csrc/flash_topk/src/flash_topk16_hdim256_bf16_causal_sm80.cu
"
compile_one() {
  src=$1
  obj=$OUT/obj/$(basename "${src%.*}").o
  if [ -f "$obj" ] && [ "$obj" -nt "$REF/$src" ]; then echo "$(date +%T) $src up to date"; return; fi
  if [ "${src##*.}" = "cu" ]; then
    nvcc $NVCC_FLAGS $DEFS $INC -c "$REF/$src" -o "$obj" > "$obj.log" 2>&1
  else
    g++ -O3 -std=c++17 -fPIC $DEFS $INC -I/usr/local/cuda/include -c "$REF/$src" -o "$obj" > "$obj.log" 2>&1
  fi
  echo "$(date +%T) $src rc=$?"
}
export -f compile_one
export OUT REF NVCC_FLAGS DEFS INC
echo $SRCS | tr ' ' '\n' | xargs -P "$JOBS" -I{} bash -c 'compile_one {}'
g++ -shared -o "$OUT/flash_moba_cuda.so" "$OUT"/obj/*.o -L"$TORCH_LIB" -ltorch -ltorch_cpu -ltorch_cuda -ltorch_python -lc10 -lc10_cuda \
    -L/usr/local/cuda/lib64 -lcudart -Wl,-rpath,"$TORCH_LIB"
echo "built $OUT/flash_moba_cuda.so"
