#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY -- never part of the shipped library.
#
# Compiles the UNMODIFIED reference (dingirsu/MXDSA) from the sources where they lie
# (location: MXDSA_REFERENCE_DIR, or a checkout named "reference" beside this repository) into
# oracle/_ref/mxdsa_ext.so.
# Nothing is copied: nvcc/c++ read the reference's csrc/ tree in place and only object files
# and the final .so are written under oracle/_ref/ (git-ignored).
#
# The reference has no CPU implementation of its kernels, so this .so is only useful on a
# Blackwell GPU: tests/golden/gen_golden.py runs it there to produce the golden vectors that
# pin the CPU oracle (oracle/mxdsa_oracle.py), and bench.py times it as the same-box GPU
# comparator.  The flags are the ones the reference's own build.sh uses (build.sh:50-56),
# restricted to the sm_100 family target that a B200 needs.
set -euo pipefail
here="$(cd "$(dirname "$0")" && pwd)"
ref="${MXDSA_REFERENCE_DIR:-$here/../../reference}"
out="$here/_ref"
if [[ ! -d "$ref/csrc" ]]; then
    echo "reference sources not found at $ref; keeping any prebuilt $out" >&2
    exit 0
fi
mkdir -p "$out"
CUDA_HOME="${CUDA_HOME:-/usr/local/cuda}"
PY="${PYTHON:-python}"
torch_root="$("$PY" -c 'import torch; print(torch.__path__[0])')"
py_inc="$("$PY" -c 'import sysconfig; print(sysconfig.get_path("include"))')"

nvflags=(-O3 -std=c++20 -DNDEBUG -D_USE_MATH_DEFINES -D_GLIBCXX_USE_CXX11_ABI=1
    --expt-relaxed-constexpr --expt-extended-lambda --use_fast_math --compiler-options=-fPIC
    -lineinfo --ptxas-options=--register-usage-level=10
    -gencode arch=compute_100f,code=sm_100f)
pids=()
for unit in attention/prefill attention/decode split_kv/scheduler split_kv/combine; do
    obj="$out/$(basename "$unit").o"
    if [[ ! -f "$obj" || "$ref/csrc/$unit.cu" -nt "$obj" ]]; then
        "$CUDA_HOME/bin/nvcc" -I"$ref/csrc" "${nvflags[@]}" -c "$ref/csrc/$unit.cu" -o "$obj" &
        pids+=($!)
    fi
done
if [[ ! -f "$out/binding.o" || "$ref/csrc/bindings/binding.cpp" -nt "$out/binding.o" ]]; then
    c++ -I"$ref/csrc" -I"$CUDA_HOME/include" -I"$torch_root/include" \
        -I"$torch_root/include/torch/csrc/api/include" -I"$py_inc" \
        -O2 -std=c++20 -DNDEBUG -D_GLIBCXX_USE_CXX11_ABI=1 -DTORCH_EXTENSION_NAME=mxdsa_ext \
        -fPIC -c "$ref/csrc/bindings/binding.cpp" -o "$out/binding.o" &
    pids+=($!)
fi
for p in "${pids[@]}"; do wait "$p"; done
c++ -shared "$out"/binding.o "$out"/prefill.o "$out"/decode.o "$out"/scheduler.o "$out"/combine.o \
    -L"$torch_root/lib" -Wl,-rpath,"$torch_root/lib" \
    -ltorch_python -ltorch_cuda -ltorch_cpu -ltorch -lc10_cuda -lc10 \
    -L"$CUDA_HOME/lib64" -Wl,-rpath,"$CUDA_HOME/lib64" -lcudart -lcuda \
    -o "$out/mxdsa_ext.so"
echo "built $out/mxdsa_ext.so"
