#!/bin/bash
# CI entry points (reference: ci_build {build,ut,model}; ci/test_case).
#   ci/run_ci.sh build   compile every CUDA / C++ source in-tree for sm_100a
#   ci/run_ci.sh ut      native unit tests of the C++ runtime under ASan + UBSan, CPU unit tests; on a GPU box also the
#                        kernel tests
#   ci/run_ci.sh model   the model x dtype x kv-dtype smoke matrix of ci/test_case with fake weights (architectures
#                        from examples/model_config) through benchmarks/benchmark.py, collecting a latency CSV
#   ci/run_ci.sh cpp     the same matrix through the C++ engine (examples/cpp/example.cpp) and a two-rank tensor-parallel
#                        self-check (examples/cpp/tp_check.cpp), with fake weights
set -e
cd "$(dirname "$0")/.."
case "${1:-ut}" in
  build) python csrc/build.py --force ;;
  ut)
    "$(python csrc/build.py --selftest)" "$(mktemp -d)"
    python -m pytest tests -x -q -m "not gpu"
    if python -c "import torch,sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then python -m pytest tests -x -q -m gpu; fi ;;
  model)
    out=${2:-ci_model.csv}; rm -f "$out"
    grep -v '^#' ci/test_case | while read -r model dt kv bs inp outp; do
      [ -n "$model" ] || continue
      echo "== $model $dt kv=$kv bs=$bs in=$inp out=$outp"
      python benchmarks/benchmark.py --model_name "$model" -d "$dt" -kvd "$kv" -bs "$bs" -in "$inp" -out "$outp" -i 1 -w 0 --fake 2 --csv "$out"
    done
    echo "results in $out" ;;
  cpp)
    # the same matrix through the C++ engine (xft_example with fake weights), plus a tensor-parallel self-check
    grep -v '^#' ci/test_case | while read -r model dt kv bs inp outp; do
      [ -n "$model" ] || continue
      echo "== C++ $model $dt kv=$kv bs=$bs in=$inp out=$outp"
      XFT_FAKE_MODEL=2 xfastertransformer_b200/lib/xft_example -m "examples/model_config/$model" -d "$dt" \
        --kv_cache_dtype "$kv" -b "$bs" -l "$inp" -o "$outp" --no_stream | tail -1
    done
    XFT_FAKE_MODEL=2 xfastertransformer_b200/lib/xft_tp_check -m examples/model_config/llama-2-7b -n 2 -o 2
    # ... and as two pipeline stages of two tensor-parallel ranks
    XFT_FAKE_MODEL=2 xfastertransformer_b200/lib/xft_tp_check -m examples/model_config/llama-2-7b -n 4 -s 2 -o 2 ;;
  *) echo "usage: $0 {build|ut|model|cpp}"; exit 2 ;;
esac
