#!/bin/bash
# CI entry points (reference: ci_build {build,ut,model}; ci/test_case).
#   ci/run_ci.sh build   compile every CUDA / C++ source in-tree for sm_100a
#   ci/run_ci.sh ut      CPU unit tests;  on a GPU box also the kernel tests
#   ci/run_ci.sh model   model x dtype x kv-dtype smoke matrix with fake weights (config.ini only) through
#                        benchmarks/benchmark.py, collecting a latency CSV like the reference's model tier
set -e
cd "$(dirname "$0")/.."
case "${1:-ut}" in
  build) python csrc/build.py --force ;;
  ut)
    python -m pytest tests -x -q -m "not gpu"
    if python -c "import torch,sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then python -m pytest tests -x -q -m gpu; fi ;;
  model)
    out=${2:-ci_model.csv}; rm -f "$out"; tmp=$(mktemp -d)
    for model in tiny-llama; do
      python - "$tmp/$model" "$model" <<'PY'
import sys
from xfastertransformer_b200.tools.synthetic import config_only, preset
config_only(sys.argv[1], preset(sys.argv[2]))
PY
      for dt in bf16 fp16 int8 w8a8 int4 nf4 bf16_int8 w8a8_nf4; do for kv in fp16 int8; do for inp in 32 2016; do
        python benchmarks/benchmark.py -m "$tmp/$model" -d $dt -kvd $kv -bs 1 -in $inp -out 32 -i 1 -w 0 --fake 2 --csv "$out"
      done; done; done
    done
    echo "results in $out" ;;
  *) echo "usage: $0 {build|ut|model}"; exit 2 ;;
esac
