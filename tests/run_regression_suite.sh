#!/usr/bin/env bash
# The regression ladder in one command, cheapest tier first; stops at the first failing tier.
#
#   tests/run_regression_suite.sh            # build + CPU tiers (no GPU needed)
#   tests/run_regression_suite.sh --gpu      # then the GPU tiers and the gated generation smokes on cuda:0
#   tests/run_regression_suite.sh --gpu --model /path/to/checkpoint --min-steady-decode-tps 50
#
# Tiers: (1) native build for sm_100a, (2) source-tree guards, (3) control plane and runtime contracts,
# (4) everything else that runs on the CPU, including the gloo multi-rank tests, (5) GPU kernels against their
# fp32 oracles and the model families on the GPU, (6) generation smoke with gates, (7) bench.py with its
# default, short configuration.  Same role as tests/run_regression_suite.sh and
# tests/run_inference_correctness_regression.sh of the reference.
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")/.."

GPU=0
MODEL="synthetic:tiny-llama-test"
GATE="0"
while [ $# -gt 0 ]; do
  case "$1" in
    --gpu) GPU=1 ;;
    --model) MODEL="$2"; shift ;;
    --min-steady-decode-tps) GATE="$2"; shift ;;
    -h|--help) sed -n 2,14p "$0"; exit 0 ;;
    *) echo "unknown argument: $1" >&2; exit 2 ;;
  esac
  shift
done

step() { echo; echo "== $* =="; }

step "1/7 native build"
python -c "import __graft_entry__ as g; g.build()"
step "2/7 source-tree guards"
python -m pytest tests/test_repo_hygiene.py -q
step "3/7 control plane and runtime contracts"
python -m pytest tests/test_control_plane.py tests/test_runtime_contracts.py tests/test_api_and_config.py -q -m "not gpu"
step "4/7 remaining CPU tests (multi-rank tests use gloo on 127.0.0.1)"
python -m pytest tests -q -m "not gpu" --deselect tests/test_repo_hygiene.py --deselect tests/test_control_plane.py \
  --deselect tests/test_runtime_contracts.py --deselect tests/test_api_and_config.py
if [ "$GPU" -eq 0 ]; then
  echo; echo "CPU tiers passed (run with --gpu for tiers 5 to 7)"; exit 0
fi
step "5/7 GPU tests"
python -m pytest tests -q -m gpu
step "6/7 generation smoke with gates ($MODEL)"
python -m litevllm_b200.diagnostics.smoke --model "$MODEL" --device cuda --prompt-length 64 --max-tokens 32 \
  --repeat 3 --min-steady-decode-tps "$GATE"
step "7/7 bench.py (default configuration)"
python bench.py
echo; echo "all tiers passed"
