#!/bin/bash
# The GPU suites once more with each non-default switch of the fused path, one process per switch so that one failure
# does not take the others with it. One GPU is enough; the last block needs 2 and is skipped otherwise.
#   bash tests/alt_paths_gpu.sh [log-directory]
cd "$(dirname "$0")/.." || exit 1
LOG=${1:-/tmp/ccfuser_alt_paths}
mkdir -p "$LOG"
status=0
run() {   # name, environment assignments..., then the pytest arguments after "--"
  local name=$1; shift
  local envs=()
  while [ "$1" != "--" ]; do envs+=("$1"); shift; done
  shift
  echo "== $name"
  if env "${envs[@]}" python -m pytest "$@" -q > "$LOG/$name.log" 2>&1; then echo "   ok"; else echo "   FAILED (see $LOG/$name.log)"; status=1; fi
  tail -n 2 "$LOG/$name.log" | sed 's/^/   /'
}
run python_launch_path CCFUSER_NATIVE_RUNTIME=0  -- tests/test_gpu_fused.py tests/test_gpu_models.py tests/test_gpu_graph.py -x
run library_router     CCFUSER_FUSED_ROUTER=0    -- tests/test_gpu_fused.py tests/test_gpu_models.py -x
run pair_kernel_always CCFUSER_SMALL_ROWS=0      -- tests/test_gpu_fused.py tests/test_gpu_models.py tests/test_gpu_graph.py -x
run one_cta_kernel     CCFUSER_TWO_CTA=0         -- tests/test_gpu_fused.py tests/test_gpu_bench_shapes.py -x
run canary             CCFUSER_CANARY=1          -- tests/test_gpu_fused.py -x -k "forward_backward or module_api"
run few_comm_ctas      CCFUSER_COMM_CTAS=16      -- tests/test_gpu_fused.py -x -k "forward_backward or module_api"
run epilogue_warps_push CCFUSER_COMM_WARPS=0     -- tests/test_gpu_fused.py tests/test_gpu_bench_shapes.py -x
if [ "$(python -c 'import torch; print(torch.cuda.device_count())')" -ge 2 ]; then
  run python_launch_path_2gpu CCFUSER_NATIVE_RUNTIME=0 -- tests/test_gpu_multi.py -x -k "fused_layer_multi_gpu and 2"
fi
exit $status
