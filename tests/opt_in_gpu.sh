#!/bin/bash
# GPU tests that are not part of the default suite, each in a process of its own so that one failure does not take the
# others with it. One GPU is enough; the last block needs 2 (or 4) and is skipped otherwise.
#   bash tests/opt_in_gpu.sh [log-directory]
cd "$(dirname "$0")/.." || exit 1
LOG=${1:-/tmp/ccfuser_opt_in}
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
run selftest        CCFUSER_TEST_SELFTEST=1      -- tests/test_gpu_selftest.py -x
run router          CCFUSER_TEST_FUSED_ROUTER=1  -- tests/test_gpu_router.py -x
run native_runtime  CCFUSER_NATIVE_RUNTIME=1     -- tests/test_gpu_fused.py tests/test_gpu_models.py -x
run router_in_layer CCFUSER_FUSED_ROUTER=1       -- tests/test_gpu_fused.py tests/test_gpu_models.py -x
run graph           CCFUSER_TEST_GRAPH=1         -- tests/test_gpu_graph.py -x
run shadow_rebalance CCFUSER_X=0                 -- tests/test_gpu_placement_shadow.py --runxfail
run canary          CCFUSER_CANARY=1             -- tests/test_gpu_fused.py -x -k "forward_backward or module_api"
if [ "$(python -c 'import torch; print(torch.cuda.device_count())')" -ge 2 ]; then
  run multi_gpu_features CCFUSER_X=0             -- tests/test_gpu_multi.py --runxfail -k "shadow_and_rebalance or inside_data_parallel"
fi
exit $status
