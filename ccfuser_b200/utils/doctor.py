"""Environment report: what this machine offers to the library (``python -m ccfuser_b200 doctor``).

Read-only: it queries versions, devices and peer access and changes no setting."""
from __future__ import annotations

import json
import os
import shutil
import subprocess
from typing import Dict


def report() -> Dict[str, object]:
    import torch
    from .. import build, native
    out: Dict[str, object] = {"torch": torch.__version__, "torch_cuda": torch.version.cuda,
                              "cuda_available": torch.cuda.is_available()}
    nvcc = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else None)
    out["nvcc"] = nvcc
    if nvcc:
        try:
            text = subprocess.run([nvcc, "--version"], capture_output=True, text=True, timeout=20).stdout
            out["nvcc_release"] = next((ln.strip() for ln in text.splitlines() if "release" in ln), None)
        except Exception as e:  # noqa: BLE001
            out["nvcc_release"] = f"error: {e}"
    out["library"] = {"path": native.lib_path(), "built": os.path.exists(native.lib_path()), "stale": build.needs_build()}
    try:
        out["nccl"] = ".".join(str(v) for v in torch.cuda.nccl.version()) if torch.cuda.is_available() else None
    except Exception:  # noqa: BLE001
        out["nccl"] = None
    gpus = []
    problems = []
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            gpus.append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                         "memory_gb": round(p.total_memory / 2 ** 30, 1)})
            if (p.major, p.minor) != (10, 0):
                problems.append(f"GPU {i} is sm_{p.major}{p.minor}: the kernels are built for sm_100a only")
        peer = [[bool(i == j or torch.cuda.can_device_access_peer(i, j)) for j in range(n)] for i in range(n)]
        out["peer_access"] = peer
        if not all(all(r) for r in peer):
            problems.append("not every GPU pair has peer access: expert-parallel groups must stay inside a peer-connected set")
    else:
        problems.append("no CUDA device: only the CPU backend (gloo) and the host-side tests can run here")
    out["gpus"] = gpus
    if not out["library"]["built"] and not nvcc:
        problems.append("the CUDA library is not built and nvcc is missing")
    peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(peaks):
        with open(peaks) as f:
            d = json.load(f)
        out["measured_peaks"] = {k: d.get(k) for k in ("bf16_tflops", "bf16_tflops_sustained", "hbm_gbs")}
    out["problems"] = problems
    return out


def main():
    print(json.dumps(report(), indent=1))


if __name__ == "__main__":
    main()
