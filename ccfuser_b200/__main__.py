"""``python -m ccfuser_b200 <command> [args...]``: one entry point for the tools that otherwise run as modules."""
import runpy
import sys

COMMANDS = {
    "doctor": ("ccfuser_b200.utils.doctor", "what this machine offers: versions, GPUs, peer access, library state"),
    "build": ("ccfuser_b200.build", "compile the CUDA library for sm_100a (--selftest: also the C++ self-test program)"),
    "layer-bench": ("ccfuser_b200.bench.layer_bench", "MoE layer forward + backward timing (fig. 10 workload, Mixtral-size layers, skewed routing, small-message forward)"),
    "kernel-bench": ("ccfuser_b200.bench.kernel_bench", "fused dispatch+GEMM / GEMM+combine against all-to-all + GEMM (fig. 12)"),
    "gemm-bench": ("ccfuser_b200.bench.gemm_bench", "grouped GEMM throughput on one GPU"),
    "ae": ("ccfuser_b200.bench.ae", "run the three evaluation experiments and write their CSV files"),
    "plot": ("ccfuser_b200.bench.plot", "figures (SVG) from the CSV files"),
    "roofline": ("ccfuser_b200.bench.roofline", "roofline target of a layer configuration, or expected time per GEMM launch"),
    "overlap-trace": ("ccfuser_b200.bench.overlap_trace", "per-tile clock trace of the fused dispatch + GEMM-1 kernel"),
    "placement": ("ccfuser_b200.parallel.placement", "plan an expert placement for a saved [ranks, experts] count table"),
    "train": ("ccfuser_b200.examples.train", "synthetic / text-file training loops: GPT, BERT-QA, Transformer-XL"),
    "hf-train": ("ccfuser_b200.examples.hf_train", "Hugging Face GPT-2 / BERT-QA with converted MoE layers"),
}


def main():
    if len(sys.argv) < 2 or sys.argv[1] in ("-h", "--help") or sys.argv[1] not in COMMANDS:
        print("usage: python -m ccfuser_b200 <command> [args...]\n")
        for name, (_, what) in COMMANDS.items():
            print(f"  {name:14s} {what}")
        return 0 if len(sys.argv) >= 2 and sys.argv[1] in ("-h", "--help") else 2
    module = COMMANDS[sys.argv[1]][0]
    sys.argv = [module] + sys.argv[2:]
    runpy.run_module(module, run_name="__main__", alter_sys=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
