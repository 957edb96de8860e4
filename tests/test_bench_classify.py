"""bench.py:classify_kernel, the table behind `bench.py --breakdown`: every kernel family of a step lands in its category."""
import importlib.util
import os


def _bench():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    spec = importlib.util.spec_from_file_location("ccf_bench_script", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_kernel_names_map_to_their_categories():
    c = _bench().classify_kernel
    kw = dict(vocab_padded=50304, d_ffn=8192, tokens=8192)
    assert c("void ccf::grouped_gemm_pair_kernel<0, 1, 4, false>(CUtensorMap_st", "", "", **kw) == "moe_fused_gemms"
    assert c("ccf::combine_wait_kernel(int const*, int*", "", "", **kw) == "moe_wait_for_peers"
    for name in ("ccf::plan_kernel(CcfPlanArgs)", "ccf::route_hist_kernel(", "ccf::combine_reduce_kernel(",
                 "void ccf::router_topk_kernel<64>(", "ccf::colsum_grouped_kernel("):
        assert c(name, "", "", **kw) == "moe_route_plan_reduce", name
    assert c("ccf::sgd_step_kernel(void*, void const*", "", "", **kw) == "optimizer"
    assert c("ccf::sgd_multi_kernel(CcfSgdMulti)", "", "", **kw) == "optimizer"
    assert c("ncclDevKernel_AllReduce_Sum_bf16_RING_LL(ncclDevKernelArgsSt", "", "", **kw) == "nccl_allreduce"
    assert c("cudnn_generated_fort_native_sdpa_sm100_flash_fprop_f16", "", "", **kw) == "attention_core"
    assert c("nvjet_tst_256x256_64x4_2x2_2cta_v_bz_NTT", "aten::mm", "[[8192, 2048], [2048, 50304]]", **kw) == "lm_head_gemms"
    assert c("nvjet_tst_256x256_64x4_2x2_2cta_v_bz_NNT", "aten::mm", "[[8192, 8192], [8192, 2048]]", **kw) == "dense_ffn_gemms"
    assert c("nvjet_tst_256x256_64x4_2x2_2cta_v_bz_NNT", "aten::mm", "[[8192, 2048], [2048, 2048]]", **kw) == "attention_projection_gemms"
    assert c("void at::native::vectorized_elementwise_kernel<8,", "aten::add", "", **kw) == "elementwise_and_other"
