"""tcgen05 grouped GEMM variants against fp32 torch references (needs a B200)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _mods():
    from ccfuser_b200 import native as N
    from ccfuser_b200.ops import gemm as G
    return N, G


def _groups(rows_list, device):
    base, cur = [], 0
    for r in rows_list:
        base.append(cur)
        cur += (r + 127) // 128 * 128
    return (torch.tensor(base, dtype=torch.int32, device=device),
            torch.tensor(rows_list, dtype=torch.int32, device=device), max(cur, 128))


def _close(got, ref, tol=2e-2):
    got, ref = got.float(), ref.float()
    scale = ref.abs().max().clamp_min(1e-6)
    err = (got - ref).abs().max() / scale
    assert torch.isfinite(got).all(), "non-finite output"
    assert err < tol, f"relative-to-max error {err:.4g}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 512, 256), (1000, 320, 1024), (4096, 1024, 4096)])
def test_plain_linear(dtype, m, n, k):
    N, G = _mods()
    torch.manual_seed(0)
    x = torch.randn(m, k, device="cuda", dtype=dtype)
    w = torch.randn(n, k, device="cuda", dtype=dtype) * 0.05
    b = torch.randn(n, device="cuda", dtype=dtype)
    y = G.linear(x, w, b)
    torch.cuda.synchronize()
    G.Workspace.get(x.device).check("linear")
    _close(y, F.linear(x.float(), w.float(), b.float()))
    y32 = G.linear(x, w, None, out_fp32=True)
    _close(y32, F.linear(x.float(), w.float()), tol=2e-3)


@pytest.mark.parametrize("act", ["gelu", "relu"])
def test_grouped_bias_act_ragged(act):
    N, G = _mods()
    torch.manual_seed(1)
    rows = [200, 0, 129, 128, 1, 517]
    e, k, n = len(rows), 256, 512
    gb, gr, total = _groups(rows, "cuda")
    x = torch.randn(total, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(e, n, k, device="cuda", dtype=torch.bfloat16) * 0.05
    b = torch.randn(e, n, device="cuda", dtype=torch.bfloat16) * 0.1
    pre = torch.full((total, n), 7.0, device="cuda", dtype=torch.bfloat16)
    out = torch.full((total, n), 7.0, device="cuda", dtype=torch.bfloat16)
    G.launch(a0=x, b0=w.view(e * n, k), a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_BIAS_ACT, n=n, k=k,
             group_base=gb, group_rows=gr, num_groups=e, b_group_rows=n, out0=out, out1=pre, bias0=b,
             act=N.ACT_CODE[act])
    torch.cuda.synchronize()
    G.Workspace.get(x.device).check("bias_act")
    fn = F.gelu if act == "gelu" else F.relu
    for i, r in enumerate(rows):
        s = int(gb[i])
        ref = F.linear(x[s:s + r].float(), w[i].float(), b[i].float())
        _close(pre[s:s + r], ref) if r else None
        _close(out[s:s + r], fn(ref)) if r else None
        pad = (r + 127) // 128 * 128
        assert (out[s + r:s + pad] == 0).all(), "padding rows of a tile must be written as zeros"


def test_swiglu_and_backward_epilogues():
    N, G = _mods()
    torch.manual_seed(2)
    rows = [130, 256, 0, 77]
    e, d, f = len(rows), 256, 384
    gb, gr, total = _groups(rows, "cuda")
    x = torch.randn(total, d, device="cuda", dtype=torch.bfloat16)
    wu = torch.randn(e, f, d, device="cuda", dtype=torch.bfloat16) * 0.06
    wg = torch.randn(e, f, d, device="cuda", dtype=torch.bfloat16) * 0.06
    bu = torch.randn(e, f, device="cuda", dtype=torch.bfloat16) * 0.1
    bg = torch.randn(e, f, device="cuda", dtype=torch.bfloat16) * 0.1
    h = torch.zeros(total, f, device="cuda", dtype=torch.bfloat16)
    gp = torch.zeros_like(h)
    up = torch.zeros_like(h)
    G.launch(a0=x, b0=wu.view(e * f, d), b1=wg.view(e * f, d), a_major=N.MAJ_K, b_major=N.MAJ_K,
             epi=N.EPI_SWIGLU, n=f, k=d, group_base=gb, group_rows=gr, num_groups=e, b_group_rows=f,
             out0=h, out1=gp, out2=up, bias0=bu, bias1=bg)
    # dgrad-2 style: dh [R, f] -> (dg, du) with the saved pre-activations; B = w2 [e, d, f] read MN-major
    w2 = torch.randn(e, d, f, device="cuda", dtype=torch.bfloat16) * 0.06
    dy = torch.randn(total, d, device="cuda", dtype=torch.bfloat16)
    dgate = torch.zeros_like(h)
    dup = torch.zeros_like(h)
    G.launch(a0=dy, b0=w2.view(e * d, f), a_major=N.MAJ_K, b_major=N.MAJ_MN, epi=N.EPI_DSWIGLU, n=f, k=d,
             group_base=gb, group_rows=gr, num_groups=e, b_group_rows=d, out0=dgate, out1=dup, aux0=gp, aux1=up)
    torch.cuda.synchronize()
    G.Workspace.get(x.device).check("swiglu")
    for i, r in enumerate(rows):
        if not r:
            continue
        s = int(gb[i])
        xr = x[s:s + r].float()
        g_ref = F.linear(xr, wg[i].float(), bg[i].float())
        u_ref = F.linear(xr, wu[i].float(), bu[i].float())
        _close(gp[s:s + r], g_ref)
        _close(up[s:s + r], u_ref)
        _close(h[s:s + r], F.silu(g_ref) * u_ref)
        dh = dy[s:s + r].float() @ w2[i].float()
        gq, uq = gp[s:s + r].float(), up[s:s + r].float()
        sg = torch.sigmoid(gq)
        _close(dgate[s:s + r], dh * uq * sg * (1 + gq * (1 - sg)))
        _close(dup[s:s + r], dh * gq * sg)


def test_dgrad_dact_and_two_segment_k():
    N, G = _mods()
    torch.manual_seed(3)
    rows = [140, 300]
    e, d, f = 2, 256, 512
    gb, gr, total = _groups(rows, "cuda")
    dy = torch.randn(total, d, device="cuda", dtype=torch.bfloat16)
    w2 = torch.randn(e, d, f, device="cuda", dtype=torch.bfloat16) * 0.06
    pre = torch.randn(total, f, device="cuda", dtype=torch.bfloat16)
    dh = torch.zeros(total, f, device="cuda", dtype=torch.bfloat16)
    G.launch(a0=dy, b0=w2.view(e * d, f), a_major=N.MAJ_K, b_major=N.MAJ_MN, epi=N.EPI_DACT, n=f, k=d,
             group_base=gb, group_rows=gr, num_groups=e, b_group_rows=d, out0=dh, aux0=pre, act=N.ACT_GELU)
    # two reduction segments: dx = dg @ Wg + du @ Wu with W* [e, f, d] read MN-major
    dg = torch.randn(total, f, device="cuda", dtype=torch.bfloat16)
    du = torch.randn(total, f, device="cuda", dtype=torch.bfloat16)
    wg = torch.randn(e, f, d, device="cuda", dtype=torch.bfloat16) * 0.05
    wu = torch.randn(e, f, d, device="cuda", dtype=torch.bfloat16) * 0.05
    dx = torch.zeros(total, d, device="cuda", dtype=torch.bfloat16)
    G.launch(a0=dg, a1=du, b0=wg.view(e * f, d), b1=wu.view(e * f, d), a_major=N.MAJ_K, b_major=N.MAJ_MN,
             epi=N.EPI_STORE, n=d, k=f, kseg=2, group_base=gb, group_rows=gr, num_groups=e, b_group_rows=f, out0=dx)
    torch.cuda.synchronize()
    G.Workspace.get(dy.device).check("dgrad")
    for i, r in enumerate(rows):
        s = int(gb[i])
        x = pre[s:s + r].float().requires_grad_(True)
        F.gelu(x).sum().backward()
        _close(dh[s:s + r], (dy[s:s + r].float() @ w2[i].float()) * x.grad)
        _close(dx[s:s + r], dg[s:s + r].float() @ wg[i].float() + du[s:s + r].float() @ wu[i].float())


def test_wgrad_kgrouped():
    N, G = _mods()
    torch.manual_seed(4)
    rows = [200, 0, 64, 385]
    e, m, n = len(rows), 256, 512
    gb, gr, total = _groups(rows, "cuda")
    a = torch.randn(total, m, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(total, n, device="cuda", dtype=torch.bfloat16)
    # rows between a group's end and the next multiple of 64 take part in the reduction: they must be zero in one operand
    for i, r in enumerate(rows):
        s = int(gb[i])
        a[s + r:s + (r + 127) // 128 * 128] = 0
    dw = torch.full((e, m, n), 3.0, device="cuda", dtype=torch.bfloat16)
    G.launch(a0=a, b0=b, a_major=N.MAJ_MN, b_major=N.MAJ_MN, epi=N.EPI_STORE, n=n, kgroup=True, m_per_group=m,
             group_base=gb, group_rows=gr, num_groups=e, out0=dw, ld_out=n)
    dw32 = torch.empty((e, m, n), device="cuda", dtype=torch.float32)
    G.launch(a0=a, b0=b, a_major=N.MAJ_MN, b_major=N.MAJ_MN, epi=N.EPI_STORE, n=n, kgroup=True, m_per_group=m,
             group_base=gb, group_rows=gr, num_groups=e, out0=dw32, ld_out=n, out_fp32=True)
    torch.cuda.synchronize()
    G.Workspace.get(a.device).check("wgrad")
    for i, r in enumerate(rows):
        s = int(gb[i])
        ref = a[s:s + r].float().t() @ b[s:s + r].float()
        if r == 0:
            assert (dw[i] == 0).all() and (dw32[i] == 0).all()
        else:
            _close(dw[i], ref)
            _close(dw32[i], ref, tol=2e-3)


@pytest.mark.parametrize("two_cta", [False, True])
def test_wgrad_with_sgd_in_the_epilogue(two_cta):
    """k-grouped product whose epilogue rewrites the weights in place (w - lr * (a^T b + wd * w)) instead of storing the
    gradient, on the one-CTA kernel and on CTA pairs, with groups of ragged and zero length."""
    N, G = _mods()
    torch.manual_seed(15)
    rows = [700, 0, 64, 1100, 255]
    e, m, n = len(rows), 512, 768
    lr, wd = 0.05, 0.1
    gb, gr, total = _groups(rows, "cuda")
    a = torch.randn(total, m, device="cuda", dtype=torch.bfloat16) * 0.1
    b = torch.randn(total, n, device="cuda", dtype=torch.bfloat16)
    for i, r in enumerate(rows):
        s = int(gb[i])
        a[s + r:s + (r + 127) // 128 * 128] = 0
    w0 = torch.randn(e, m, n, device="cuda", dtype=torch.bfloat16)
    w = w0.clone()
    G.launch(a0=a, b0=b, a_major=N.MAJ_MN, b_major=N.MAJ_MN, epi=N.EPI_STORE, n=n, kgroup=True, m_per_group=m,
             group_base=gb, group_rows=gr, num_groups=e, out0=w, ld_out=n, two_cta=two_cta, sgd=(lr, wd))
    torch.cuda.synchronize()
    G.Workspace.get(a.device).check("wgrad with sgd")
    for i, r in enumerate(rows):
        s = int(gb[i])
        dw = a[s:s + r].float().t() @ b[s:s + r].float()
        ref = w0[i].float() - lr * (dw + wd * w0[i].float())
        assert float((w[i].float() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())


def test_combine_epilogue_local_rank():
    """GEMM-2 epilogue on one GPU: rows go to `slot` rows of this rank's own combine buffer, scaled by the gate."""
    N, G = _mods()
    torch.manual_seed(5)
    rows = [150, 90]
    e, kdim, n = 2, 256, 512
    gb, gr, total = _groups(rows, "cuda")
    h = torch.randn(total, kdim, device="cuda", dtype=torch.bfloat16)
    w2 = torch.randn(e, n, kdim, device="cuda", dtype=torch.bfloat16) * 0.06
    b2 = torch.randn(e, n, device="cuda", dtype=torch.bfloat16) * 0.1
    nslots = sum(rows)
    perm = torch.randperm(nslots, device="cuda").int()
    row_src = torch.full((total,), -1, dtype=torch.int32, device="cuda")
    row_gate = torch.zeros(total, dtype=torch.float32, device="cuda")
    cur = 0
    for i, r in enumerate(rows):
        s = int(gb[i])
        row_src[s:s + r] = perm[cur:cur + r]  # rank 0 in the high byte
        row_gate[s:s + r] = torch.rand(r, device="cuda") + 0.1
        cur += r
    comb = torch.zeros(nslots, n, device="cuda", dtype=torch.bfloat16)
    done = torch.zeros(8, dtype=torch.int32, device="cuda")
    G.launch(a0=h, b0=w2.view(e * n, kdim), a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_COMBINE, n=n, k=kdim,
             group_base=gb, group_rows=gr, num_groups=e, b_group_rows=n, bias0=b2, row_src=row_src, row_gate=row_gate,
             peer_comb=[comb.data_ptr()], peer_done=[done.data_ptr()], world=1, send_finish=1, max_slots=nslots)
    torch.cuda.synchronize()
    G.Workspace.get(h.device).check("combine")
    assert int(done[0]) == nslots * G.combine_units(n) + 1
    for i, r in enumerate(rows):
        s = int(gb[i])
        ref = F.linear(h[s:s + r].float(), w2[i].float(), b2[i].float()) * row_gate[s:s + r, None]
        _close(comb[row_src[s:s + r].long()], ref)


@pytest.mark.parametrize("two_cta", [False, True])
def test_one_cta_and_two_cta_kernels_agree(two_cta):
    """Both tile shapes (128x256 per CTA, 256x256 per CTA pair) against the fp32 reference on ragged groups."""
    N, G = _mods()
    torch.manual_seed(6)
    rows = [257, 128, 0, 1, 600, 129]
    e, k, n = len(rows), 512, 768
    gb, gr, total = _groups(rows, "cuda")
    x = torch.randn(total + 256, k, device="cuda", dtype=torch.bfloat16)   # rows past the last group exist
    w = torch.randn(e, n, k, device="cuda", dtype=torch.bfloat16) * 0.05
    b = torch.randn(e, n, device="cuda", dtype=torch.bfloat16) * 0.1
    out = torch.full((total + 256, n), 5.0, device="cuda", dtype=torch.bfloat16)
    G.launch(a0=x, b0=w.view(e * n, k), a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_BIAS_ACT, n=n, k=k,
             group_base=gb, group_rows=gr, num_groups=e, b_group_rows=n, out0=out, bias0=b, act=N.ACT_GELU,
             two_cta=two_cta)
    torch.cuda.synchronize()
    G.Workspace.get(x.device).check("bias_act")
    for i, r in enumerate(rows):
        s = int(gb[i])
        if r:
            _close(out[s:s + r], F.gelu(F.linear(x[s:s + r].float(), w[i].float(), b[i].float())))
        pad = (r + 127) // 128 * 128
        assert (out[s + r:s + pad] == 0).all()
    # nothing outside the padded regions of the groups was touched
    assert (out[total:] == 5.0).all()
    used = torch.zeros(total + 256, dtype=torch.bool, device="cuda")
    for i, r in enumerate(rows):
        s = int(gb[i])
        used[s:s + (r + 127) // 128 * 128] = True
    assert (out[~used] == 5.0).all()


def test_scheduler_counters_return_to_zero():
    N, G = _mods()
    x = torch.randn(512, 128, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        G.linear(x, w)
    torch.cuda.synchronize()
    assert int(G.Workspace.get(x.device).sched.abs().sum()) == 0


@pytest.mark.parametrize("m,n,k", [(256, 4096, 1024), (300, 320, 256), (129, 128, 64)])
def test_narrow_tiles_on_the_one_cta_kernel(m, n, k):
    """128-column output tiles (bn=128): the tile shape of launches that would otherwise leave most SMs without work.
    Same product and bias as with 256-column tiles, including a column count that is not a multiple of the tile."""
    N, G = _mods()
    torch.manual_seed(1)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.05
    b = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    gb, gr = G.single_group(m, "cuda")
    outs = []
    for bn in (128, 256):
        y = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
        G.launch(a0=x, b0=w, a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_STORE, n=n, k=k, group_base=gb, group_rows=gr,
                 num_groups=1, b_group_rows=n, out0=y, bias0=b.view(1, n), two_cta=False, bn=bn)
        outs.append(y)
    torch.cuda.synchronize()
    G.Workspace.get(x.device).check("narrow tiles")
    _close(outs[0], F.linear(x.float(), w.float(), b.float()))
    assert torch.equal(outs[0], outs[1])
    # the CTA-pair kernel and MN-major operands have no narrow tile: refused on the host
    with pytest.raises(RuntimeError):
        G.launch(a0=x, b0=w, a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_STORE, n=n, k=k, group_base=gb, group_rows=gr,
                 num_groups=1, b_group_rows=n, out0=outs[0], two_cta=True, bn=128)
