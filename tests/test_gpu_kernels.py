"""Per-kernel parity on a B200: every C-ABI entry point against the CPU oracle (or, for the plain
GEMM, an fp32 matmul of the same bf16 inputs).  Tolerances: bf16 kernels max-abs 2e-2 relative to the
output scale (BASELINE north_star), fp32 kernels 1e-4, indices bit-exact."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import rte_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from speedup_thingy_b200.ops import CudaOps
    return CudaOps(DEV)


def _close(got, ref, tol, what=""):
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    scale = max(ref.abs().max().item(), 1e-6)
    err = (got - ref).abs().max().item()
    assert err <= tol * scale, f"{what}: max-abs {err:.3e} vs scale {scale:.3e} (tol {tol})"


def _bf(t):
    return t.to(torch.bfloat16)


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (300, 200, 136), (1024, 1536, 512),
                                   (8192, 512, 2048), (64, 96, 512)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_bf16_all_majors(ops, M, N, K, a_mn, b_mn):
    g = torch.Generator().manual_seed(M + N + K)
    a = _bf(torch.randn(M, K, generator=g))
    b = _bf(torch.randn(N, K, generator=g))
    ref = a.float() @ b.float().t()
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a row stride that is a multiple of 8 elements")
    a_dev = (a.t().contiguous() if a_mn else a).to(DEV)
    b_dev = (b.t().contiguous() if b_mn else b).to(DEV)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    keep, ops.small_gemm_rows = ops.small_gemm_rows, 0          # this test is about the tcgen05 kernel at every size
    try:
        ops.gemm(a_dev, b_dev, out, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn)
    finally:
        ops.small_gemm_rows = keep
    torch.cuda.synchronize()
    ops.check_status()
    _close(out, ref, 1e-2, f"gemm {M}x{N}x{K} a_mn={a_mn} b_mn={b_mn}")


@pytest.mark.parametrize("M,N,K", [(64, 1536, 512), (64, 512, 4096), (70, 104, 136), (256, 2048, 512), (1, 8, 8), (130, 96, 72)])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("mode", ["bf16", "f32_residual", "f32_split"])
def test_gemm_few_rows_kernel(ops, M, N, K, b_mn, mode):
    """The cp.async + mma.sync kernel the replay's chain uses (rte_gemm_bf16_small), every epilogue and both B majors."""
    g = torch.Generator().manual_seed(M * 7 + N + K)
    a, b = _bf(torch.randn(M, K, generator=g)), _bf(torch.randn(N, K, generator=g))
    ref = a.float() @ b.float().t()
    b_dev = (b.t().contiguous() if b_mn else b).to(DEV)
    assert M <= ops.small_gemm_rows
    before = ops.launches
    if mode == "bf16":
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        ops.gemm(a.to(DEV), b_dev, out, M=M, N=N, K=K, b_mn=b_mn)
        tol = 1e-2
    elif mode == "f32_residual":
        r = torch.randn(M, N, generator=g)
        ref = ref + r
        out = r.clone().to(DEV)
        ops.gemm(a.to(DEV), b_dev, out, M=M, N=N, K=K, b_mn=b_mn, epilogue=1, residual=out)
        tol = 2e-3
    else:
        out = torch.full((M, N), 3.0, device=DEV)
        ws = torch.empty(16 * M * N, device=DEV)
        ops.gemm_f32_few_rows(a.to(DEV), b_dev, out, M=M, N=N, K=K, b_mn=b_mn, ws=ws, accumulate=True)
        ref = ref + 3.0
        tol = 2e-3
        # the in-launch reduction (each tile's last CTA sums the partials) against the separate reduction launch, and a
        # second fused call: the arrival counters must be back at zero
        keep, ops.small_fused_reduce = ops.small_fused_reduce, True
        try:
            fused, again = torch.full((M, N), 3.0, device=DEV), torch.full((M, N), 3.0, device=DEV)
            ops.gemm_f32_few_rows(a.to(DEV), b_dev, fused, M=M, N=N, K=K, b_mn=b_mn, ws=ws, accumulate=True)
            ops.gemm_f32_few_rows(a.to(DEV), b_dev, again, M=M, N=N, K=K, b_mn=b_mn, ws=ws, accumulate=True)
        finally:
            ops.small_fused_reduce = keep
        torch.cuda.synchronize()
        assert torch.equal(out, fused) and torch.equal(out, again)
        assert not bool(ops._split_counters.any())
    torch.cuda.synchronize()
    ops.check_status()
    assert ops.launches > before
    _close(out, ref, tol, f"few-row gemm {M}x{N}x{K} b_mn={b_mn} {mode}")


def test_gemm_f32_residual_and_alias(ops):
    M, N, K = 512, 384, 256
    g = torch.Generator().manual_seed(1)
    a, b, r = _bf(torch.randn(M, K, generator=g)), _bf(torch.randn(N, K, generator=g)), torch.randn(M, N, generator=g)
    ref = a.float() @ b.float().t() + r
    out = r.clone().to(DEV)
    ops.gemm(a.to(DEV), b.to(DEV), out, M=M, N=N, K=K, epilogue=1, residual=out)
    torch.cuda.synchronize()
    _close(out, ref, 2e-3, "gemm f32 + residual (aliased)")


@pytest.mark.parametrize("Mo,No,Kred", [(1536, 512, 8192), (512, 512, 8192), (4096, 512, 4096), (96, 64, 1024), (200, 72, 520)])
def test_gemm_wgrad_split_k(ops, Mo, No, Kred):
    g = torch.Generator().manual_seed(Mo + No)
    a_t, b_t = _bf(torch.randn(Kred, Mo, generator=g)), _bf(torch.randn(Kred, No, generator=g))
    ref = a_t.float().t() @ b_t.float()
    out = torch.full((Mo, No), 7.0, dtype=torch.float32, device=DEV)
    ops.gemm_wgrad(a_t.to(DEV), b_t.to(DEV), out, M=Mo, N=No, K=Kred)
    torch.cuda.synchronize()
    ops.check_status()
    _close(out, ref, 2e-3, f"wgrad {Mo}x{No} over {Kred}")
    ops.gemm_wgrad(a_t.to(DEV), b_t.to(DEV), out, M=Mo, N=No, K=Kred, accumulate=True)
    torch.cuda.synchronize()
    _close(out, 2 * ref, 2e-3, "wgrad accumulate")


@pytest.mark.parametrize("Mo,No,Kred", [(2048, 512, 64), (512, 4096, 64), (1536, 512, 128), (512, 512, 256), (104, 72, 64), (8, 8, 8),
                                        (200, 136, 200)])
def test_gemm_wgrad_of_few_rows(ops, Mo, No, Kred):
    """Weight gradient of one audited sample: a rank-Kred update (Kred = the sample's rows) through the few-row kernel's
    transposed-A form, plain and accumulating."""
    g = torch.Generator().manual_seed(Mo + No + Kred)
    a_t, b_t = _bf(torch.randn(Kred, Mo, generator=g)), _bf(torch.randn(Kred, No, generator=g))
    ref = a_t.float().t() @ b_t.float()
    assert Kred <= ops.small_gemm_rows
    out = torch.full((Mo, No), 7.0, dtype=torch.float32, device=DEV)
    keep, ops.small_wgrad = ops.small_wgrad, True
    try:
        ops.gemm_wgrad(a_t.to(DEV), b_t.to(DEV), out, M=Mo, N=No, K=Kred)
        torch.cuda.synchronize()
        ops.check_status()
        _close(out, ref, 2e-3, f"few-row wgrad {Mo}x{No} over {Kred}")
        ops.gemm_wgrad(a_t.to(DEV), b_t.to(DEV), out, M=Mo, N=No, K=Kred, accumulate=True)
        torch.cuda.synchronize()
        _close(out, 2 * ref, 2e-3, "few-row wgrad accumulate")
    finally:
        ops.small_wgrad = keep


@pytest.mark.parametrize("M,d,f", [(256, 128, 256), (512, 512, 2048), (100, 64, 64), (8192, 512, 2048)])
def test_swiglu_epilogues(ops, M, d, f):
    g = torch.Generator().manual_seed(f)
    x, wug, wd = _bf(torch.randn(M, d, generator=g)), _bf(torch.randn(2 * f, d, generator=g) * 0.05), _bf(torch.randn(d, f, generator=g) * 0.05)
    z = torch.zeros(M, f, dtype=torch.bfloat16, device=DEV)
    ug = torch.zeros(M, 2 * f, dtype=torch.bfloat16, device=DEV)
    ops.gemm(x.to(DEV), wug.to(DEV), z, M=M, N=2 * f, K=d, epilogue=2, out2=ug, pair=f)
    torch.cuda.synchronize()
    ops.check_status()
    acc = x.float() @ wug.float().t()
    up, gate = acc[:, :f], acc[:, f:]
    _close(ug[:, :f], up, 1e-2, "saved up")
    _close(ug[:, f:], gate, 1e-2, "saved gate")
    _close(z, up * F.silu(gate), 1.5e-2, "z = up*silu(gate)")
    # backward epilogue: dz = dout @ wd  (wd stored [d, f]),  (dup | dgate) from the saved (up | gate)
    dout = _bf(torch.randn(M, d, generator=g))
    dug = torch.zeros(M, 2 * f, dtype=torch.bfloat16, device=DEV)
    ops.gemm(dout.to(DEV), wd.to(DEV), dug, M=M, N=f, K=d, b_mn=True, epilogue=3, residual=ug, pair=f)
    torch.cuda.synchronize()
    ops.check_status()
    ups, gts = ug[:, :f].float().cpu(), ug[:, f:].float().cpu()
    dz = dout.float() @ wd.float()
    sg = torch.sigmoid(gts)
    _close(dug[:, :f], dz * gts * sg, 1.5e-2, "d up")
    _close(dug[:, f:], dz * ups * sg * (1 + gts * (1 - sg)), 1.5e-2, "d gate")


# ------------------------------------------------------------------ norm / CE / embedding
@pytest.mark.parametrize("rows,d", [(64, 128), (1000, 512), (333, 1024), (17, 64)])
def test_rmsnorm_fwd_bwd(ops, rows, d):
    g = torch.Generator().manual_seed(d)
    x, w = torch.randn(rows, d, generator=g), torch.randn(d, generator=g)
    fg, fb = torch.randn(d, generator=g) * 0.1, torch.randn(d, generator=g) * 0.1
    dy, dres = torch.randn(rows, d, generator=g), torch.randn(rows, d, generator=g)
    for film in (False, True):
        xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        fgr, fbr = fg.clone().requires_grad_(True), fb.clone().requires_grad_(True)
        y = O.rmsnorm(xr, wr)
        if film:
            y = y * (1 + fgr) + fbr
        y.backward(dy)
        y32 = torch.zeros(rows, d, device=DEV)
        y16 = torch.zeros(rows, d, dtype=torch.bfloat16, device=DEV)
        rstd = torch.zeros(rows, device=DEV)
        kw = dict(film_gamma=fg.to(DEV), film_beta=fb.to(DEV)) if film else {}
        ops.rmsnorm_fwd(x.to(DEV), w.to(DEV), y16, rstd, y_f32=y32, **kw)
        _close(y32, y, 1e-5, "rmsnorm f32")
        _close(y16, y, 1e-2, "rmsnorm bf16")
        dx = torch.zeros(rows, d, device=DEV)
        dx16 = torch.zeros(rows, d, dtype=torch.bfloat16, device=DEV)
        dw, dgm, dbt = (torch.zeros(d, device=DEV) for _ in range(3))
        part, pg, pb = (torch.zeros(296, d, device=DEV) for _ in range(3))
        kwb = dict(film_gamma=fg.to(DEV), dgamma_out=dgm, dbeta_out=dbt, partial_g=pg, partial_b=pb) if film else {}
        ops.rmsnorm_bwd(x.to(DEV), w.to(DEV), rstd, dy.to(DEV), dres.to(DEV), dx, dx16, dw, part, **kwb)
        torch.cuda.synchronize()
        _close(dx, xr.grad + dres, 1e-4, "rmsnorm dx")
        _close(dx16, xr.grad + dres, 1e-2, "rmsnorm dx bf16")
        _close(dw, wr.grad, 1e-4, "rmsnorm dw")
        if film:
            _close(dgm, fgr.grad, 1e-4, "film dgamma")
            _close(dbt, fbr.grad, 1e-4, "film dbeta")


@pytest.mark.parametrize("B,S,V", [(4, 16, 96), (8, 64, 2048), (3, 5, 1000)])
def test_cross_entropy_fwd_bwd(ops, B, S, V):
    g = torch.Generator().manual_seed(V)
    logits = _bf(torch.randn(B * S, V, generator=g) * 3)
    tg = torch.randint(0, V, (B, S), generator=g)
    wgt = torch.rand(B, generator=g)
    lr = logits.float().requires_grad_(True)
    per = O.lm_loss_per_sample(lr.view(B, S, V), tg)
    (per * wgt).sum().backward()
    ld = logits.to(DEV).clone()
    loss_tok = torch.zeros(B * S, device=DEV)
    ops.ce_fwd_bwd(ld, tg.to(DEV).view(-1), wgt.to(DEV), S, loss_tok, ld)
    per_dev = torch.zeros(B, device=DEV)
    ops.segment_sum(loss_tok, per_dev, B, S)
    torch.cuda.synchronize()
    ops.check_status()
    _close(per_dev, per, 1e-4, "per-sample CE")
    _close(ld, lr.grad, 1e-2, "dlogits")


def test_embedding_fwd_bwd(ops):
    g = torch.Generator().manual_seed(5)
    V, d, n = 300, 64, 1000
    table, tok, dx = torch.randn(V, d, generator=g), torch.randint(0, V, (n,), generator=g), torch.randn(n, d, generator=g)
    out = torch.zeros(n, d, device=DEV)
    ops.embed_fwd(tok.to(DEV), table.to(DEV), out)
    assert torch.equal(out.cpu(), table[tok])
    dt = torch.zeros(V, d, device=DEV)
    acc = torch.full((V * d,), 12345, dtype=torch.int64, device=DEV)      # scratch: any contents
    ops.embed_bwd(tok.to(DEV), dx.to(DEV), dt, acc)
    torch.cuda.synchronize()
    _close(dt, torch.zeros(V, d).index_add_(0, tok, dx), 1e-5, "embedding grad")
    # order-free accumulation: a second run is identical bit for bit, and accumulates onto what is there
    dt2 = torch.zeros(V, d, device=DEV)
    ops.embed_bwd(tok.to(DEV), dx.to(DEV), dt2, acc)
    assert torch.equal(dt, dt2)
    ops.embed_bwd(tok.to(DEV), dx.to(DEV), dt2, acc)
    _close(dt2, 2 * torch.zeros(V, d).index_add_(0, tok, dx), 1e-5, "embedding grad accumulates")


# ------------------------------------------------------------------ attention (+RoPE)
@pytest.mark.parametrize("B,S,H,hd", [(2, 16, 4, 8), (3, 64, 4, 32), (2, 64, 8, 64), (1, 200, 2, 64), (2, 33, 2, 128), (2, 256, 2, 64)])
def test_attention_fwd_bwd(ops, B, S, H, hd):
    g = torch.Generator().manual_seed(S * H)
    d = H * hd
    qkv = _bf(torch.randn(B * S, 3 * d, generator=g))
    dy = _bf(torch.randn(B * S, d, generator=g))
    lr = qkv.float().requires_grad_(True)
    q, k, v = (t.transpose(1, 2) for t in lr.view(B, S, 3, H, hd).unbind(2))
    cos, sin = O.rope_tables(S, hd)
    yref = O.causal_attention(O.rope_apply(q, cos, sin), O.rope_apply(k, cos, sin), v).transpose(1, 2).reshape(B * S, d)
    yref.backward(dy.float())
    y = torch.zeros(B * S, d, dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros(B * H * S, device=DEV)
    dq = torch.zeros(B * S, 3 * d, dtype=torch.bfloat16, device=DEV)
    qd = qkv.to(DEV)
    ops.attn_fwd(qd, y, lse, B=B, S=S, n_heads=H, head_dim=hd)
    ops.attn_bwd(qd, y, dy.to(DEV), lse, dq, B=B, S=S, n_heads=H, head_dim=hd)
    torch.cuda.synchronize()
    _close(y, yref, 2e-2, "attention out")
    _close(dq, lr.grad, 2e-2, "attention dqkv")
    # forward with the column-masked second output == forward, then the mask as its own pass (same bits)
    R = 3
    tab = (torch.rand(R, d, generator=g) > 0.5).float().mul(0.5).to(DEV)
    rows = torch.randint(0, R, (B,), generator=g).to(DEV, torch.int32)
    y2, ym, lse2 = torch.zeros_like(y), torch.zeros_like(y), torch.zeros_like(lse)
    ops.attn_fwd_masked(qd, y2, ym, lse2, rows, tab, B=B, S=S, n_heads=H, head_dim=hd)
    ref_m = torch.zeros_like(y)
    ops.colmask_mul(y, rows, tab, S, ref_m, B * S, d)
    torch.cuda.synchronize()
    assert torch.equal(y, y2) and torch.equal(lse, lse2) and torch.equal(ym, ref_m)
    # backward on a masked upstream gradient == the mask as its own pass, then the plain backward (same bits), with
    # dy left alone on the tensor-core path
    dyd = dy.to(DEV)
    dy_m, dq_ref, dq_m = torch.zeros_like(dyd), torch.zeros_like(dq), torch.zeros_like(dq)
    ops.colmask_mul(dyd, rows, tab, S, dy_m, B * S, d)
    ops.attn_bwd(qd, y, dy_m, lse, dq_ref, B=B, S=S, n_heads=H, head_dim=hd)
    keep = dyd.clone()
    ops.attn_bwd_masked(qd, y, dyd, lse, dq_m, rows, tab, B=B, S=S, n_heads=H, head_dim=hd)
    torch.cuda.synchronize()
    assert torch.equal(dq_m, dq_ref)
    if hd in (32, 64, 128):
        assert torch.equal(dyd, keep)


# ------------------------------------------------------------------ router / top-k
def test_router_fwd_indices_and_aux_bwd(ops):
    cfg = O.ModelCfg(vocab_size=64, d_model=64, n_heads=4, d_ff=64, recipe_count=5, head_groups=4, ffn_groups=4,
                     active_head_groups=2, active_ffn_groups=2, macro_rank=8)
    B, S, d, hid, R, K, T = 12, 8, 64, 64, 5, 3, 4
    params = O.init_params(cfg, seed=2)
    g = torch.Generator().manual_seed(9)
    for n in list(params):
        if n.startswith("router."):
            params[n] = torch.randn(params[n].shape, generator=g) * 0.3
    h0 = torch.randn(B, S, d, generator=g)
    leaves = {n: v.clone().requires_grad_(True) for n, v in params.items()}
    h0r = h0.clone().requires_grad_(True)
    route = O.router_forward(leaves, cfg, h0r, None, None)
    tr = O.TrainCfg()
    aux = O.router_aux_losses(tr, route["recipe_probs"], route["expected_depth"], torch.zeros(R))
    (aux["load"] + aux["depth"]).backward()
    f32, i32 = torch.float32, torch.int32
    e = lambda *s, dtype=f32: torch.zeros(*s, dtype=dtype, device=DEV)  # noqa: E731
    w = dict(r_w0=params["router.recipe_mlp.0.weight"], r_b0=params["router.recipe_mlp.0.bias"],
             r_w2=params["router.recipe_mlp.2.weight"], r_b2=params["router.recipe_mlp.2.bias"],
             d_w0=params["router.depth_mlp.0.weight"], d_b0=params["router.depth_mlp.0.bias"],
             d_w2=params["router.depth_mlp.2.weight"], d_b2=params["router.depth_mlp.2.bias"],
             pass_recipe_bias=params["router.pass_recipe_bias"])
    w = {k: v.to(DEV).contiguous() for k, v in w.items()}
    out = dict(pooled=e(B, d), r_hidden_pre=e(B, hid), d_hidden_pre=e(B, hid), recipe_logits=e(B, R), recipe_probs=e(B, R),
               depth_probs=e(B, K), expected_depth=e(B), router_entropy=e(B), recipe_id=e(B, dtype=i32),
               recipe_id_by_pass=e(B, T, dtype=i32), depth_id=e(B, dtype=i32), depth=e(B, dtype=i32))
    dv = torch.tensor(cfg.depth_choices, dtype=i32, device=DEV)
    ops.router_fwd(h0.to(DEV), w, dv, out, B=B, S=S, d=d, hid=hid, R=R, K=K, T=T, fixed_recipe=None, fixed_depth_id=None)
    torch.cuda.synchronize()
    _close(out["recipe_logits"], route["recipe_logits"], 1e-4, "recipe logits")
    _close(out["recipe_probs"], route["recipe_probs"], 1e-4, "recipe probs")
    _close(out["expected_depth"], route["expected_depth"], 1e-4, "expected depth")
    _close(out["router_entropy"], route["router_entropy"], 1e-4, "entropy")
    # indices: bit-exact given the kernel's own logits (lowest index on ties)
    rl = out["recipe_logits"].cpu()
    assert torch.equal(out["recipe_id"].cpu().long(), O.argmax_lowest(torch.softmax(rl, -1)))
    by_pass = O.argmax_lowest(torch.softmax(rl[:, None, :] + params["router.pass_recipe_bias"][None], -1))
    assert torch.equal(out["recipe_id_by_pass"].cpu().long(), by_pass)
    assert torch.equal(out["depth_id"].cpu().long(), O.argmax_lowest(out["depth_probs"].cpu()))
    assert torch.equal(out["depth"].cpu().long(), torch.tensor(cfg.depth_choices)[out["depth_id"].cpu().long()])
    grads = {k: e(*w[k].shape) for k in ("r_w0", "r_b0", "r_w2", "r_b2", "d_w0", "d_b0", "d_w2", "d_b2")}
    dh0 = e(B * S, d)
    auxd = e(2)
    scratch = e(32 + B * (2 * hid + R + K + 4 * d) + 4)
    ops.router_aux_bwd(w, out, dv, tr.lambda_load, tr.lambda_depth, auxd, grads, dh0, scratch, B=B, S=S, d=d, hid=hid, R=R, K=K)
    torch.cuda.synchronize()
    assert abs(float(auxd[0]) - float(aux["load"])) < 1e-6 and abs(float(auxd[1]) - float(aux["depth"])) < 1e-7
    _close(dh0.view(B, S, d), h0r.grad, 1e-3, "router dh0")
    names = dict(r_w0="router.recipe_mlp.0.weight", r_b0="router.recipe_mlp.0.bias", r_w2="router.recipe_mlp.2.weight",
                 r_b2="router.recipe_mlp.2.bias", d_w0="router.depth_mlp.0.weight", d_b0="router.depth_mlp.0.bias",
                 d_w2="router.depth_mlp.2.weight", d_b2="router.depth_mlp.2.bias")
    for k, n in names.items():
        _close(grads[k], leaves[n].grad, 1e-3, n)
    # the two-part form (everything but the add into dh0 first, the add later) gives the same bits
    grads2 = {k: e(*w[k].shape) for k in grads}
    dh0b, aux2, scratch2 = e(B * S, d), e(2), e(32 + B * (2 * hid + R + K + 4 * d) + 4)
    ops.router_aux_bwd_early(w, out, dv, tr.lambda_load, tr.lambda_depth, aux2, grads2, scratch2, B=B, S=S, d=d, hid=hid, R=R, K=K)
    ops.router_aux_add_dh0(dh0b, scratch2, B=B, S=S, d=d, hid=hid, R=R, K=K)
    torch.cuda.synchronize()
    assert torch.equal(dh0, dh0b) and torch.equal(auxd, aux2)
    for k in grads:
        assert torch.equal(grads[k], grads2[k]), k


def test_router_fixed_ids(ops):
    B, S, d, hid, R, K, T = 4, 4, 32, 32, 4, 3, 4
    f32, i32 = torch.float32, torch.int32
    e = lambda *s, dtype=f32: torch.zeros(*s, dtype=dtype, device=DEV)  # noqa: E731
    w = dict(r_w0=e(hid, d), r_b0=e(hid), r_w2=e(R, hid), r_b2=e(R), d_w0=e(hid, d), d_b0=e(hid), d_w2=e(K, hid), d_b2=e(K),
             pass_recipe_bias=e(T, R))
    out = dict(pooled=e(B, d), r_hidden_pre=e(B, hid), d_hidden_pre=e(B, hid), recipe_logits=e(B, R), recipe_probs=e(B, R),
               depth_probs=e(B, K), expected_depth=e(B), router_entropy=e(B), recipe_id=e(B, dtype=i32),
               recipe_id_by_pass=e(B, T, dtype=i32), depth_id=e(B, dtype=i32), depth=e(B, dtype=i32))
    dv = torch.tensor([1, 2, 4], dtype=i32, device=DEV)
    ops.router_fwd(e(B * S, d), w, dv, out, B=B, S=S, d=d, hid=hid, R=R, K=K, T=T, fixed_recipe=2, fixed_depth_id=1)
    torch.cuda.synchronize()
    assert out["recipe_id"].tolist() == [2] * B and out["depth"].tolist() == [2] * B
    assert out["recipe_id_by_pass"].flatten().tolist() == [2] * (B * T)
    # all-equal logits: the tie goes to index 0
    ops.router_fwd(e(B * S, d), w, dv, out, B=B, S=S, d=d, hid=hid, R=R, K=K, T=T, fixed_recipe=None, fixed_depth_id=None)
    torch.cuda.synchronize()
    assert out["recipe_id"].tolist() == [0] * B and out["depth_id"].tolist() == [0] * B


@pytest.mark.parametrize("rows,n,k", [(7, 16, 4), (100, 2048, 256), (33, 100, 100), (5, 6, 2)])
def test_topk_lowest_index_bit_exact(ops, rows, n, k):
    g = torch.Generator().manual_seed(n)
    scores = torch.randn(rows, n, generator=g)
    scores[0] = 1.0                                          # all-equal row
    scores[1, ::3] = scores[1, 0]                            # many ties
    scores = (scores * 4).round() / 4                        # quantise -> constructed ties everywhere
    vals, idx = O.topk_lowest(scores, k)
    gi = torch.zeros(rows, k, dtype=torch.int32, device=DEV)
    gv = torch.zeros(rows, k, device=DEV)
    ops.topk_lowest_index(scores.to(DEV), k, gi, gv)
    torch.cuda.synchronize()
    assert torch.equal(gi.cpu().long(), idx)
    assert torch.equal(gv.cpu(), vals)


@pytest.mark.parametrize("n,S,d,with_select,with_add2", [(3, 8, 64, False, False), (2, 16, 512, True, True), (5, 4, 128, True, False)])
def test_residual_rmsnorm_fwd_matches_the_separate_steps(ops, n, S, d, with_select, with_add2):
    g = torch.Generator().manual_seed(d + n)
    rows = n * S
    base, branch, pas, add2 = (torch.randn(rows, d, generator=g) for _ in range(4))
    w, fg, fb = torch.randn(d, generator=g), torch.randn(d, generator=g) * 0.1, torch.randn(d, generator=g) * 0.1
    s1, s2 = torch.tensor([0.7]), torch.tensor([0.1])
    active = torch.tensor([i % 2 for i in range(n)], dtype=torch.int32)
    x1 = base + 0.7 * branch
    if with_select:
        x1 = torch.where(active.bool().repeat_interleave(S)[:, None], x1, pas)
    x = x1 + 0.1 * add2 if with_add2 else x1
    y_ref = O.rmsnorm(x, w) * (1 + fg) + fb
    dev = lambda t: t.to(DEV)  # noqa: E731
    x1_out, x_out = torch.zeros(rows, d, device=DEV), torch.zeros(rows, d, device=DEV)
    y16, rstd = torch.zeros(rows, d, dtype=torch.bfloat16, device=DEV), torch.zeros(rows, device=DEV)
    ops.residual_rmsnorm_fwd(dev(base), dev(branch), dev(s1), x_out, dev(w), y16, rstd, S=S,
                             active=dev(active) if with_select else None, passthrough=dev(pas) if with_select else None,
                             add2=dev(add2) if with_add2 else None, scale2=dev(s2) if with_add2 else None, x1_out=x1_out,
                             film_gamma=dev(fg), film_beta=dev(fb))
    torch.cuda.synchronize()
    assert (x1_out.cpu() - x1).abs().max() <= 1e-6 and (x_out.cpu() - x).abs().max() <= 1e-6
    assert (y16.cpu().float() - y_ref).abs().max() <= 2e-2 * y_ref.abs().max()
    assert (rstd.cpu() - torch.rsqrt(x.pow(2).mean(-1) + 1e-5)).abs().max() <= 1e-5


@pytest.mark.parametrize("n,S,d,splits,film", [(1, 64, 512, 4, True), (3, 16, 128, 3, True), (2, 8, 64, 2, False)])
def test_norm_launches_fed_with_split_partials_equal_reduce_then_launch(ops, n, S, d, splits, film):
    """rte_residual_rmsnorm_fwd_splits / rte_rmsnorm_bwd_splits: a branch (or dy) handed over as split-K partials gives
    the bits of rte_reduce_splits followed by the plain launch, and the summed branch comes back in branch_out."""
    g = torch.Generator().manual_seed(11 * d + splits)
    rows = n * S
    stride = rows * d + 64                                           # partials need not be packed
    dev = lambda t: t.to(DEV)  # noqa: E731
    parts = dev(torch.randn(splits, stride, generator=g))
    base, pas, add2 = (dev(torch.randn(rows, d, generator=g)) for _ in range(3))
    w, fg, fb = (dev(torch.randn(d, generator=g) * 0.3) for _ in range(3))
    s1, s2 = dev(torch.tensor([0.7])), dev(torch.tensor([0.1]))
    active = dev(torch.tensor([i % 2 for i in range(n)], dtype=torch.int32))
    summed = torch.zeros(rows, d, device=DEV)
    ops.reduce_splits(parts, splits, stride, rows * d, summed, False)
    outs = []
    for fused in (False, True):
        x1, x = torch.zeros(rows, d, device=DEV), torch.zeros(rows, d, device=DEV)
        y16, rstd = torch.zeros(rows, d, dtype=torch.bfloat16, device=DEV), torch.zeros(rows, device=DEV)
        kept = torch.full((rows, d), 7.0, device=DEV)
        ops.residual_rmsnorm_fwd(base, parts if fused else summed, s1, x, w, y16, rstd, S=S, active=active, passthrough=pas,
                                 add2=add2, scale2=s2, x1_out=x1, film_gamma=fg if film else None, film_beta=fb if film else None,
                                 branch_splits=(splits, stride) if fused else (1, 0), branch_out=kept if fused else None)
        outs.append((x1, x, y16, rstd, kept))
    torch.cuda.synchronize()
    for a, b in zip(outs[0][:4], outs[1][:4]):
        assert torch.equal(a, b)
    assert torch.equal(outs[1][4], summed)                          # every row's sum is kept, frozen samples' too
    # backward
    xin, dres = dev(torch.randn(rows, d, generator=g)), dev(torch.randn(rows, d, generator=g))
    rstd = dev(torch.rand(rows, generator=g) + 0.5)
    res = []
    for fused in (False, True):
        dx, dx16 = torch.zeros(rows, d, device=DEV), torch.zeros(rows, d, dtype=torch.bfloat16, device=DEV)
        dw, dg_, db_ = (torch.zeros(d, device=DEV) for _ in range(3))
        pw, pg, pb = (torch.zeros(128, d, device=DEV) for _ in range(3))
        ops.rmsnorm_bwd(xin, w, rstd, parts if fused else summed, dres, dx, dx16, dw, pw, film_gamma=fg if film else None,
                        dgamma_out=dg_ if film else None, dbeta_out=db_ if film else None, partial_g=pg if film else None,
                        partial_b=pb if film else None, dy_splits=(splits, stride) if fused else (1, 0))
        res.append((dx, dx16, dw, dg_, db_))
    torch.cuda.synchronize()
    for a, b in zip(res[0], res[1]):
        assert torch.equal(a, b)
    with pytest.raises(Exception):
        ops.rmsnorm_bwd(xin, w, rstd, parts, dres, res[0][0], None, None, None, dy_splits=(splits, rows * d - 4))   # overlapping partials


def test_swiglu_standalone_pass_matches_fused_epilogue_math(ops):
    g = torch.Generator().manual_seed(12)
    rows, F_ = 300, 192
    ug = torch.randn(rows, 2 * F_, generator=g).bfloat16()
    dz = torch.randn(rows, F_, generator=g).bfloat16()
    up, gate = ug[:, :F_].float().requires_grad_(), ug[:, F_:].float().requires_grad_()
    z_ref = up * torch.nn.functional.silu(gate)
    (z_ref * dz.float()).sum().backward()
    z = torch.empty(rows, F_, dtype=torch.bfloat16, device=DEV)
    dug = torch.empty(rows, 2 * F_, dtype=torch.bfloat16, device=DEV)
    ops.swiglu_fwd(ug.to(DEV), z, rows, F_)
    ops.swiglu_bwd(ug.to(DEV), dz.to(DEV), dug, rows, F_)
    torch.cuda.synchronize()
    assert (z.cpu().float() - z_ref.detach()).abs().max() <= 1e-2 * z_ref.abs().max()
    ref = torch.cat([up.grad, gate.grad], dim=1)
    assert (dug.cpu().float() - ref).abs().max() <= 1e-2 * ref.abs().max()


# ------------------------------------------------------------------ vocabulary shortlist
@pytest.mark.parametrize("B,S,V,C,TC,HN,RN,K", [(3, 7, 96, 8, 2, 4, 4, 16), (4, 33, 2048, 64, 2, 32, 32, 128),
                                                (2, 5, 50, 7, 3, 60, 0, 50), (2, 9, 4096, 64, 1, 0, 8, 256)])
def test_shortlist_build_bit_exact(ops, B, S, V, C, TC, HN, RN, K):
    g = torch.Generator().manual_seed(V + K)
    oc = O.OutputCfg(mode="shortlist", num_clusters=C, shortlist_top_clusters=TC, shortlist_max_tokens=K,
                     hard_negatives=HN, random_negatives=RN)
    targets = torch.randint(0, V, (B, S), generator=g)
    targets[0, 0], targets[-1, -1] = 0, V - 1
    top = torch.stack([torch.randperm(C, generator=g)[:TC] for _ in range(B * S)]).view(B, S, TC)
    rnd = torch.randint(0, V, (B, S, RN), generator=g)
    cands = O.shortlist_candidates(targets, top, rnd, V, oc)
    want = O.dedupe_preserve_first(cands, K)
    dups = torch.tensor([cands.shape[-1] - len(set(r.tolist())) for r in cands.view(B * S, -1)])
    out = torch.full((B * S, K), -1, dtype=torch.int32, device=DEV)
    dc = torch.zeros(B * S, dtype=torch.int32, device=DEV)
    rnd_dev = rnd.view(B * S, RN).to(torch.int32).to(DEV) if RN else torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.shortlist_build(targets.to(DEV), top.view(B * S, TC).to(torch.int32).to(DEV), rnd_dev, out, dc,
                        V=V, C=C, TC=TC, HN=HN, RN=RN, K=K)
    ops.check_status()
    assert torch.equal(out.cpu().long().view(B, S, K), want)
    assert torch.equal(dc.cpu().long(), dups)
    assert torch.equal(out[:, 0].cpu().long(), targets.view(-1))


@pytest.mark.parametrize("rows,S,d,V,K", [(21, 7, 64, 96, 16), (256, 64, 512, 2048, 128)])
def test_shortlist_ce_matches_reference_math(ops, rows, S, d, V, K):
    g = torch.Generator().manual_seed(rows)
    hidden = torch.randn(rows, d, generator=g).bfloat16()
    W = (torch.randn(V, d, generator=g) * 0.2).bfloat16()
    sl = torch.stack([torch.randperm(V, generator=g)[:K] for _ in range(rows)])
    wgt = torch.rand(rows // S, generator=g) + 0.5
    lg = torch.einsum("rd,rkd->rk", hidden.float(), W.float()[sl]).bfloat16().float().requires_grad_(True)
    loss_tok = torch.nn.functional.cross_entropy(lg, torch.zeros(rows, dtype=torch.long), reduction="none")
    (loss_tok.view(-1, S).sum(1) * wgt).sum().backward()
    dense_ref = torch.zeros(rows, V).scatter_(1, sl, lg.grad)
    out_loss = torch.zeros(rows, device=DEV)
    out_lg = torch.zeros(rows, K, dtype=torch.bfloat16, device=DEV)
    dense = torch.full((rows, V), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.shortlist_ce(hidden.to(DEV), W.to(DEV), sl.to(torch.int32).to(DEV), wgt.to(DEV), S, out_loss, out_lg, dense)
    torch.cuda.synchronize()
    assert (out_lg.cpu().float() - lg.detach()).abs().max() <= 0.02 * lg.detach().abs().max()
    assert (out_loss.cpu() - loss_tok.detach()).abs().max() <= 2e-2
    assert (dense.cpu().float() - dense_ref).abs().max() <= 1e-2 * dense_ref.abs().max() + 1e-3
    assert (dense.cpu().float() != 0).sum(1).max() <= K


# ------------------------------------------------------------------ macro operator
@pytest.mark.parametrize("rows,S,d,V,K", [(21, 7, 64, 96, 16), (256, 64, 512, 2048, 128)])
def test_shortlist_ce_from_full_logits_equals_the_gathered_form(ops, rows, S, d, V, K):
    """rte_shortlist_ce_from_logits (dot products taken from a full-vocabulary GEMM) against rte_shortlist_ce (K weight
    rows gathered per token): same bf16 logits, so the loss and the dense gradient agree to rounding."""
    g = torch.Generator().manual_seed(rows + K)
    hidden = _bf(torch.randn(rows, d, generator=g)).to(DEV)
    W = _bf(torch.randn(V, d, generator=g) * 0.1).to(DEV)
    ids = torch.stack([torch.randperm(V, generator=g)[:K] for _ in range(rows)]).to(torch.int32).to(DEV)
    rw = (torch.rand(-(-rows // S), generator=g) + 0.5).to(DEV)
    loss_a, loss_b = torch.zeros(rows, device=DEV), torch.zeros(rows, device=DEV)
    dense_a = torch.full((rows, V), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.shortlist_ce(hidden, W, ids, rw, S, loss_a, None, dense_a)
    logits = torch.zeros(rows, V, dtype=torch.bfloat16, device=DEV)
    keep, ops.small_gemm_rows = ops.small_gemm_rows, 0
    try:
        ops.gemm(hidden, W, logits, M=rows, N=V, K=d)
    finally:
        ops.small_gemm_rows = keep
    ops.shortlist_ce_from_logits(logits, ids, rw, S, loss_b)
    torch.cuda.synchronize()
    ops.check_status()
    _close(loss_b, loss_a, 1e-3, "loss from full logits")
    assert (logits.float() - dense_a.float()).abs().max().item() <= 2e-2 * dense_a.float().abs().max().item()
    assert int((logits != 0).sum(1).max()) <= K


@pytest.mark.parametrize("tensor", [False, True])       # True: transposed weights prepared -> tensor-core forward
@pytest.mark.parametrize("B,S,d,m,R", [(4, 16, 64, 8, 5), (6, 64, 128, 32, 5), (3, 40, 512, 32, 5), (2, 8, 64, 48, 3)])
def test_macro_phi_fwd_bwd(ops, B, S, d, m, R, tensor):
    K = 3
    cfg = O.ModelCfg(d_model=d, macro_rank=m, recipe_count=R, macro_update_scale=0.05)
    g = torch.Generator().manual_seed(d + m)
    p = {"macro.d_gain": torch.randn(R, K, d, generator=g) * 0.1, "macro.v": torch.randn(R, K, 3 * d, m, generator=g) * 0.05,
         "macro.u": torch.randn(R, K, m, d, generator=g) * 0.3, "macro.bias": torch.randn(R, K, d, generator=g) * 0.1}
    h0 = torch.randn(B, S, d, generator=g)
    rid, sid = torch.randint(0, R, (B,), generator=g), torch.randint(0, K, (B,), generator=g)
    rid[0] = rid[-1]
    sid[0] = sid[-1]                                          # at least one key shared by two samples
    dout = torch.randn(B, S, d, generator=g)
    leaves = {k: v.clone().requires_grad_(True) for k, v in p.items()}
    hr = h0.clone().requires_grad_(True)
    ref = O.macro_phi(leaves, cfg, hr, hr, rid, sid)
    ref.backward(dout)
    e = lambda *s: torch.zeros(*s, device=DEV)  # noqa: E731
    pd = dict(gain=p["macro.d_gain"].to(DEV), v=p["macro.v"].to(DEV), u=p["macro.u"].to(DEV), bias=p["macro.bias"].to(DEV),
              scale=torch.ones(R, K, d, device=DEV))
    out, rstd, pooled, act = e(B * S, d), e(B * S), e(B * d + B * m), e(B * S, m)
    ri, si = rid.to(DEV, torch.int32), sid.to(DEV, torch.int32)
    if tensor:
        pd["wt"] = e(R * K * 4 * d * m)
        ops.macro_phi_prepare(pd)
    ops.macro_phi_fwd(h0.to(DEV).view(B * S, d), pd, ri, si, 0.05, out, rstd, pooled, act, B=B, S=S, d=d, m=m, K=K)
    torch.cuda.synchronize()
    _close(out.view(B, S, d), ref, 1e-4, "phi out")
    dh0 = e(B * S, d)
    gr = dict(gain=e(R, K, d), v=e(R, K, 3 * d, m), u=e(R, K, m, d), bias=e(R, K, d))
    for t in gr.values():
        t.fill_(3.0)                                          # must be overwritten, including unused keys
    scratch = e(ops.phi_bwd_scratch_floats(B, S, d, m))
    ops.macro_phi_bwd(h0.to(DEV).view(B * S, d), dout.to(DEV).view(B * S, d), pd, ri, si, 0.05, rstd, pooled, act, dh0, gr,
                      scratch, B=B, S=S, d=d, m=m, R=R, K=K)
    torch.cuda.synchronize()
    _close(dh0.view(B, S, d), hr.grad, 2e-4, "phi dh0")
    _close(gr["gain"], leaves["macro.d_gain"].grad, 2e-4, "phi dgain")
    _close(gr["bias"], leaves["macro.bias"].grad, 2e-4, "phi dbias")
    _close(gr["u"], leaves["macro.u"].grad, 2e-4, "phi du")
    _close(gr["v"], leaves["macro.v"].grad, 2e-4, "phi dv")


@pytest.mark.parametrize("B,S,d,m,R,tensor", [(3, 16, 64, 8, 4, True), (2, 12, 40, 6, 3, False), (4, 64, 128, 32, 5, True),
                                              (2, 32, 96, 48, 3, True)])
def test_macro_phi_on_a_state_other_than_h0(ops, B, S, d, m, R, tensor):
    """Phi(h, h0) with h != h0 (the second application inside the consistency term, macro.py:342-359): output, the two
    separate data gradients (dh overwritten, dh0 accumulated into) and the parameter gradients against autograd."""
    K = 3
    cfg = O.ModelCfg(d_model=d, macro_rank=m, recipe_count=R, macro_update_scale=0.05)
    g = torch.Generator().manual_seed(d + m + 1)
    p = {"macro.d_gain": torch.randn(R, K, d, generator=g) * 0.1, "macro.v": torch.randn(R, K, 3 * d, m, generator=g) * 0.05,
         "macro.u": torch.randn(R, K, m, d, generator=g) * 0.3, "macro.bias": torch.randn(R, K, d, generator=g) * 0.1}
    h, h0 = torch.randn(B, S, d, generator=g), torch.randn(B, S, d, generator=g)
    rid, sid = torch.randint(0, R, (B,), generator=g), torch.randint(0, K, (B,), generator=g)
    rid[0], sid[0] = rid[-1], sid[-1]
    dout, seed0 = torch.randn(B, S, d, generator=g), torch.randn(B, S, d, generator=g)
    leaves = {k: v.clone().requires_grad_(True) for k, v in p.items()}
    hr, h0r = h.clone().requires_grad_(True), h0.clone().requires_grad_(True)
    ref = O.macro_phi(leaves, cfg, hr, h0r, rid, sid)
    ref.backward(dout)
    e = lambda *s: torch.zeros(*s, device=DEV)  # noqa: E731
    pd = dict(gain=p["macro.d_gain"].to(DEV), v=p["macro.v"].to(DEV), u=p["macro.u"].to(DEV), bias=p["macro.bias"].to(DEV),
              scale=torch.ones(R, K, d, device=DEV))
    out, rstd, pooled, act = e(B * S, d), e(B * S), e(B * d + B * m), e(B * S, m)
    ri, si = rid.to(DEV, torch.int32), sid.to(DEV, torch.int32)
    if tensor:
        pd["wt"] = e(R * K * 4 * d * m)
        ops.macro_phi_prepare(pd)
    hd, h0d = h.to(DEV).view(B * S, d), h0.to(DEV).view(B * S, d)
    ops.macro_phi_fwd_hx(hd, h0d, pd, ri, si, 0.05, out, rstd, pooled, act, B=B, S=S, d=d, m=m, K=K)
    torch.cuda.synchronize()
    _close(out.view(B, S, d), ref, 1e-4, "phi(h, h0) out")
    dh, dh0 = torch.full((B * S, d), 9.0, device=DEV), seed0.to(DEV).view(B * S, d).clone()
    gr = dict(gain=e(R, K, d), v=e(R, K, 3 * d, m), u=e(R, K, m, d), bias=e(R, K, d))
    scratch = e(ops.phi_bwd_scratch_floats(B, S, d, m))
    ops.macro_phi_bwd_hx(hd, h0d, dout.to(DEV).view(B * S, d), pd, ri, si, 0.05, rstd, pooled, act, dh, dh0, gr, scratch,
                         B=B, S=S, d=d, m=m, R=R, K=K)
    torch.cuda.synchronize()
    ops.check_status()
    _close(dh.view(B, S, d), hr.grad, 2e-4, "phi(h, h0) dh")
    _close(dh0.view(B, S, d), seed0 + h0r.grad, 2e-4, "phi(h, h0) dh0 (accumulated)")
    _close(gr["gain"], leaves["macro.d_gain"].grad, 2e-4, "phi(h, h0) dgain")
    _close(gr["bias"], leaves["macro.bias"].grad, 2e-4, "phi(h, h0) dbias")
    _close(gr["u"], leaves["macro.u"].grad, 2e-4, "phi(h, h0) du")
    _close(gr["v"], leaves["macro.v"].grad, 2e-4, "phi(h, h0) dv")


# ------------------------------------------------------------------ optimiser
def test_adamw_multi_tensor_matches_oracle_and_skips_absent(ops):
    from speedup_thingy_b200.ops import AdamWPlan
    g = torch.Generator().manual_seed(3)
    shapes = [(5000,), (37,), (128, 64), (4097,)]
    ps = [torch.randn(s, generator=g) for s in shapes]
    ref = [p.clone() for p in ps]
    ms, vs = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
    dev = [dict(p=p.to(DEV), g=torch.zeros_like(p, device=DEV), m=torch.zeros_like(p, device=DEV),
                v=torch.zeros_like(p, device=DEV), shadow=torch.zeros(p.shape, dtype=torch.bfloat16, device=DEV) if i == 2 else None,
                lr_group=i % 2) for i, p in enumerate(ps)]
    plan = AdamWPlan(dev, 2, DEV)
    lrs = [1e-2, 3e-3]
    plan.lr_table.copy_(torch.tensor(lrs))
    coef = torch.tensor([0.5], device=DEV)
    for step in range(1, 4):
        grads = [torch.randn(s, generator=g) for s in shapes]
        for e_, gr in zip(dev, grads):
            e_["g"].copy_(gr)
        ops.adamw(plan, 0.9, 0.999, 1e-8, 0.1, coef)
        for i, gr in enumerate(grads):
            O.adamw_update(ref[i], gr * 0.5, ms[i], vs[i], step, lrs[i % 2], 0.1)
    torch.cuda.synchronize()
    for i in range(len(ps)):
        _close(dev[i]["p"], ref[i], 1e-5, f"adamw tensor {i}")
    _close(dev[2]["shadow"], ref[2], 1e-2, "bf16 shadow")
    assert plan.step_count.tolist() == [3, 3, 3, 3]
    # global gradient norm + clip coefficient
    partial = torch.zeros(plan.total_chunks, device=DEV)
    sumsq, clip = torch.zeros(1, device=DEV), torch.zeros(1, device=DEV)
    ops.grad_norm(plan, partial, sumsq, 1.0, clip)
    torch.cuda.synchronize()
    tot = sum(float(e_["g"].double().pow(2).sum()) for e_ in dev)
    assert abs(float(sumsq) - tot) <= 1e-4 * tot
    assert abs(float(clip) - min(1.0, 1.0 / (math.sqrt(tot) + 1e-6))) < 1e-5


def test_adamw_skip_flag_metric_sums_and_nonfinite_guard(ops):
    """rte_adamw_multi_tensor_ex + rte_nonfinite_guard + rte_add_f32_guarded: a set flag makes the launch a no-op
    (training.py:448-452); the per-group sums feed the gradient metrics (training.py:386-443)."""
    from speedup_thingy_b200.ops import AdamWPlan
    g = torch.Generator().manual_seed(5)
    shapes = [(9000,), (130, 70), (4096,), (33,)]
    groups = [0, 2, 0, 1]
    ps = [torch.randn(s, generator=g) for s in shapes]
    gs = [torch.randn(s, generator=g) for s in shapes]
    dev = [dict(p=p.to(DEV), g=gr.to(DEV), m=torch.zeros_like(p, device=DEV), v=torch.zeros_like(p, device=DEV), shadow=None,
                lr_group=0, metric_group=mg) for p, gr, mg in zip(ps, gs, groups)]
    plan = AdamWPlan(dev, 1, DEV, n_metric_groups=3)
    plan.lr_table.fill_(1e-2)
    skip = torch.zeros(1, dtype=torch.int32, device=DEV)
    flag = torch.zeros(1, device=DEV)
    sums = torch.full((3, 2), -1.0, device=DEV)
    coef = torch.tensor([0.5], device=DEV)
    # guard: finite values -> 0, one NaN or inf in any range -> 1
    a, b, c = torch.randn(7, device=DEV), torch.randn(300, device=DEV), torch.randn(5, device=DEV)
    ops.nonfinite_guard([a, b, c], skip, flag)
    assert int(skip) == 0 and float(flag) == 0.0
    b[277] = float("inf")
    ops.nonfinite_guard([a, b, c], skip, flag)
    assert int(skip) == 1 and float(flag) == 1.0
    b[277] = 0.0
    c[4] = float("nan")
    ops.nonfinite_guard([a, None, c], skip, flag)
    assert int(skip) == 1
    # flagged: nothing moves, sums are zero
    ops.adamw(plan, 0.9, 0.999, 1e-8, 0.1, coef, skip=skip, metric_out=sums)
    torch.cuda.synchronize()
    for e_, p in zip(dev, ps):
        assert torch.equal(e_["p"].cpu(), p) and float(e_["m"].abs().max()) == 0.0
    assert plan.step_count.tolist() == [0, 0, 0, 0] and float(sums.abs().max()) == 0.0
    dst = torch.ones(1000, device=DEV)
    ops.add_guarded_(dst, torch.ones(1000, device=DEV), skip)
    assert float(dst.sum()) == 1000.0
    # not flagged: the ordinary update plus the sums of (0.5 g)^2 and p^2 (before the update) per metric group
    c[4] = 0.0
    ops.nonfinite_guard([a, b, c], skip, flag)
    ops.add_guarded_(dst, torch.ones(1000, device=DEV), skip)
    assert float(dst.sum()) == 2000.0
    ops.adamw(plan, 0.9, 0.999, 1e-8, 0.1, coef, skip=skip, metric_out=sums)
    torch.cuda.synchronize()
    ref = [p.clone() for p in ps]
    for i, gr in enumerate(gs):
        O.adamw_update(ref[i], gr * 0.5, torch.zeros_like(gr), torch.zeros_like(gr), 1, 1e-2, 0.1)
        _close(dev[i]["p"], ref[i], 1e-5, f"adamw_ex tensor {i}")
    assert plan.step_count.tolist() == [1, 1, 1, 1]
    for mg in range(3):
        g2 = sum(float((gr * 0.5).double().pow(2).sum()) for gr, k in zip(gs, groups) if k == mg)
        p2 = sum(float(p.double().pow(2).sum()) for p, k in zip(ps, groups) if k == mg)
        assert abs(float(sums[mg, 0]) - g2) <= 1e-5 * g2 and abs(float(sums[mg, 1]) - p2) <= 1e-5 * p2


def test_cpu_tensors_are_rejected(ops):
    with pytest.raises(RuntimeError, match="strict_cuda"):
        ops.gemm(torch.zeros(128, 64, dtype=torch.bfloat16), torch.zeros(128, 64, dtype=torch.bfloat16),
                 torch.zeros(128, 128, dtype=torch.bfloat16), M=128, N=128, K=64)


# ------------------------------------------------------------------ exact-audit helpers
def test_audit_distillation_terms_and_gradients(ops):
    n, S, d, V = 3, 16, 64, 200
    g = torch.Generator().manual_seed(77)
    h0 = torch.randn(n, S, d, generator=g)
    hot = (h0 + 0.3 * torch.randn(n, S, d, generator=g)).requires_grad_(True)
    exact = h0 + 0.3 * torch.randn(n, S, d, generator=g)
    hot_logits = _bf(torch.randn(n * S, V, generator=g) * 2)
    exact_logits = _bf(torch.randn(n * S, V, generator=g) * 2)
    tr = O.TrainCfg()
    hl = hot_logits.float().view(n, S, V).requires_grad_(True)
    aux = O.macro_distill_loss(tr, hot, exact, hl, exact_logits.float().view(n, S, V), h0)
    sum(aux.values()).backward()
    terms, dhot = torch.zeros(n, 4, device=DEV), torch.zeros(n * S, d, device=DEV)
    ops.macro_distill(hot.detach().to(DEV), exact.to(DEV), h0.to(DEV), tr.lambda_delta_dir, tr.lambda_delta_rms,
                      tr.lambda_endpoint_normed, tr.lambda_endpoint_raw, terms, dhot, n, S, d)
    B = 7
    idx = torch.tensor([1, 4, 6], dtype=torch.int32, device=DEV)
    dlog = torch.zeros(B * S, V, dtype=torch.bfloat16, device=DEV)
    kl_rows = torch.zeros(n * S, device=DEV)
    temp = tr.distill_temperature
    ops.kl_distill(hot_logits.to(DEV), exact_logits.to(DEV), temp, tr.lambda_kl * temp / n, idx, S, dlog, kl_rows, n * S, V)
    torch.cuda.synchronize()
    _close(dhot.view(n, S, d), hot.grad, 1e-3, "distill d hot")
    t = terms.cpu()
    assert abs(tr.lambda_delta_dir * float(t[:, 0].mean()) - float(aux["delta_dir"])) < 1e-4
    assert abs(tr.lambda_delta_rms * float(t[:, 1].mean()) - float(aux["delta_rms"])) < 1e-4
    assert abs(tr.lambda_endpoint_normed * float(t[:, 2].sum()) / (n * S * d) - float(aux["endpoint_normed"])) < 1e-4
    assert abs(tr.lambda_endpoint_raw * float(t[:, 3].sum()) / (n * S * d) - float(aux["endpoint_raw"])) < 1e-4
    assert abs(tr.lambda_kl * float(kl_rows.sum()) / n * temp * temp - float(aux["kl"])) < 1e-3 * max(1.0, float(aux["kl"]))
    rows = (idx.cpu().long()[:, None] * S + torch.arange(S)[None]).reshape(-1)
    _close(dlog.cpu()[rows], hl.grad.view(n * S, V), 2e-2, "KL gradient rows")
    others = torch.ones(B * S, dtype=torch.bool)
    others[rows] = False
    assert float(dlog.cpu()[others].abs().max()) == 0.0
    # the two-launch form (gradient kept apart, added to the dlogits afterwards) gives the same bits
    base = _bf(torch.randn(B * S, V, generator=g) * 0.01).to(DEV)
    fused, split = base.clone(), base.clone()
    ops.kl_distill(hot_logits.to(DEV), exact_logits.to(DEV), temp, tr.lambda_kl * temp / n, idx, S, fused, kl_rows, n * S, V)
    dsep, kl2 = torch.zeros(n * S, V, device=DEV), torch.zeros(n * S, device=DEV)
    kl1_side = torch.zeros(n * S, device=DEV)
    ops.kl_distill_grad(hot_logits.to(DEV), exact_logits.to(DEV), temp, tr.lambda_kl * temp / n, dsep, kl2, n * S, V,
                        kl1_rows=kl1_side)
    ops.add_rows_to_bf16(split, idx, S, dsep, n * S, V)
    torch.cuda.synchronize()
    assert torch.equal(fused, split) and torch.equal(kl_rows, kl2)
    # the temperature-1 KL of macro.py:538-543: as a by-product of that launch, and alone without a gradient buffer
    kl1 = torch.zeros(n * S, device=DEV)
    ops.kl_distill_grad(hot_logits.to(DEV), exact_logits.to(DEV), 1.0, 0.0, None, kl1, n * S, V)
    torch.cuda.synchronize()
    le, lh = torch.log_softmax(exact_logits.float(), -1), torch.log_softmax(hot_logits.float(), -1)
    _close(kl1, (le.exp() * (le - lh)).sum(-1), 1e-3, "KL rows at temperature 1")
    _close(kl1_side, (le.exp() * (le - lh)).sum(-1), 1e-3, "KL rows at temperature 1, by-product")


def test_audit_mask_and_residual_helpers(ops):
    g = torch.Generator().manual_seed(5)
    n, S, d, F_, R = 3, 8, 64, 128, 4
    rows = n * S
    rid = torch.tensor([2, 0, 3], dtype=torch.int32)
    tab = (torch.rand(R, d, generator=g) > 0.5).float() * 0.5
    x = _bf(torch.randn(rows, d, generator=g))
    out = torch.zeros(rows, d, dtype=torch.bfloat16, device=DEV)
    ops.colmask_mul(x.to(DEV), rid.to(DEV), tab.to(DEV), S, out, rows, d)
    _close(out, x.float() * tab[rid.long()].repeat_interleave(S, 0), 1e-2, "colmask")
    ftab = (torch.rand(R, F_, generator=g) > 0.5).float()
    ug = _bf(torch.randn(rows, 2 * F_, generator=g))
    z = torch.zeros(rows, F_, dtype=torch.bfloat16, device=DEV)
    ops.swiglu_masked_fwd(ug.to(DEV), rid.to(DEV), ftab.to(DEV), S, z, rows, F_)
    m = ftab[rid.long()].repeat_interleave(S, 0)
    ugr = ug.float().requires_grad_(True)
    zr = ugr[:, :F_] * F.silu(ugr[:, F_:]) * m
    _close(z, zr, 1e-2, "masked swiglu")
    dz = _bf(torch.randn(rows, F_, generator=g))
    zr.backward(dz.float())
    dug = torch.zeros(rows, 2 * F_, dtype=torch.bfloat16, device=DEV)
    ops.swiglu_masked_bwd(ug.to(DEV), dz.to(DEV), rid.to(DEV), ftab.to(DEV), S, dug, rows, F_)
    _close(dug, ugr.grad, 1e-2, "masked swiglu backward")
    # gather / scatter-add / routing
    Bn = 6
    src = torch.randn(Bn, S * d, generator=g)
    idx = torch.tensor([0, 3, 5], dtype=torch.int32, device=DEV)
    dst = torch.zeros(n, S * d, device=DEV)
    ops.gather_rows(src.to(DEV), idx, dst, n, S * d * 4)
    assert torch.equal(dst.cpu(), src[idx.cpu().long()])
    acc = src.clone().to(DEV)
    ops.scatter_add_rows(acc, idx, dst, n, S * d)
    ref = src.clone()
    ref[idx.cpu().long()] *= 2
    _close(acc, ref, 1e-6, "scatter add")
    by_pass = torch.randint(0, R, (Bn, 4), generator=g, dtype=torch.int32)
    depth = torch.tensor([1, 2, 4, 4, 1, 2], dtype=torch.int32)
    ro, ao = torch.zeros(4, n, dtype=torch.int32, device=DEV), torch.zeros(4, n, dtype=torch.int32, device=DEV)
    ops.audit_route(by_pass.to(DEV), depth.to(DEV), idx, ro, ao, n, 4)
    ii = idx.cpu().long()
    assert torch.equal(ro.cpu(), by_pass[ii].t().contiguous())
    assert torch.equal(ao.cpu(), (depth[ii][None] > torch.arange(4)[:, None]).int())
    # scaled residual forward / backward with a frozen sample
    base, br, pas = (torch.randn(n, S * d, generator=g) for _ in range(3))
    sc = torch.tensor([0.7])
    act = torch.tensor([1, 0, 1], dtype=torch.int32)
    o2 = torch.zeros(n, S * d, device=DEV)
    ops.scaled_residual_fwd(base.to(DEV), br.to(DEV), sc.to(DEV), act.to(DEV), pas.to(DEV), o2, n, S * d)
    on = act.view(n, 1) != 0
    _close(o2, torch.where(on, base + 0.7 * br, pas), 1e-6, "scaled residual")
    dout = torch.randn(n, S * d, generator=g)
    dbase, db32, dpas = torch.zeros(n, S * d, device=DEV), torch.ones(n, S * d, device=DEV), torch.ones(n, S * d, device=DEV)
    db16 = torch.zeros(n, S * d, dtype=torch.bfloat16, device=DEV)
    part = torch.zeros(64, device=DEV)
    ops.scaled_residual_bwd(dout.to(DEV), br.to(DEV), sc.to(DEV), act.to(DEV), dbase, db16, db32, dpas, part, n, S * d)
    torch.cuda.synchronize()
    zero = torch.zeros_like(dout)
    _close(dbase, torch.where(on, dout, zero), 1e-6, "d base")
    _close(db16, torch.where(on, 0.7 * dout, zero), 1e-2, "d branch bf16")
    _close(db32, 1 + torch.where(on, 0.7 * dout, zero), 1e-6, "d branch f32 accumulate")
    _close(dpas, 1 + torch.where(on, zero, dout), 1e-6, "d passthrough")
    assert abs(float(part.sum()) - float((torch.where(on, dout, zero) * br).sum())) < 1e-2
    # hand-through of frozen samples folded into the launch: dbase = dout + (frozen ? src : 0)
    src2 = torch.randn(n, S * d, generator=g)
    dbase2 = torch.zeros(n, S * d, device=DEV)
    ops.scaled_residual_bwd(dout.to(DEV), br.to(DEV), sc.to(DEV), None, dbase2, None, None, None, None, n, S * d,
                            frozen_active=act.to(DEV), frozen_src=src2.to(DEV))
    torch.cuda.synchronize()
    _close(dbase2, dout + torch.where(on, zero, src2), 1e-6, "d base with hand-through")


def test_audit_residual_clip_factors_and_row_scaling(ops):
    """rte_audit_clip / rte_scale_rows_bf16 against their definitions (audit.py:306-321): factors 1 - 1/p and 1 inside the
    clip, 1 and 0 outside; rows scaled through the sample index or in place order; untouched rows stay bit-identical."""
    from tests.emul_ops import EmulOps
    g = torch.Generator().manual_seed(5)
    B, n, S, V = 12, 5, 8, 72
    hot, exact = torch.randn(B, generator=g) + 40, torch.randn(n, generator=g) + 40
    idx = torch.tensor([1, 4, 6, 7, 11], dtype=torch.int32)
    exact[2] = hot[6] + 0.01                         # well inside
    f_hot, f_exact = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    ops.audit_clip(hot.to(DEV), exact.to(DEV), idx.to(DEV), n, 1.0 / 0.25, 0.5, f_hot, f_exact)
    r_hot, r_exact = torch.zeros(n), torch.zeros(n)
    EmulOps().audit_clip(hot, exact, idx, n, 1.0 / 0.25, 0.5, r_hot, r_exact)
    torch.cuda.synchronize()
    assert torch.equal(f_hot.cpu(), r_hot) and torch.equal(f_exact.cpu(), r_exact)
    assert r_exact[2] == 1.0 and r_hot[2] == -3.0 and set(r_exact.tolist()) == {0.0, 1.0}
    x = _bf(torch.randn(B * S, V + 8, generator=g))
    for use_idx in (True, False):
        got, want = x.clone().to(DEV), x.clone()
        ops.scale_rows_bf16(got, idx.to(DEV) if use_idx else None, S, f_hot, n * S, V)
        EmulOps().scale_rows_bf16(want, idx if use_idx else None, S, r_hot, n * S, V)
        torch.cuda.synchronize()
        assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("B,R,cap,n_cap,p_lo,p_hi,mode", [(128, 5, 6, 6, 0.05, 0.25, 1), (128, 5, None, 40, 0.05, 0.25, 1),
                                                         (64, 8, 3, 3, 0.3, 0.9, 0), (8, 5, None, 8, 0.0, 1.0, 1),
                                                         (32, 4, 40, 32, 0.1, 0.4, 1)])
def test_bernoulli_audit_sampler_matches_its_definition(ops, B, R, cap, n_cap, p_lo, p_hi, mode):
    """rte_audit_sample_bernoulli against the emulation (audit.py:62-132): probabilities with all three adaptive terms,
    the cap's thinning through the staged permutation table, per-slot outputs in ascending order with unused slots
    marked, both loss-weight vectors, the coverage average, the statistics; plus the two small kernels beside it."""
    from tests.emul_ops import EmulOps
    g = torch.Generator().manual_seed(B + R + n_cap)
    for trial in range(4):
        entropy = torch.rand(B, generator=g) * 2.5
        rid = torch.randint(0, R, (B,), generator=g).int()
        u = torch.rand(B, generator=g)
        ema0 = torch.rand(R, generator=g) * 0.02
        recent = torch.rand(1, generator=g) * 0.3
        perm = None
        if cap is not None and cap < B:
            perm = torch.stack([torch.randperm(c, generator=g)[:cap] for c in range(cap + 1, B + 1)]).int().reshape(-1)
        prm = dict(p_min=p_lo, p_max=p_hi, alpha=0.4, beta=0.5, gamma=0.3, coverage_min=0.01, coverage_beta=0.98,
                   inv_r_plus_k=1.0 / (R + 3), w0=1.0 / (B * 16), B=B, R=R, cap=-1 if (cap is None or cap >= B) else cap, n_cap=n_cap,
                   weight_mode=mode)

        def run(o, dev):
            t = lambda x: x.clone().to(dev)  # noqa: E731
            z = lambda n_, dt=torch.float32: torch.full((n_,), 7, dtype=dt, device=dev)  # noqa: E731
            out = dict(ema=t(ema0), idx=z(n_cap, torch.int32), idx_scatter=z(n_cap, torch.int32), valid=z(n_cap), inv_p=z(n_cap),
                       dist=z(n_cap), rw=z(B), rwa=z(n_cap), stats=z(4))
            o.audit_sample_bernoulli(t(entropy), t(rid), t(u), t(perm) if perm is not None else None, out["ema"], t(recent), prm,
                                     out["idx"], out["idx_scatter"], out["valid"], out["inv_p"], out["dist"], out["rw"],
                                     out["rwa"], out["stats"])
            return {k: v.cpu() for k, v in out.items()}

        got, emu = run(ops, DEV), EmulOps()
        emu.status = torch.zeros(1, dtype=torch.int32)
        want = run(emu, "cpu")
        torch.cuda.synchronize()
        ops.check_status()
        for k in ("idx", "idx_scatter", "valid"):
            assert torch.equal(got[k], want[k]), (k, trial, got[k], want[k])
        assert torch.equal(got["stats"][:2], want["stats"][:2]), (got["stats"], want["stats"])
        for k in ("inv_p", "dist", "rw", "rwa", "ema", "stats"):
            assert torch.allclose(got[k], want[k], rtol=1e-5, atol=1e-7), (k, trial, got[k], want[k])
    x = torch.randn(6, 200, generator=g)
    f = torch.tensor([1.0, 0.0, 2.5, 1.0, 0.0, 3.0])
    xd = x.clone().to(DEV)
    ops.scale_rows_f32(xd, f.to(DEV), 6, 200)
    assert torch.allclose(xd.cpu(), x * f[:, None])
    a, b_ = torch.randn(6, 300, generator=g), torch.randn(6, 300, generator=g)
    valid = torch.tensor([1.0, 1.0, 0.0, 1.0, 0.0, 0.0])
    rec, cosd = torch.full((1,), 0.5, device=DEV), torch.zeros(6, device=DEV)
    ops.audit_recent_residual(a.to(DEV), b_.to(DEV), valid.to(DEV), 6, 300, cosd, rec)
    cos = torch.nn.functional.cosine_similarity(a, b_, dim=-1, eps=1e-8)
    assert torch.allclose(rec.cpu(), (1 - (cos * valid).sum() / valid.sum()).clamp_min(0).view(1), atol=1e-5)
    ops.audit_recent_residual(a.to(DEV), b_.to(DEV), torch.zeros(6, device=DEV), 6, 300, cosd, rec)      # nobody audited: unchanged
    assert torch.allclose(rec.cpu(), (1 - (cos * valid).sum() / valid.sum()).clamp_min(0).view(1), atol=1e-5)


def test_adamw_leaves_tensors_without_a_gradient_alone(ops):
    """absent_flag + absent_mask of rte_adamw_multi_tensor_ex: while the flag is set the masked tensors keep their
    weights, moments and step counts (torch.optim.AdamW skips `grad is None`) and leave the metric sums; the other
    tensors step as usual; with the flag clear everything steps."""
    from speedup_thingy_b200.ops import AdamWPlan
    g = torch.Generator().manual_seed(9)
    shapes = [(3000,), (64, 65), (5000,)]
    ps = [torch.randn(s_, generator=g) for s_ in shapes]
    dev = [dict(p=p.clone().to(DEV), g=torch.randn(p.shape, generator=g).to(DEV), m=torch.zeros_like(p, device=DEV),
                v=torch.zeros_like(p, device=DEV), shadow=None, lr_group=0, metric_group=i % 2) for i, p in enumerate(ps)]
    plan = AdamWPlan(dev, 1, DEV, n_metric_groups=2)
    plan.lr_table.fill_(1e-2)
    mask = torch.tensor([0, 1, 0], dtype=torch.uint8, device=DEV)
    flag = torch.ones(1, dtype=torch.int32, device=DEV)
    sums = torch.zeros(2, 2, device=DEV)
    ops.adamw(plan, 0.9, 0.999, 1e-8, 0.1, None, metric_out=sums, absent_flag=flag, absent_mask=mask)
    torch.cuda.synchronize()
    assert torch.equal(dev[1]["p"].cpu(), ps[1]) and not dev[1]["m"].any() and not dev[1]["v"].any()
    assert not torch.equal(dev[0]["p"].cpu(), ps[0]) and not torch.equal(dev[2]["p"].cpu(), ps[2])
    assert plan.step_count.cpu().tolist() == [1, 0, 1]
    assert float(sums[1, 0]) == 0.0 and float(sums[0, 0]) > 0.0            # group 1 holds only the masked tensor
    flag.zero_()
    ops.adamw(plan, 0.9, 0.999, 1e-8, 0.1, None, metric_out=sums, absent_flag=flag, absent_mask=mask)
    torch.cuda.synchronize()
    assert not torch.equal(dev[1]["p"].cpu(), ps[1]) and plan.step_count.cpu().tolist() == [2, 1, 2]
    assert float(sums[1, 0]) > 0.0


@pytest.mark.parametrize("L", [64 * 96, 1001])          # 16-byte loads | scalar loads (length not a multiple of 4)
def test_alignment_sums_match_their_definition(ops, L):
    """rte_audit_alignment_sums (the seven per-sample sums behind macro_alignment_metrics, macro.py:499-546)."""
    from tests.emul_ops import EmulOps
    g = torch.Generator().manual_seed(4)
    n = 5
    a, b, z = (torch.randn(n, L, generator=g) for _ in range(3))
    got = torch.full((n, 8), 9.0, device=DEV)
    ops.audit_alignment_sums(a.to(DEV), b.to(DEV), z.to(DEV), n, L, got)
    want = torch.full((n, 8), 9.0)                                 # column 7 stays the caller's
    EmulOps().audit_alignment_sums(a, b, z, n, L, want)
    torch.cuda.synchronize()
    assert torch.allclose(got.cpu(), want, rtol=1e-4, atol=1e-2)
    assert torch.equal(got[:, 7].cpu(), torch.full((n,), 9.0))
