"""The drop-in operator table (`speedup_thingy_b200.kernels`, the counterpart of the reference's
`kernels/optimized.py`) on a B200: outputs against the reference-generated per-op golden vectors
(`tests/golden/per_op.npz`, inputs regenerated from the same seed) and against the oracle's fp32 restatements,
gradients against autograd through those restatements.  Tolerances: fp32 operators 1e-4, bf16 operators 2e-2 of
the output scale."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import rte_oracle as O
from speedup_thingy_b200 import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = np.load(Path(__file__).resolve().parent / "golden" / "per_op.npz")


def _golden_inputs():
    """Same draws, in the same order, as tests/golden/make_golden.py::per_op_vectors."""
    g = torch.Generator().manual_seed(11)
    x, w = torch.randn(3, 5, 24, generator=g), torch.randn(24, generator=g)
    q, k, v = (torch.randn(2, 3, 7, 8, generator=g) for _ in range(3))
    logits = torch.randn(4, 6, 17, generator=g)
    tg = torch.randint(0, 17, (4, 6), generator=g)
    return x, w, q, k, v, logits, tg


def _close(a, b, rel, abs_=0.0):
    a, b = a.detach().float().cpu(), torch.as_tensor(b).float()
    assert a.shape == b.shape
    err = (a - b).abs().max().item()
    assert err <= rel * b.abs().max().item() + abs_, err


def test_rmsnorm_matches_reference_golden_and_grads():
    x, w, *_ = _golden_inputs()
    xg, wg = x.to(DEV).requires_grad_(), w.to(DEV).requires_grad_()
    out, summed = K.k_fused_rmsnorm(xg, wg)
    assert summed is None
    _close(out, GOLD["rmsnorm"], 1e-5, 1e-5)
    xr, wr = x.clone().requires_grad_(), w.clone().requires_grad_()
    ref = O.rmsnorm(xr, wr)
    probe = torch.randn_like(ref)
    (ref * probe).sum().backward()
    (out * probe.to(DEV)).sum().backward()
    _close(xg.grad, xr.grad, 1e-4, 1e-5)
    _close(wg.grad, wr.grad, 1e-4, 1e-5)


def test_rmsnorm_with_residual_returns_sum_and_routes_both_grads():
    g = torch.Generator().manual_seed(3)
    x, r, w = torch.randn(4, 9, 64, generator=g), torch.randn(4, 9, 64, generator=g), torch.randn(64, generator=g)
    leaves = [t.to(DEV).requires_grad_() for t in (x, r, w)]
    out, summed = K.k_fused_rmsnorm(leaves[0], leaves[2], leaves[1])
    ref_leaves = [t.clone().requires_grad_() for t in (x, r, w)]
    y = ref_leaves[0] + ref_leaves[1]
    ref = O.rmsnorm(y, ref_leaves[2])
    _close(out, ref, 1e-5, 1e-5)
    _close(summed, y, 1e-6, 1e-6)
    (ref.sum() + (y * y).sum()).backward()
    (out.sum() + (summed * summed).sum()).backward()
    for a, b in zip(leaves, ref_leaves):
        _close(a.grad, b.grad, 1e-4, 1e-5)
    assert torch.equal(leaves[0].detach().cpu(), x)            # inputs untouched


def test_rope_matches_reference_golden_and_is_orthogonal():
    _, _, q, k, *_ = _golden_inputs()
    cos, sin = O.rope_tables(7, 8)
    qg, kg = q.to(DEV).requires_grad_(), k.to(DEV).requires_grad_()
    rq, rk = K.k_rope_apply(qg, kg, cos.to(DEV), sin.to(DEV))
    _close(rq, GOLD["rope_q"], 1e-5, 1e-6)
    _close(rk, GOLD["rope_k"], 1e-5, 1e-6)
    probe = torch.randn(2, 3, 7, 8, generator=torch.Generator().manual_seed(1))
    ((rq + 2 * rk) * probe.to(DEV)).sum().backward()
    qr = q.clone().requires_grad_()
    (O.rope_apply(qr, cos, sin) * probe).sum().backward()
    _close(qg.grad, qr.grad, 1e-5, 1e-6)
    _close(kg.grad, 2 * qr.grad, 1e-5, 1e-6)             # the rotation is linear: d/dk of 2*rope(k) = 2 * adjoint(probe)
    # bf16 data path
    rq16, _ = K.k_rope_apply(q.to(DEV).bfloat16(), k.to(DEV).bfloat16(), cos.to(DEV), sin.to(DEV))
    assert rq16.dtype == torch.bfloat16
    _close(rq16, GOLD["rope_q"], 2e-2)


@pytest.mark.parametrize("B,H,S,hd", [(2, 3, 7, 8), (3, 4, 64, 64), (2, 2, 130, 32)])
def test_flash_causal_dense_output_and_grads(B, H, S, hd):
    if (B, H, S, hd) == (2, 3, 7, 8):
        _, _, _, _, v, *_ = _golden_inputs()
        q, k = torch.from_numpy(GOLD["rope_q"]), torch.from_numpy(GOLD["rope_k"])
    else:
        g = torch.Generator().manual_seed(S)
        q, k, v = (torch.randn(B, H, S, hd, generator=g) for _ in range(3))
    leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
    out = K.k_flash_causal_grouped(*leaves)
    ref_leaves = [t.bfloat16().float().requires_grad_() for t in (q, k, v)]
    ref = O.causal_attention(*ref_leaves)
    if (B, H, S, hd) == (2, 3, 7, 8):
        _close(out, GOLD["attn"], 2e-2)
    _close(out, ref, 2e-2)
    probe = torch.randn(B, H, S, hd, generator=torch.Generator().manual_seed(2))
    (ref * probe).sum().backward()
    (out * probe.to(DEV)).sum().backward()
    for a, b in zip(leaves, ref_leaves):
        _close(a.grad, b.grad, 3e-2)


def test_cross_entropy_matches_reference_golden_and_grads():
    *_, logits, tg = _golden_inputs()
    lg = logits.to(DEV).requires_grad_()
    loss = K.k_cross_entropy_unreduced(lg, tg.to(DEV))
    assert loss.shape == tg.shape
    _close(loss, GOLD["ce"], 2e-2)
    lr = logits.bfloat16().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lr.flatten(0, 1), tg.flatten(), reduction="none").view_as(tg)
    wgt = torch.rand(4, 6, generator=torch.Generator().manual_seed(4)) + 0.5
    (ref * wgt).sum().backward()
    (loss * wgt.to(DEV)).sum().backward()
    _close(lg.grad, lr.grad, 2e-2)


def test_logits_full_qkv_dense_and_out_proj_grouped():
    g = torch.Generator().manual_seed(5)
    h, W = torch.randn(3, 40, 64, generator=g), torch.randn(96, 64, generator=g) * 0.2
    hg, Wg = h.to(DEV).requires_grad_(), W.to(DEV).requires_grad_()
    out = K.k_logits_full(hg, Wg)
    hr, Wr = h.bfloat16().float().requires_grad_(), W.bfloat16().float().requires_grad_()
    ref = hr @ Wr.t()
    _close(out, ref, 2e-2)
    probe = torch.randn(3, 40, 96, generator=g)
    (ref * probe.bfloat16().float()).sum().backward()
    (out * probe.to(DEV)).sum().backward()
    _close(hg.grad, hr.grad, 2e-2)
    _close(Wg.grad, Wr.grad, 2e-2)

    wq, wk, wv = (torch.randn(64, 48, generator=g) * 0.2 for _ in range(3))
    outs = K.k_qkv_dense(h.to(DEV), wq.to(DEV), wk.to(DEV), wv.to(DEV))
    for o, w in zip(outs, (wq, wk, wv)):
        _close(o, h.bfloat16().float() @ w.bfloat16().float(), 2e-2)

    wo = (torch.randn(64, 40, generator=g) * 0.2)
    rows = torch.tensor([8, 9, 10, 11, 12, 13, 14, 15, 40, 41, 42, 43, 44, 45, 46, 47])
    x = torch.randn(5, 7, 16, generator=g)
    xg, wog = x.to(DEV).requires_grad_(), wo.to(DEV).requires_grad_()
    out = K.k_out_proj_grouped(xg, wog, rows.to(DEV))
    xr, wor = x.bfloat16().float().requires_grad_(), wo.bfloat16().float().requires_grad_()
    ref = xr @ wor[rows, :]
    _close(out, ref, 2e-2)
    ref.sum().backward()
    out.sum().backward()
    _close(xg.grad, xr.grad, 2e-2)
    _close(wog.grad, wor.grad, 2e-2)
    assert (wog.grad.cpu()[:8] == 0).all()                    # unselected rows get an exact zero


def test_logits_shortlist_shape_values_and_grads():
    g = torch.Generator().manual_seed(6)
    h, W = torch.randn(2, 33, 64, generator=g), torch.randn(96, 64, generator=g) * 0.2
    sl = torch.stack([torch.randperm(96, generator=g)[:16] for _ in range(66)]).view(2, 33, 16)
    hg, Wg = h.to(DEV).requires_grad_(), W.to(DEV).requires_grad_()
    out = K.k_logits_shortlist(hg, Wg, sl.to(DEV))
    assert out.shape == (2, 33, 16)
    hr, Wr = h.bfloat16().float().requires_grad_(), W.bfloat16().float().requires_grad_()
    ref = (hr.unsqueeze(-2) * Wr[sl]).sum(-1)
    _close(out, ref, 2e-2)
    probe = torch.randn(2, 33, 16, generator=g).bfloat16().float()
    (ref * probe).sum().backward()
    (out * probe.to(DEV)).sum().backward()
    _close(hg.grad, hr.grad, 2e-2)
    _close(Wg.grad, Wr.grad, 2e-2)


def test_strict_cuda_and_status_contract():
    with pytest.raises(RuntimeError, match="strict_cuda"):
        K.k_fused_rmsnorm(torch.randn(2, 3, 4), torch.ones(4))
    st = K.backend_status()
    assert st["mode"] == "cuda_sm100a_ext" and st["uses_reference_fallback"] is False and st["cuda_available"]
    K.cuda_required()
    with pytest.raises(RuntimeError, match="strict_cuda"):
        K.k_swiglu_dense(torch.randn(4, 8), torch.randn(8, 8), torch.randn(8, 8), torch.randn(8, 8))
    with pytest.raises(ValueError):
        K.k_fused_rmsnorm(torch.randn(2, 8, device=DEV), torch.ones(4, device=DEV))


@pytest.mark.parametrize("N,d,m", [(50, 64, 64), (1500, 128, 192), (40, 64, 24)])
def test_packed_swiglu_ffn_matches_reference_math_and_grads(N, d, m):
    g = torch.Generator().manual_seed(N)
    x, wug, wdr = torch.randn(N, d, generator=g), torch.randn(2 * m, d, generator=g) * 0.2, torch.randn(m, d, generator=g) * 0.2
    L = [t.to(DEV).requires_grad_() for t in (x, wug, wdr)]
    out = K.triton_packed_swiglu_ffn(*L)
    R = [t.bfloat16().float().requires_grad_() for t in (x, wug, wdr)]
    up, gate = (R[0] @ R[1].t()).chunk(2, dim=-1)
    ref = (up * torch.nn.functional.silu(gate)) @ R[2]
    _close(out, ref, 2e-2)
    probe = torch.randn(N, d, generator=g)
    (ref * probe).sum().backward()
    (out * probe.to(DEV)).sum().backward()
    for a, b in zip(L, R):
        _close(a.grad, b.grad, 3e-2)
    with pytest.raises(ValueError):
        K.packed_swiglu_ffn(L[0], L[1][:-1], L[2])


def test_active_union_swiglu_evaluates_only_the_active_rows():
    g = torch.Generator().manual_seed(8)
    d, F_ = 64, 256
    x, wug, wd = torch.randn(3, 20, d, generator=g), torch.randn(2 * F_, d, generator=g) * 0.2, torch.randn(d, F_, generator=g) * 0.2
    ids = torch.randperm(F_, generator=g)[:64].repeat(2)             # duplicates collapse (layers.py:262)
    L = [t.to(DEV).requires_grad_() for t in (x, wug, wd)]
    out = K.active_union_swiglu(L[0], L[1], L[2], ids.to(DEV))
    R = [t.bfloat16().float().requires_grad_() for t in (x, wug, wd)]
    u = torch.unique(ids)
    ref = ((R[0] @ R[1][u].t()) * torch.nn.functional.silu(R[0] @ R[1][u + F_].t())) @ R[2].t()[u]
    _close(out, ref, 2e-2)
    ref.sum().backward()
    out.sum().backward()
    _close(L[1].grad, R[1].grad, 3e-2)
    _close(L[2].grad, R[2].grad, 3e-2)
    inactive = torch.ones(F_, dtype=torch.bool)
    inactive[u] = False
    assert (L[1].grad.cpu()[:F_][inactive] == 0).all()


def _ref_leaves(*ts):
    return [t.bfloat16().float().requires_grad_() for t in ts]


def test_swiglu_dense_and_grouped_match_reference_math_and_grads():
    """k_swiglu_dense / k_swiglu_grouped (kernels/reference.py:62-78), weights stored [in, out]."""
    g = torch.Generator().manual_seed(21)
    x, wu, wg, wd = (torch.randn(3, 20, 64, generator=g), torch.randn(64, 128, generator=g) * 0.2,
                     torch.randn(64, 128, generator=g) * 0.2, torch.randn(128, 64, generator=g) * 0.2)
    slabs = torch.cat([torch.arange(32, 64), torch.arange(96, 128)])
    for fn, extra, ref_fn in ((K.k_swiglu_dense, (), lambda X, U, G, D: (X @ U) * torch.nn.functional.silu(X @ G) @ D),
                              (K.k_swiglu_grouped, (slabs,),
                               lambda X, U, G, D: (X @ U[:, slabs]) * torch.nn.functional.silu(X @ G[:, slabs]) @ D[slabs, :])):
        L = [t.to(DEV).requires_grad_() for t in (x, wu, wg, wd)]
        out = fn(*L, *[e.to(DEV) for e in extra])
        R = _ref_leaves(x, wu, wg, wd)
        ref = ref_fn(*R)
        _close(out, ref, 2e-2)
        probe = torch.randn(ref.shape, generator=g)
        (ref * probe).sum().backward()
        (out * probe.to(DEV)).sum().backward()
        for a, b in zip(L, R):
            _close(a.grad, b.grad, 2.5e-2, 1e-4)


def test_qkv_grouped_matches_reference_math_and_grads():
    g = torch.Generator().manual_seed(22)
    x = torch.randn(2, 16, 64, generator=g)
    ws = [torch.randn(64, 64, generator=g) * 0.2 for _ in range(3)]
    cols = torch.cat([torch.arange(16, 32), torch.arange(48, 64)])
    L = [t.to(DEV).requires_grad_() for t in (x, *ws)]
    outs = K.k_qkv_grouped(*L, cols.to(DEV))
    R = _ref_leaves(x, *ws)
    refs = [R[0] @ w[:, cols] for w in R[1:]]
    probe = torch.randn(refs[0].shape, generator=g)
    for o, r in zip(outs, refs):
        _close(o, r, 2e-2)
    sum((r * probe).sum() for r in refs).backward()
    sum((o * probe.to(DEV)).sum() for o in outs).backward()
    for a, b in zip(L, R):
        _close(a.grad, b.grad, 2.5e-2, 1e-4)


def test_macro_phi_simplified_form_matches_reference_math():
    """k_macro_phi (kernels/reference.py:111-124)."""
    g = torch.Generator().manual_seed(23)
    B, S, d, m = 3, 16, 64, 16
    h, h0 = torch.randn(B, S, d, generator=g), torch.randn(B, S, d, generator=g)
    d_gain, bias = torch.randn(d, generator=g) * 0.1, torch.randn(d, generator=g) * 0.1
    v, u = torch.randn(3 * d, m, generator=g) * 0.1, torch.randn(m, d, generator=g) * 0.1
    out = K.k_macro_phi(*[t.to(DEV) for t in (h, h0, d_gain, v, u, bias)])
    normed = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5)
    z = torch.cat([normed, normed.mean(1, keepdim=True).expand_as(normed), h0], dim=-1)
    ref = h + d_gain * h + torch.nn.functional.silu(z @ v) @ u + bias
    _close(out, ref, 2e-2)


def test_pack_by_recipe_round_trip_and_grads():
    """k_pack_by_recipe / k_unpack_from_recipe (kernels/reference.py:91-108): stable order by (recipe, depth, audited)."""
    g = torch.Generator().manual_seed(24)
    hidden = torch.randn(10, 6, 8, generator=g)
    recipe = torch.tensor([2, 0, 1, 2, 0, 1, 1, 0, 2, 0])
    depth = torch.tensor([1, 2, 1, 1, 2, 0, 1, 1, 0, 2])
    hg = hidden.to(DEV).requires_grad_()
    packed = K.k_pack_by_recipe(hg, recipe.to(DEV), depth.to(DEV))
    keys = recipe * 1_000_000 + depth * 10
    order = torch.sort(keys, stable=True).indices
    assert torch.equal(packed.permutation.cpu(), order)
    assert torch.equal(packed.packed.detach().cpu(), hidden[order])
    assert torch.equal(packed.keys.cpu(), keys[order])
    assert packed.offsets[-1].item() == 10 and packed.unique_keys.numel() == packed.offsets.numel() - 1
    back = K.k_unpack_from_recipe(packed.packed, packed.inverse_permutation)
    assert torch.equal(back.detach().cpu(), hidden)
    probe = torch.randn(10, 6, 8, generator=g)
    (packed.packed * probe.to(DEV)).sum().backward()
    want = torch.empty_like(probe)
    want[order] = probe
    assert torch.equal(hg.grad.cpu(), want)
    mask = K.k_sample_audit_mask(torch.full((64,), 0.25, device=DEV), 5)
    assert mask.dtype == torch.bool and mask.shape == (64,)
