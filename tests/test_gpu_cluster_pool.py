"""Static cluster-pool sparse FFN on a B200 (`speedup_thingy_b200.cluster_pool`) against the oracle and the
reference-generated golden case: routing indices, deterministic packing, pooled forward, every gradient.
Tolerances: indices bit-exact (routing: wherever the fp32 score gap exceeds bf16 resolution); bf16 arithmetic
2e-2 of the output scale."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import rte_oracle as O
from speedup_thingy_b200.cluster_pool import StaticClusterPoolSwiGLU, cluster_pool_swiglu
from tests.golden.cases import cluster_pool_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = np.load(Path(__file__).resolve().parent / "golden" / "cluster_pool.npz")


def _module(t, max_tokens):
    wug, wd = t["wug"].to(DEV), t["wd"].to(DEV)
    return StaticClusterPoolSwiGLU(wug, wd, {"up_a": t["up_a"], "gate_a": t["gate_a"]},
                                   {"centers": t["centers"], "candidate_ids": t["candidate_ids"]},
                                   rank=t["up_a"].shape[1], max_tokens=max_tokens)


def _close(a, b, rel=2e-2):
    a, b = a.detach().float().cpu(), torch.as_tensor(b).float()
    assert a.shape == b.shape
    err = (a - b).abs().max().item()
    assert err <= rel * b.abs().max().item() + 1e-6, (err, b.abs().max().item())


def test_routing_matches_reference_where_scores_are_separated():
    t = cluster_pool_inputs()
    m = _module(t, 200)
    flat = t["x"].reshape(-1, 64).to(DEV)
    scores = torch.empty(200, 4, device=DEV)
    got = m.route(flat, scores).cpu().long()
    m.ops.check_status()
    ref_scores = torch.cat([flat.cpu() @ t["up_a"], flat.cpu() @ t["gate_a"]], dim=-1) @ t["centers"].t()
    top2 = ref_scores.topk(2, dim=-1).values
    separated = (top2[:, 0] - top2[:, 1]) > 2e-2 * ref_scores.abs().max()
    want = torch.from_numpy(GOLD["assignments"])
    assert separated.float().mean() > 0.8
    assert torch.equal(got[separated], want[separated])
    # the kernel's own arg-max is exact on its own scores, lowest index on ties
    assert torch.equal(got, O.argmax_lowest(scores.cpu()))


@pytest.mark.parametrize("n,C,pattern", [(200, 4, "golden"), (1000, 16, "random"), (777, 8, "one_cluster"),
                                          (4096, 16, "skewed"), (130, 64, "random")])
def test_pack_is_the_stable_counting_sort(n, C, pattern):
    from speedup_thingy_b200.ops import CudaOps
    ops = CudaOps(DEV)
    g = torch.Generator().manual_seed(n)
    if pattern == "golden":
        a = torch.from_numpy(GOLD["assignments"]).long()
    elif pattern == "one_cluster":
        a = torch.full((n,), C - 2)
    elif pattern == "skewed":
        a = (torch.rand(n, generator=g) ** 4 * C).long().clamp_(max=C - 1)
    else:
        a = torch.randint(0, C, (n,), generator=g)
    cap = -(-n // 128) * 128 + 128 * C
    i32 = dict(dtype=torch.int32, device=DEV)
    perm, pos = torch.empty(cap, **i32), torch.empty(n, **i32)
    counts, offsets, kb = torch.empty(C, **i32), torch.empty(C + 1, **i32), torch.empty(C + 1, **i32)
    tg = torch.empty(cap // 128, **i32)
    ops.cluster_pack(a.to(DEV, torch.int32), C, perm, pos, counts, offsets, tg, kb)
    ops.check_status()
    perm, pos, counts, offsets, kb, tg = (t_.cpu().long() for t_ in (perm, pos, counts, offsets, kb, tg))
    pack_index, flat_gather, ref_counts, _ = O.cluster_pack_indices(a, C)
    assert torch.equal(counts, ref_counts)
    assert (offsets % 128 == 0).all() and torch.equal(kb, offsets // 64)
    assert torch.equal(offsets[1:] - offsets[:-1], (ref_counts + 127) // 128 * 128)
    for c in range(C):
        rows = perm[offsets[c]: offsets[c + 1]]
        assert torch.equal(rows[: ref_counts[c]], pack_index[c, : ref_counts[c]])      # ascending token order
        assert (rows[ref_counts[c]:] == -1).all()
        assert (tg[offsets[c] // 128: offsets[c + 1] // 128] == c).all()
    assert (tg[offsets[C] // 128:] == -1).all() and (perm[offsets[C]:] == -1).all()
    assert torch.equal(perm[pos], torch.arange(n))


def test_forward_and_every_gradient_match_reference_golden():
    t = cluster_pool_inputs()
    m = _module(t, 256)
    x = t["x"].to(DEV).requires_grad_()
    m.wug.requires_grad_()
    m.wd.requires_grad_()
    assign = torch.from_numpy(GOLD["assignments"]).to(DEV, torch.int32)
    out = cluster_pool_swiglu(m, x, assign)
    (out * t["probe"].to(DEV)).sum().backward()
    m.ops.check_status()
    _close(out, GOLD["out"])
    _close(x.grad, GOLD["dx"])
    _close(m.wug.grad, GOLD["dwug"])
    _close(m.wd.grad, GOLD["dwd"])
    unused = torch.ones(128, dtype=torch.bool)
    unused[t["candidate_ids"].unique()] = False
    assert (m.wug.grad.cpu()[:128][unused] == 0).all()              # neurons in no pool: exact zeros


def test_full_pool_recovers_the_dense_ffn():
    """tests/test_kernels.py:82-106 of the reference: with every neuron in every pool the result is the dense FFN."""
    g = torch.Generator().manual_seed(2)
    d, F_, C = 64, 128, 2
    t = dict(wug=torch.randn(2 * F_, d, generator=g) * 0.1, wd=torch.randn(d, F_, generator=g) * 0.1,
             up_a=torch.randn(d, 4, generator=g), gate_a=torch.randn(d, 4, generator=g),
             centers=torch.randn(C, 8, generator=g), candidate_ids=torch.arange(F_).repeat(C, 1))
    m = _module(t, 300)
    x = torch.randn(300, d, generator=g).to(DEV)
    out = m.forward(x)
    dense = m.dense_forward(x)
    m.ops.check_status()
    _close(out, dense.cpu(), rel=1e-2)
    xr = x.cpu().bfloat16().float()
    wug, wd = t["wug"].bfloat16().float(), t["wd"].bfloat16().float()
    ref = ((xr @ wug[:F_].t()) * torch.nn.functional.silu(xr @ wug[F_:].t())) @ wd.t()
    _close(out, ref)


def test_c3_shaped_pools_against_the_oracle():
    """Stand-alone shape of the headline configuration: 8192 tokens, d 512, F 2048, 16 clusters of 512."""
    g = torch.Generator().manual_seed(3)
    N, d, F_, C, Mc, r = 8192, 512, 2048, 16, 512, 64
    t = dict(wug=torch.randn(2 * F_, d, generator=g) * 0.03, wd=torch.randn(d, F_, generator=g) * 0.03,
             up_a=torch.randn(d, r, generator=g) * 0.1, gate_a=torch.randn(d, r, generator=g) * 0.1,
             centers=torch.nn.functional.normalize(torch.randn(C, 2 * r, generator=g), dim=-1),
             candidate_ids=torch.stack([torch.randperm(F_, generator=g)[:Mc] for _ in range(C)]))
    m = _module(t, N)
    x = torch.randn(N, d, generator=g)
    xg = x.to(DEV).requires_grad_()
    m.wug.requires_grad_()
    m.wd.requires_grad_()
    out = cluster_pool_swiglu(m, xg)
    probe = torch.randn(N, d, generator=g)
    (out * probe.to(DEV)).sum().backward()
    m.ops.check_status()
    assign = m.assign[:N].cpu().long()
    assert torch.bincount(assign, minlength=C).min() > 0
    xr = x.bfloat16().float().requires_grad_()
    wug, wd = t["wug"].bfloat16().float().requires_grad_(), t["wd"].bfloat16().float().requires_grad_()
    ref, _ = O.static_cluster_pool_swiglu(xr, wug, wd, t["up_a"], t["gate_a"], t["centers"], t["candidate_ids"], assign)
    (ref * probe).sum().backward()
    _close(out, ref.detach())
    _close(xg.grad, xr.grad)
    _close(m.wug.grad, wug.grad)
    _close(m.wd.grad, wd.grad)
