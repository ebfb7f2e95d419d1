"""Stand-alone timing of the step's memory-bound kernels against their algorithmic bytes
(`python bench.py --probe-kernels`): one JSON line per kernel with its duration, the bytes one launch has to move,
the achieved GB/s and the fraction of the measured HBM copy bandwidth.

Shapes are those of BASELINE configs[2] (8192 tokens, d 512, F 2048, V 2048, 8 heads, batch 128 x 64).  Every
kernel runs from a CUDA graph of `iters` launches that rotate over enough operand sets to exceed the 126 MB L2, so the
figures are DRAM figures; the same command under `ncu -k regex:<kernel> -c 1` gives the per-kernel DRAM counters.
"""
from __future__ import annotations

import json

import torch

from . import _abi as A
from .ops import AdamWPlan, CudaOps

L2_BYTES = 126 * 1024 * 1024


def _time(fn, n_sets: int, iters: int, warmup: int) -> float:
    """Microseconds per launch of fn(i) (i = operand set), measured over a CUDA graph of `iters` launches."""
    for i in range(max(warmup, 1)):
        fn(i % n_sets)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i % n_sets)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def _sets(bytes_per_set: int) -> int:
    return max(2, -(-2 * L2_BYTES // max(bytes_per_set, 1)))


def probe_kernels(iters: int, warmup: int, hbm_gbs: float) -> None:
    dev = "cuda:0"
    o = CudaOps(dev)
    B, S, d, F, V, H = 128, 64, 512, 2048, 2048, 8
    M, hd = B * S, d // H
    f32, bf, i32, i64 = torch.float32, torch.bfloat16, torch.int32, torch.int64
    r = lambda *s, dtype=f32: torch.randn(*s, device=dev).to(dtype)         # noqa: E731
    z = lambda *s, dtype=f32: torch.zeros(*s, device=dev, dtype=dtype)      # noqa: E731

    def report(name: str, us: float, nbytes: float, note: str = "") -> None:
        gbs = nbytes / us / 1e3
        print(json.dumps({"kernel": name, "us": round(us, 2), "algorithmic_MB": round(nbytes / 1e6, 2), "GBps": round(gbs, 1),
                          "frac_of_hbm_peak": round(gbs / hbm_gbs, 3), "note": note}), flush=True)

    # ---- RMSNorm forward: x f32 read, y bf16 + rstd written
    nb = M * d * 4 + M * d * 2 + M * 4
    n = _sets(nb)
    x, w, y, rs = [r(M, d) for _ in range(n)], r(d), [z(M, d, dtype=bf) for _ in range(n)], [z(M) for _ in range(n)]
    report("rmsnorm_fwd_kernel", _time(lambda i: o.rmsnorm_fwd(x[i], w, y[i], rs[i]), n, iters, warmup), nb)
    # ---- RMSNorm backward: x f32, dy bf16, dres f32 read; dx f32 + dx bf16 written (+ column partials)
    nb = M * d * (4 + 2 + 4 + 4 + 2)
    dy, dres, dx, dx16 = [r(M, d, dtype=bf) for _ in range(n)], [r(M, d) for _ in range(n)], [z(M, d) for _ in range(n)], [z(M, d, dtype=bf) for _ in range(n)]
    part, dw = z(8 * 148, d), z(d)
    report("rmsnorm_bwd_kernel (+colsum)", _time(lambda i: o.rmsnorm_bwd(x[i], w, rs[i], dy[i], dres[i], dx[i], dx16[i], dw, part), n, iters, warmup), nb)
    del x, y, dy, dres, dx, dx16
    # ---- cross entropy: logits bf16 read twice (max/sum, gradient), gradient written over them
    nb = M * V * 2 * 2
    n = _sets(M * V * 2)
    lg = [r(M, V, dtype=bf) for _ in range(n)]
    tg, rw, lt = torch.randint(0, V, (M,), device=dev), torch.full((B,), 1.0 / M, device=dev), z(M)
    report("ce_kernel", _time(lambda i: o.ce_fwd_bwd(lg[i], tg, rw, S, lt, lg[i]), n, iters, warmup), nb, "read 2V + write 2V bytes per token")
    del lg
    # ---- SwiGLU element-wise passes (the un-fused path): 6F / 10F bytes per row
    n = _sets(M * F * 6)
    ug, zz, dz, dug = [r(M, 2 * F, dtype=bf) for _ in range(n)], [z(M, F, dtype=bf) for _ in range(n)], [r(M, F, dtype=bf) for _ in range(n)], [z(M, 2 * F, dtype=bf) for _ in range(n)]
    report("swiglu_fwd_kernel", _time(lambda i: o.swiglu_fwd(ug[i], zz[i], M, F), n, iters, warmup), M * F * 6)
    report("swiglu_bwd_kernel", _time(lambda i: o.swiglu_bwd(ug[i], dz[i], dug[i], M, F), n, iters, warmup), M * F * 10)
    del ug, zz, dz, dug
    # ---- attention forward / backward (S = 64, 8 heads of 64): qkv read, y + lse written; backward reads qkv, y, dy, lse
    n = _sets(M * 3 * d * 2 * 2)
    qkv, yy, lse = [r(M, 3 * d, dtype=bf) for _ in range(n)], [z(M, d, dtype=bf) for _ in range(n)], [z(B * H * S) for _ in range(n)]
    dyy, dqkv = [r(M, d, dtype=bf) for _ in range(n)], [z(M, 3 * d, dtype=bf) for _ in range(n)]
    o.rope_table(S, hd)
    us = _time(lambda i: o.attn_fwd(qkv[i], yy[i], lse[i], B=B, S=S, n_heads=H, head_dim=hd), n, iters, warmup)
    report("attn fwd_kernel", us, M * 3 * d * 2 + M * d * 2 + B * H * S * 4, f"{4.0 * S * d * M / us / 1e6:.1f} TFLOP/s (QK^T + PV, causal counted as full)")
    us = _time(lambda i: o.attn_bwd(qkv[i], yy[i], dyy[i], lse[i], dqkv[i], B=B, S=S, n_heads=H, head_dim=hd), n, iters, warmup)
    report("attn bwd_kernel", us, M * 3 * d * 2 * 2 + M * d * 2 * 2 + B * H * S * 4, f"{10.0 * S * d * M / us / 1e6:.1f} TFLOP/s (5 products)")
    del qkv, yy, dyy, dqkv
    # ---- embedding gather and its reproducible scatter-add
    emb = r(V, d)
    n = _sets(M * d * 4)
    toks = [torch.randint(0, V, (M,), device=dev) for _ in range(n)]
    xo, dxs = [z(M, d) for _ in range(n)], [r(M, d) for _ in range(n)]
    demb, acc = z(V, d), torch.zeros(V * d, dtype=i64, device=dev)
    report("embed_fwd_kernel", _time(lambda i: o.embed_fwd(toks[i], emb, xo[i]), n, iters, warmup), M * d * 4 * 2 + M * 8)
    report("embed_bwd (accumulate + apply)", _time(lambda i: o.embed_bwd(toks[i], dxs[i], demb, acc), n, iters, warmup),
           M * d * 4 + V * d * (8 * 2 + 4), "dx read + int64 accumulator read/write + table write")
    del xo, dxs
    # ---- AdamW over 15.7 M parameters in 40 tensors (28 B per parameter + 2 B bf16 shadow on the GEMM weights)
    shapes = [(V, d)] + [(3 * d, d), (d, d), (2 * F, d), (d, F), (d,), (d,)] * 4
    ents = [dict(p=r(*s), g=r(*s), m=z(*s), v=z(*s), shadow=z(*s, dtype=bf) if len(s) == 2 else None, lr_group=0, metric_group=0)
            for s in shapes]
    plan = AdamWPlan(ents, 1, dev, n_metric_groups=1)
    plan.lr_table.fill_(1e-3)
    n_par = sum(e["p"].numel() for e in ents)
    n_sh = sum(e["p"].numel() for e in ents if e["shadow"] is not None)
    report("adamw_kernel", _time(lambda i: o.adamw(plan, 0.9, 0.999, 1e-8, 0.1, None), 1, iters, warmup), n_par * 28 + n_sh * 2,
           f"{n_par / 1e6:.1f} M parameters; operands exceed L2 ({n_par * 16 / 1e6:.0f} MB resident)")
    sk, ms_ = torch.zeros(1, dtype=i32, device=dev), z(1, 2)
    report("adamw_kernel (skip flag + metric sums)", _time(lambda i: o.adamw(plan, 0.9, 0.999, 1e-8, 0.1, None, skip=sk, metric_out=ms_), 1, iters, warmup),
           n_par * 28 + n_sh * 2)
    gp, ssq, cl = z(plan.total_chunks), z(1), z(1)
    report("gradnorm_partial_kernel (+final)", _time(lambda i: o.grad_norm(plan, gp, ssq, 1.0, cl), 1, iters, warmup), n_par * 4)
    del ents, plan
    # ---- router: mean-pool read of h0 dominates (B*S*d*4 bytes) + the two small MLPs
    hid, R, K, T = 512, 5, 3, 4
    n = _sets(M * d * 4)
    h0 = [r(M, d) for _ in range(n)]
    wts = dict(r_w0=r(hid, d) * 0.02, r_b0=z(hid), r_w2=r(R, hid) * 0.02, r_b2=z(R), d_w0=r(hid, d) * 0.02, d_b0=z(hid),
               d_w2=r(K, hid) * 0.02, d_b2=z(K), pass_recipe_bias=z(T, R))
    route = dict(pooled=z(B, d), r_hidden_pre=z(B, hid), d_hidden_pre=z(B, hid), recipe_logits=z(B, R), recipe_probs=z(B, R),
                 depth_probs=z(B, K), expected_depth=z(B), router_entropy=z(B), recipe_id=z(B, dtype=i32),
                 recipe_id_by_pass=z(B, T, dtype=i32), depth_id=z(B, dtype=i32), depth=z(B, dtype=i32))
    dv = torch.tensor([1, 2, 4], dtype=i32, device=dev)
    report("router_fwd (pool + hidden + heads)", _time(lambda i: o.router_fwd(h0[i], wts, dv, route, B=B, S=S, d=d, hid=hid, R=R, K=K, T=T,
                                                                                 fixed_recipe=None, fixed_depth_id=None), n, iters, warmup),
           M * d * 4 + 2 * hid * d * 4, "pooled read of h0 + first-layer weights")
    del h0
    # ---- top-k (ties to the lowest index): cluster logits [M, 64] -> top 2; hidden-unit scores [M, 2048] -> top 256
    sc = [r(M, 64) for _ in range(_sets(M * 64 * 4))]
    idx = z(M, 2, dtype=i32)
    report("topk_kernel n=64 k=2", _time(lambda i: o.topk_lowest_index(sc[i], 2, idx), len(sc), iters, warmup), M * 64 * 4 + M * 2 * 4)
    del sc
    # ---- shortlist build (c4 head: V 2048, 64 clusters, top 2, 32 hard + 32 random negatives, 128 slots)
    Ms = 128 * 128
    tc_ = torch.randint(0, 64, (Ms, 2), device=dev, dtype=i32)
    rn = torch.randint(0, V, (Ms, 32), device=dev, dtype=i32)
    tgs = torch.randint(0, V, (Ms,), device=dev)
    sl, dups = z(Ms, 128, dtype=i32), z(Ms, dtype=i32)
    report("shortlist_build_kernel", _time(lambda i: o.shortlist_build(tgs, tc_, rn, sl, dups, V=V, C=64, TC=2, HN=32, RN=32, K=128), 1, iters, warmup),
           Ms * (8 + 2 * 4 + 32 * 4 + 128 * 4 + 4), "16384 tokens; reads target + top clusters + random negatives, writes 128 ids")
    hid16, w16 = r(Ms, d, dtype=bf), (r(V, d) * 0.02).to(bf)
    rw2, lt2 = torch.full((128,), 1.0 / Ms, device=dev), z(Ms)
    dl = [z(Ms, V, dtype=bf) for _ in range(3)]
    report("shortlist_ce_kernel", _time(lambda i: o.shortlist_ce(hid16, w16, sl, rw2, 128, lt2, None, dl[i]), 3, iters, warmup),
           Ms * (d * 2 + 128 * 4 + V * 2), "hidden + ids read, dense dlogits row written (gathered weight rows stay in L2)")
    o.check_status()
