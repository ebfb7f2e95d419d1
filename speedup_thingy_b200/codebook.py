"""Offline build of the cluster-pool codebook on the GPU: what the reference does on the CPU before the static
cluster-pool FFN can run (src/recursive_training_engine/cli.py:3244-3261 SVD factor cache, 3297-3323 cosine k-means,
3326-3351 per-cluster score aggregation, 3357-3389 selector features and pool scores, 4703-4782 the calibration
loop, 4914-4941 capped active union).

The calibration activations (the FFN's normed inputs) stay on the device; every product is a tcgen05 GEMM, the
k-means assignment is `rte_cluster_route`, the centre update and the score aggregation are fixed-order reductions
(`rte_kmeans_update`, `rte_cluster_aggregate`), the per-cluster candidate lists come from `rte_topk_lowest_index`.
The truncated SVD of the two weight halves stays on the host (`torch.linalg.svd`, once per refresh, as in the
reference): it is a dense factorisation of two d x F matrices, not part of any per-token path.

The result -- ``dict(centers [C, 2r], candidate_ids [C, M])`` -- is what ``StaticClusterPoolSwiGLU.update_codebook``
consumes.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _abi as A
from .ops import CudaOps, _ptr

SCORE_MODES = {"sum": 0, "upgate": 1, "product": 2}


def svd_factor_cache(wug: torch.Tensor, max_rank: int, device) -> dict[str, torch.Tensor]:
    """cli.py:3244-3261 for one layer: `up_a`/`gate_a` = U[:, :r] * S[:r] ([d, r]), `up_b`/`gate_b` = Vh[:r, :] ([r, F])
    of the transposed up / gate halves of the fused W_ug [2F, d].  Host SVD, factors returned on `device`."""
    up_w, gate_w = wug.detach().float().cpu().chunk(2, dim=0)
    out: dict[str, torch.Tensor] = {}
    for name, mat in (("up", up_w.t().contiguous()), ("gate", gate_w.t().contiguous())):
        u, s, vh = torch.linalg.svd(mat, full_matrices=False)
        r = min(max_rank, s.numel())
        out[f"{name}_a"] = (u[:, :r] * s[:r]).to(device)
        out[f"{name}_b"] = vh[:r, :].contiguous().to(device)
    return out


class CodebookBuilder:
    """Launch sequences of the codebook build over one device (`ops`: the C-ABI operator table)."""

    def __init__(self, ops: CudaOps):
        self.ops = ops
        self.dev = ops.device

    # ------------------------------------------------------------------ selector features and pool scores
    def features_and_scores(self, normed: torch.Tensor, factors: dict, wd: torch.Tensor, *, rank: int,
                            score_mode: str = "sum") -> tuple[torch.Tensor, torch.Tensor]:
        """cli.py:3357-3389.  normed [..., d] (the FFN's normed input, any float dtype), wd [d, F] (the down projection,
        whose column norms weight the scores).  Returns features f32 [n, 2r] = [q_up | q_gate] and scores f32 [n, F]."""
        o, dev, bf, f32 = self.ops, self.dev, torch.bfloat16, torch.float32
        flat = normed.reshape(-1, normed.shape[-1])
        n, d = flat.shape
        F = wd.shape[1]
        r = min(max(1, int(rank)), factors["up_a"].shape[1], factors["gate_a"].shape[1])
        if d % 8 or r % 8 or F % 8:
            raise ValueError("kernel limits: d_model, rank and d_ff must be multiples of 8")
        x16 = flat.to(bf).contiguous()
        sel16 = torch.cat([factors["up_a"][:, :r], factors["gate_a"][:, :r]], dim=1).to(dev, bf).contiguous()      # [d, 2r]
        feats = torch.empty(n, 2 * r, dtype=f32, device=dev)
        o.gemm(x16, sel16, feats, M=n, N=2 * r, K=d, b_mn=True, epilogue=A.EPI_F32)
        q16 = torch.empty(n, 2 * r, dtype=bf, device=dev)
        o.cast_bf16(feats, q16)
        hats = torch.empty(2, n, F, dtype=f32, device=dev)
        for j, name in enumerate(("up_b", "gate_b")):
            b16 = factors[name][:r, :].to(dev, bf).contiguous()                                                   # [r, F]
            o.gemm(q16[:, j * r:(j + 1) * r], b16, hats[j], M=n, N=F, K=r, b_mn=True, epilogue=A.EPI_F32, lda=2 * r)
        wd_norm = torch.empty(F, dtype=f32, device=dev)
        o.row_norm(wd.detach().float().t().contiguous().to(dev), wd_norm)          # ||wd[:, j]||: rows of wd^T
        scores = torch.empty(n, F, dtype=f32, device=dev)
        o._call("rte_cluster_pool_scores", _ptr(hats[0]), _ptr(hats[1]), _ptr(wd_norm), _ptr(scores), n, F,
                SCORE_MODES[score_mode], o.stream)
        return feats, scores

    # ------------------------------------------------------------------ cosine k-means
    def fit_centers(self, features: torch.Tensor, cluster_count: int, iters: int) -> tuple[torch.Tensor, torch.Tensor]:
        """cli.py:3297-3323.  features f32 [n, W] on the device.  Returns (assignments int32 [n], centers f32 [C, W])."""
        o, dev, f32 = self.ops, self.dev, torch.float32
        n, W = features.shape
        Cn = min(max(1, int(cluster_count)), max(1, n))
        if W > 256:
            raise ValueError("kernel limit: feature width (2 * rank) <= 256")
        x = torch.empty(n, W, dtype=f32, device=dev)
        o._call("rte_normalize_rows_f32", _ptr(features.contiguous()), _ptr(x), n, W, o.stream)
        assign = torch.zeros(n, dtype=torch.int32, device=dev)
        if Cn == 1 or n == 1:
            mean = x.mean(dim=0, keepdim=True).contiguous()
            centers = torch.empty_like(mean)
            o._call("rte_normalize_rows_f32", _ptr(mean), _ptr(centers), 1, W, o.stream)
            return assign, centers
        init_idx = torch.linspace(0, n - 1, steps=Cn).round().long().to(dev)
        centers = x.index_select(0, init_idx).contiguous()
        nxt = torch.empty_like(centers)
        for _ in range(max(1, int(iters))):
            o.cluster_route(x, centers, assign)
            o._call("rte_kmeans_update", _ptr(x), _ptr(assign), _ptr(centers), _ptr(nxt), None, n, W, Cn, o.stream)
            centers, nxt = nxt, centers
        return assign, centers

    # ------------------------------------------------------------------ the codebook of one layer
    def build(self, features: torch.Tensor, scores: torch.Tensor, *, cluster_count: int, candidate_m: int,
              aggregation: str = "mean", iters: int = 8) -> dict[str, torch.Tensor]:
        """cli.py:4741-4771: centres from the calibration features; candidate ids = the `candidate_m` best neurons of
        every cluster by aggregated pool score, best first, ties to the lowest index (the reference leaves the tie
        order to torch.topk)."""
        if aggregation not in ("mean", "max"):
            raise ValueError(f"unsupported cluster score aggregation: {aggregation}")
        o, dev = self.ops, self.dev
        assign, centers = self.fit_centers(features, cluster_count, iters)
        Cn, (n, F) = centers.shape[0], scores.shape
        agg = torch.empty(Cn, F, dtype=torch.float32, device=dev)
        o._call("rte_cluster_aggregate", _ptr(scores.contiguous()), _ptr(assign), _ptr(agg), n, F, Cn, int(aggregation == "max"), o.stream)
        m = min(int(candidate_m), F)
        ids = torch.empty(Cn, m, dtype=torch.int32, device=dev)
        o.topk_lowest_index(agg, m, ids)
        sizes = torch.bincount(assign.long(), minlength=Cn).float()
        nonempty = sizes[sizes > 0]
        return dict(centers=centers, candidate_ids=ids.long(), assignments=assign, aggregate=agg,
                    nonempty_clusters=int(nonempty.numel()),
                    cluster_imbalance=float(nonempty.max() / nonempty.mean().clamp_min(1.0)) if nonempty.numel() else 0.0)


def active_union_ids(candidate_ids: torch.Tensor, hidden: int, cap: int | None = None) -> torch.Tensor:
    """cli.py:4914-4941: the sorted union of every cluster's candidates; above `cap`, the `cap` best ids by the
    frequency-plus-rank score (weights 1 .. 1/M along each cluster's list), ties to the lowest id.  Index
    bookkeeping on a few thousand integers: plain tensor operations on whatever device the ids live on."""
    ids = candidate_ids.long()
    full = torch.unique(ids.reshape(-1), sorted=True)
    if cap is None or int(cap) <= 0 or full.numel() <= int(cap):
        return full
    cap = min(int(cap), hidden)
    c, m = ids.shape
    weight = torch.linspace(1.0, 1.0 / max(m, 1), steps=m, device=ids.device).unsqueeze(0).expand(c, m).reshape(-1)
    score = torch.zeros(hidden, device=ids.device).index_add_(0, ids.reshape(-1), weight)
    order = torch.sort(-score.double(), stable=True).indices[:cap]        # (score desc, id asc)
    return torch.sort(order).values
