"""Static cluster-pool sparse SwiGLU FFN on the sm_100a kernels: the counterpart of the reference's
``StaticClusterPoolSwiGLU`` (layers.py:119-220) and ``kernels/cluster_pool_ffn.py``.

What the reference does per forward -- route tokens to fixed centres, build pack/gather indices in a Python loop
over clusters, gather the pool weights, pad every cluster to the largest one, three ``bmm``s, gather back
(cluster_pool_ffn.py:162-211) -- becomes here, with no host synchronisation and no routing-dependent shape:

  route   GEMM x @ [up_a | gate_a] (tcgen05) + ``rte_cluster_route`` (arg-max, lowest index on ties)
  pack    ``rte_cluster_pack``: stable counting sort into one row order whose clusters start on 128-row
          boundaries (capacity = tokens rounded up to 128, plus 128 rows per cluster)
  pools   ``rte_gather_rows`` of the bf16 weight rows named by ``candidate_ids`` (the dense weights stay the
          trainable source of truth, so this is redone every forward exactly as the reference does)
  FFN     two grouped ``rte_gemm_bf16`` launches (tile -> cluster table) with the SwiGLU pass between them
  grads   grouped data-gradient GEMMs, ragged split-K weight-gradient GEMMs (one split per cluster), and a
          CSR gather-reduce of pool rows into dense rows (``scatter_cluster_pool_grads`` without atomics)

There is no CPU path: the constructor needs a CUDA device and the built library.
"""
from __future__ import annotations

import torch

from . import _abi as A
from .ops import CudaOps


def _csr_by_dense_row(dense_rows: torch.Tensor, n_dense: int) -> tuple[torch.Tensor, torch.Tensor]:
    """CSR over dense rows f -> the pool-slot indices whose dense row is f, slots in ascending order (the fixed
    summation order of the gradient reduce).  Host work, done once per codebook."""
    order = torch.argsort(dense_rows, stable=True)
    counts = torch.bincount(dense_rows, minlength=n_dense)
    row_ptr = torch.zeros(n_dense + 1, dtype=torch.int64)
    row_ptr[1:] = counts.cumsum(0)
    return row_ptr.to(torch.int32), order.to(torch.int32)


class StaticClusterPoolSwiGLU:
    """wug [2F, d] (up rows | gate rows) and wd [d, F] are fp32 CUDA tensors owned by the caller (the dense FFN's
    parameters); ``factors`` = {"up_a", "gate_a"} [d, r...], ``codebook`` = {"centers" [C, 2r], "candidate_ids"
    [C, Mc]} as in layers.py:150-186.  ``max_tokens`` fixes the buffer sizes."""

    def __init__(self, wug: torch.Tensor, wd: torch.Tensor, factors: dict, codebook: dict, *, rank: int,
                 max_tokens: int, ops: CudaOps | None = None):
        if not wug.is_cuda or not wd.is_cuda:
            raise RuntimeError("strict_cuda: StaticClusterPoolSwiGLU needs CUDA tensors (no CPU or Triton path)")
        self.ops = ops if ops is not None else CudaOps(wug.device)
        self.wug, self.wd = wug, wd
        self.d, self.F = wd.shape
        if wug.shape != (2 * self.F, self.d):
            raise ValueError("wug must be [2*d_ff, d_model] and wd [d_model, d_ff]")
        self.max_tokens = int(max_tokens)
        self.update_codebook(factors, codebook, rank=rank)

    # ------------------------------------------------------------------ codebook (layers.py:150-186)
    def update_codebook(self, factors: dict, codebook: dict, *, rank: int | None = None) -> None:
        dev, d, F = self.wug.device, self.d, self.F
        r = min(max(1, int(rank if rank is not None else self.rank)), factors["up_a"].shape[1], factors["gate_a"].shape[1])
        self.rank = r
        ids = codebook["candidate_ids"].detach().to("cpu", torch.int64)
        centers = codebook["centers"].detach().float()
        self.C, self.Mc = ids.shape
        if centers.shape != (self.C, 2 * r):
            raise ValueError("centers must be [clusters, 2*rank]")
        if d % 8 or self.Mc % 64 or (2 * r) % 8:
            raise ValueError("kernel limits: d_model % 8 == 0, candidate pool size % 64 == 0, 2*rank % 8 == 0")
        if int(ids.min()) < 0 or int(ids.max()) >= F:
            raise ValueError("candidate_ids out of range")
        C, Mc, bf, f32, i32 = self.C, self.Mc, torch.bfloat16, torch.float32, torch.int32
        # selector as a GEMM operand: rows = selector features, K-major
        self.selector16 = torch.cat([factors["up_a"][:, :r], factors["gate_a"][:, :r]], dim=1).t().contiguous().to(dev, bf)
        self.centers = centers.to(dev).contiguous()
        self.candidate_ids = ids.to(dev)
        # pool row -> dense row, for the weight gathers ...
        up_rows = ids.reshape(C, Mc)
        self.idx_ug = torch.cat([up_rows, up_rows + F], dim=1).reshape(-1).to(dev, i32)          # [C * 2Mc] rows of wug
        self.idx_d = ids.reshape(-1).to(dev, i32)                                                  # [C * Mc] rows of wd^T
        # ... and dense row -> pool rows, for the gradient reduce (fixed order)
        ptr, order = _csr_by_dense_row(torch.cat([up_rows, up_rows + F], dim=1).reshape(-1), 2 * F)
        self.csr_ug = (ptr.to(dev), order.to(dev))
        ptr, order = _csr_by_dense_row(ids.reshape(-1), F)
        self.csr_d = (ptr.to(dev), order.to(dev))
        # buffers (sizes depend on max_tokens and the codebook only, never on the routing)
        N = self.max_tokens
        self.cap = -(-N // 128) * 128 + 128 * C
        e = lambda *s, dtype=bf: torch.empty(*s, dtype=dtype, device=dev)  # noqa: E731
        self.wug16, self.wdT16 = e(2 * F, d), e(F, d)
        self.wug_pool, self.wd_pool = e(C * 2 * Mc, d), e(C * Mc, d)
        self.q = e(N, 2 * r, dtype=f32)
        self.assign, self.pos = e(N, dtype=i32), e(N, dtype=i32)
        self.perm, self.tile_group = e(self.cap, dtype=i32), e(self.cap // 128, dtype=i32)
        self.counts, self.offsets, self.kblocks = e(C, dtype=i32), e(C + 1, dtype=i32), e(C + 1, dtype=i32)
        self.x16 = e(N, d)
        self.xp, self.ugp, self.zp = e(self.cap, d), e(self.cap, 2 * Mc), e(self.cap, Mc)
        self.yp = e(self.cap, d, dtype=f32)
        self.dyp, self.dzp, self.dugp = e(self.cap, d), e(self.cap, Mc), e(self.cap, 2 * Mc)
        self.dxp = e(self.cap, d, dtype=f32)
        self.dwug_pool, self.dwd_pool = e(C * 2 * Mc, d, dtype=f32), e(C * Mc, d, dtype=f32)
        self.dwdT = e(F, d, dtype=f32)
        self._tokens = 0

    # ------------------------------------------------------------------ routing / packing
    def route(self, x: torch.Tensor, scores: torch.Tensor | None = None) -> torch.Tensor:
        """assignments int32 [tokens] (route_to_static_centers, cluster_pool_ffn.py:127-139)."""
        o, N = self.ops, x.shape[0]
        o.cast_bf16(x, self.x16[:N]) if x.dtype == torch.float32 else self.x16[:N].copy_(x)
        o.gemm(self.x16[:N], self.selector16, self.q[:N], M=N, N=2 * self.rank, K=self.d, epilogue=A.EPI_F32)
        o.cluster_route(self.q[:N], self.centers, self.assign[:N], scores)
        return self.assign[:N]

    def pack(self, assignments: torch.Tensor) -> None:
        """Fills perm / pos / tile_group / kblocks for `assignments` (build_static_pack_gather_indices)."""
        self.ops.cluster_pack(assignments, self.C, self.perm, self.pos[: assignments.numel()], self.counts, self.offsets,
                              self.tile_group, self.kblocks)

    def prepare_pools(self) -> None:
        """bf16 pool weights from the current dense weights (prepare_cluster_pool_weights, cluster_pool_ffn.py:90-124)."""
        o = self.ops
        o.cast_bf16(self.wug, self.wug16)
        o.transpose(self.wd, self.wdT16)
        o.gather_rows(self.wug16, self.idx_ug, self.wug_pool, self.idx_ug.numel(), self.d * 2)
        o.gather_rows(self.wdT16, self.idx_d, self.wd_pool, self.idx_d.numel(), self.d * 2)

    # ------------------------------------------------------------------ forward / backward
    def forward(self, x: torch.Tensor, assignments: torch.Tensor | None = None) -> torch.Tensor:
        """x [..., d] fp32 or bf16 on the device -> fp32 [..., d].  `assignments` (int32 [tokens]) overrides the
        router, as cluster_pool_ffn_forward_from_assignments does."""
        if not x.is_cuda:
            raise RuntimeError("strict_cuda: StaticClusterPoolSwiGLU needs CUDA tensors (no CPU or Triton path)")
        o, d, Mc, C = self.ops, self.d, self.Mc, self.C
        flat = x.reshape(-1, d).contiguous()
        N = flat.shape[0]
        if N > self.max_tokens:
            raise ValueError(f"{N} tokens exceed max_tokens={self.max_tokens}")
        self._tokens = N
        a = self.route(flat) if assignments is None else assignments.to(torch.int32).contiguous()
        self.pack(a)
        self.prepare_pools()
        o.gather_rows_convert(flat, self.perm, self.xp)                                   # pack + cast, zero padding rows
        grp = dict(tile_group=self.tile_group, n_groups=C)
        o.gemm(self.xp, self.wug_pool, self.ugp, M=self.cap, N=2 * Mc, K=d, b_group_stride=2 * Mc, **grp)
        # pooled (up | gate) per cluster: columns [0, Mc) = up, [Mc, 2Mc) = gate of the cluster's candidates
        o.swiglu_fwd(self.ugp, self.zp, self.cap, Mc)
        o.gemm(self.zp, self.wd_pool, self.yp, M=self.cap, N=d, K=Mc, b_mn=True, epilogue=A.EPI_F32,
               b_group_stride=Mc, **grp)
        out = torch.empty(N, d, dtype=torch.float32, device=x.device)
        o.gather_rows_convert(self.yp, self.pos[:N], out)
        return out.view(*x.shape[:-1], d)

    def backward(self, dout: torch.Tensor, dwug: torch.Tensor, dwd: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
        """Gradients of the last forward: returns dx fp32 and writes (or adds) the dense weight gradients
        dwug [2F, d], dwd [d, F] (rows of neurons outside every used pool receive exact zeros)."""
        o, d, Mc, C, N = self.ops, self.d, self.Mc, self.C, self._tokens
        grp = dict(tile_group=self.tile_group, n_groups=C)
        o.gather_rows_convert(dout.reshape(-1, d).contiguous(), self.perm, self.dyp)
        o.gemm(self.dyp, self.wd_pool, self.dzp, M=self.cap, N=Mc, K=d, b_group_stride=Mc, **grp)
        o.swiglu_bwd(self.ugp, self.dzp, self.dugp, self.cap, Mc)
        o.gemm(self.dugp, self.wug_pool, self.dxp, M=self.cap, N=d, K=2 * Mc, b_mn=True, epilogue=A.EPI_F32,
               b_group_stride=2 * Mc, **grp)
        # per-cluster weight gradients: the reduction runs over the cluster's packed rows (ragged split-K)
        o.gemm(self.zp, self.dyp, self.dwd_pool, M=Mc, N=d, K=self.cap, a_mn=True, b_mn=True, epilogue=A.EPI_F32,
               splits=C, split_stride=Mc * d, split_kblocks=self.kblocks, ldc=d)
        o.gemm(self.dugp, self.xp, self.dwug_pool, M=2 * Mc, N=d, K=self.cap, a_mn=True, b_mn=True, epilogue=A.EPI_F32,
               splits=C, split_stride=2 * Mc * d, split_kblocks=self.kblocks, ldc=d)
        o.csr_row_reduce(self.dwug_pool, *self.csr_ug, dwug, accumulate)
        o.csr_row_reduce(self.dwd_pool, *self.csr_d, self.dwdT, False)
        o.transpose(self.dwdT, dwd, accumulate)
        dx = torch.empty(N, d, dtype=torch.float32, device=dout.device)
        o.gather_rows_convert(self.dxp, self.pos[:N], dx)
        return dx.view(dout.shape)

    def dense_forward(self, x: torch.Tensor) -> torch.Tensor:
        """The un-pooled FFN (layers.py:184-186) through the same GEMM kernel, for comparisons."""
        o, d, F = self.ops, self.d, self.F
        flat = x.reshape(-1, d).contiguous()
        N = flat.shape[0]
        x16 = flat.to(torch.bfloat16)
        o.cast_bf16(self.wug, self.wug16)
        wd16 = self.wd.to(torch.bfloat16)
        ug = torch.empty(N, 2 * F, dtype=torch.bfloat16, device=x.device)
        z = torch.empty(N, F, dtype=torch.bfloat16, device=x.device)
        out = torch.empty(N, d, dtype=torch.float32, device=x.device)
        o.gemm(x16, self.wug16, ug, M=N, N=2 * F, K=d)
        o.swiglu_fwd(ug, z, N, F)
        o.gemm(z, wd16, out, M=N, N=d, K=F, epilogue=A.EPI_F32)
        return out.view(*x.shape[:-1], d)


class _ClusterPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wug, wd, module, assignments):
        ctx.module = module
        return module.forward(x.detach(), assignments)

    @staticmethod
    def backward(ctx, dout):
        m = ctx.module
        dwug, dwd = torch.empty_like(m.wug), torch.empty_like(m.wd)
        dx = m.backward(dout.contiguous(), dwug, dwd)
        return dx, dwug, dwd, None, None


def cluster_pool_swiglu(module: StaticClusterPoolSwiGLU, x: torch.Tensor, assignments: torch.Tensor | None = None) -> torch.Tensor:
    """Autograd entry point: gradients flow to x and to the module's dense wug / wd."""
    return _ClusterPoolFn.apply(x, module.wug, module.wd, module, assignments)
