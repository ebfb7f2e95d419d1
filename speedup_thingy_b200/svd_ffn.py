"""SVD-factor sparse SwiGLU FFN on the sm_100a kernels: the counterpart of the reference's ``SVDFactorSparseFFN``
in mask and slots mode (layers.py:342-643) and of ``triton_svd_sparse_ffn_forward`` (svd_sparse_ffn_triton.py:480-714).

The reference scores all F neurons with two low-rank products, takes three top-m lists, gathers the candidate
weight rows per token (``w_up[candidate_ids]``: an [N, candidates, d] tensor), evaluates them exactly, re-ranks
and sums the selected ``w_down`` rows.  On a B200 the exact pre-activations of ALL neurons are one tensor-core
GEMM that costs less than the per-token row gather, so the same result is computed as

  selector  x @ [up_a | gate_a] -> q;  q_up @ up_b, q_gate @ gate_b -> hats            (tcgen05 GEMMs)
  exact     x @ [w_up ; w_gate]^T -> (up | gate) for every neuron                        (tcgen05 GEMM)
  select    ``rte_svd_ffn_select``: the three candidate lists, the exact re-rank, z_masked (one warp per token)
  down      z_masked @ w_down                                                            (tcgen05 GEMM)

and the backward pass is the dense backward restricted to the selected neurons.  The selected set is the
reference's whenever the scores agree (ties: lowest index).  No CPU path.
"""
from __future__ import annotations

import torch

from . import _abi as A
from .ops import CudaOps


class SVDFactorSparseFFN:
    """Parameters as in the reference module: w_up, w_gate, w_down [d_ff, d_model] (fp32 CUDA, owned by the caller),
    factors up_a / gate_a [d_model, rank], up_b / gate_b [rank, d_ff]."""

    def __init__(self, w_up, w_gate, w_down, up_a, up_b, gate_a, gate_b, *, top_k: int, up_m: int,
                 gate_m: int | None = None, product_m: int = 0, max_tokens: int, ops: CudaOps | None = None,
                 candidate_mode: str = "mask"):
        # "mask" (layers.py:473-502) keeps the union of the three candidate lists as a mask, "slots" (layers.py:504-527)
        # as their concatenation with first occurrences valid: the same SET of candidates as long as no token falls
        # short of top_k of them -- which the limit below rules out (one list alone holds top_k distinct neurons) -- so
        # both modes select the same neurons and give the same output (the reference's own two outputs are equal on
        # the golden inputs, tests/golden/svd_ffn.npz); only the reported slot count differs
        if candidate_mode not in ("mask", "slots"):
            raise NotImplementedError(f"candidate_mode={candidate_mode!r}: 'mask' and 'slots' are implemented "
                                      "(the Triton path of the reference is not translated)")
        self.candidate_mode = candidate_mode
        if not (w_up.is_cuda and w_gate.is_cuda and w_down.is_cuda):
            raise RuntimeError("strict_cuda: SVDFactorSparseFFN needs CUDA tensors (no CPU or Triton path)")
        self.ops = ops if ops is not None else CudaOps(w_up.device)
        self.w_up, self.w_gate, self.w_down = w_up, w_gate, w_down
        self.F, self.d = w_up.shape
        F, d = self.F, self.d
        self.rank = up_a.shape[1]
        self.top_k = min(max(1, int(top_k)), F)
        self.up_m = min(max(0, int(up_m)), F)
        self.gate_m = self.up_m if gate_m is None else min(max(0, int(gate_m)), F)
        self.product_m = min(max(0, int(product_m)), F)
        if max(self.up_m, self.gate_m, self.product_m) < self.top_k:
            raise NotImplementedError("max(up_m, gate_m, product_m) >= top_k is required (with fewer candidates than "
                                      "top_k the reference's result depends on an unspecified ordering)")
        r = self.rank
        if d % 8 or F % 8 or r % 8:
            raise ValueError("kernel limits: d_model, d_ff and rank must be multiples of 8")
        dev, bf, f32 = w_up.device, torch.bfloat16, torch.float32
        self.selector16 = torch.cat([up_a, gate_a], dim=1).t().contiguous().to(dev, bf)        # [2r, d]
        self.up_b16, self.gate_b16 = up_b.contiguous().to(dev, bf), gate_b.contiguous().to(dev, bf)   # [r, F]
        N = self.max_tokens = int(max_tokens)
        e = lambda *s, dtype=bf: torch.empty(*s, dtype=dtype, device=dev)  # noqa: E731
        self.wug16, self.wd16, self.wn = e(2 * F, d), e(F, d), e(F, dtype=f32)
        self.x16, self.q16 = e(N, d), e(N, 2 * r)
        self.hats = e(N, 2 * F, dtype=f32)
        self.ug, self.z = e(N, 2 * F), e(N, F)
        self.selected = e(N, F, dtype=torch.uint8)
        self.cand_count = e(N, dtype=torch.int32)
        self.dout16, self.dz, self.dug = e(N, d), e(N, F), e(N, 2 * F)
        self.dwug = e(2 * F, d, dtype=f32)
        self._tokens = 0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("strict_cuda: SVDFactorSparseFFN needs CUDA tensors (no CPU or Triton path)")
        o, d, F, r = self.ops, self.d, self.F, self.rank
        flat = x.reshape(-1, d).contiguous()
        N = self._tokens = flat.shape[0]
        if N > self.max_tokens:
            raise ValueError(f"{N} tokens exceed max_tokens={self.max_tokens}")
        x16, q16, hats, ug, z = self.x16[:N], self.q16[:N], self.hats[:N], self.ug[:N], self.z[:N]
        o.cast_bf16(flat, x16) if flat.dtype == torch.float32 else x16.copy_(flat)
        o.cast_bf16(self.w_up, self.wug16[:F])
        o.cast_bf16(self.w_gate, self.wug16[F:])
        o.cast_bf16(self.w_down, self.wd16)
        o.row_norm(self.w_down, self.wn)
        o.gemm(x16, self.selector16, q16, M=N, N=2 * r, K=d)
        o.gemm(q16, self.up_b16, hats, M=N, N=F, K=r, b_mn=True, epilogue=A.EPI_F32, lda=2 * r, ldc=2 * F)
        o.gemm(q16[:, r:], self.gate_b16, hats[:, F:], M=N, N=F, K=r, b_mn=True, epilogue=A.EPI_F32, lda=2 * r, ldc=2 * F)
        o.gemm(x16, self.wug16, ug, M=N, N=2 * F, K=d)
        o.svd_ffn_select(hats, ug, self.wn, z, self.selected[:N], self.cand_count[:N], up_m=self.up_m, gate_m=self.gate_m,
                         product_m=self.product_m, top_k=self.top_k)
        out = torch.empty(N, d, dtype=torch.float32, device=x.device)
        o.gemm(z, self.wd16, out, M=N, N=d, K=F, b_mn=True, epilogue=A.EPI_F32)
        return out.view(*x.shape[:-1], d)

    def backward(self, dout: torch.Tensor, dw_up, dw_gate, dw_down) -> torch.Tensor:
        """Gradients of the last forward: returns dx (fp32) and fills dw_up, dw_gate, dw_down [F, d] (fp32);
        neurons no token selected receive exact zeros."""
        o, d, F, N = self.ops, self.d, self.F, self._tokens
        x16, ug, z, dz, dug, dout16 = self.x16[:N], self.ug[:N], self.z[:N], self.dz[:N], self.dug[:N], self.dout16[:N]
        flat = dout.reshape(-1, d).contiguous()
        o.cast_bf16(flat, dout16) if flat.dtype == torch.float32 else dout16.copy_(flat)
        o.gemm(dout16, self.wd16, dz, M=N, N=F, K=d)
        o.svd_ffn_swiglu_bwd(ug, dz, self.selected[:N], dug)
        dx = torch.empty(N, d, dtype=torch.float32, device=dout.device)
        o.gemm(dug, self.wug16, dx, M=N, N=d, K=2 * F, b_mn=True, epilogue=A.EPI_F32)
        o.gemm_wgrad(dug, x16, self.dwug, M=2 * F, N=d, K=N)
        dw_up.copy_(self.dwug[:F])
        dw_gate.copy_(self.dwug[F:])
        o.gemm_wgrad(z, dout16, dw_down, M=F, N=d, K=N)
        return dx.view(dout.shape)

    @property
    def avg_candidate_size(self) -> float:
        return float(self.cand_count[: self._tokens].float().mean())

    @property
    def candidate_slots(self) -> int:
        """`candidate_slots` of the reference's aux (layers.py:636-640): the width of its candidate id table."""
        total = self.up_m + self.gate_m + self.product_m
        return total if self.candidate_mode == "slots" else min(self.F, max(self.top_k, total))


class _SvdFfnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_up, w_gate, w_down, module):
        ctx.module = module
        return module.forward(x.detach())

    @staticmethod
    def backward(ctx, dout):
        m = ctx.module
        g = [torch.empty_like(m.w_up), torch.empty_like(m.w_gate), torch.empty_like(m.w_down)]
        dx = m.backward(dout.contiguous(), *g)
        return dx, g[0], g[1], g[2], None


def svd_sparse_ffn(module: SVDFactorSparseFFN, x: torch.Tensor) -> torch.Tensor:
    """Autograd entry point: gradients flow to x and the module's w_up / w_gate / w_down."""
    return _SvdFfnFn.apply(x, module.w_up, module.w_gate, module.w_down, module)
