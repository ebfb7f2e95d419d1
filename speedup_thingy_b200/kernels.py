"""Operator table with the names, argument meaning and error behaviour of the reference's
``recursive_training_engine.kernels.optimized`` (optimized.py:12-154; arithmetic of kernels/reference.py:9-157).

Assigning these functions over the reference's symbols (or importing this module in its place) routes the
six operators the reference model actually calls -- ``k_fused_rmsnorm`` (layers.py:33), ``k_rope_apply``
(layers.py:50), ``k_flash_causal_dense`` (layers.py:73), ``k_flash_causal_grouped`` (layers.py:725),
``k_out_proj_grouped`` (layers.py:727), ``k_logits_shortlist`` (output.py:125) -- and the benchmarked
``k_logits_full`` / ``k_qkv_dense`` / ``k_cross_entropy_unreduced`` through the sm_100a kernels of the C ABI.
Every operator is a ``torch.autograd.Function`` whose forward and backward are C-ABI launches; tensors go in
and come out as the reference's do (fresh outputs, inputs untouched, non-contiguous inputs made contiguous).

There is no fallback: CPU tensors raise ``RuntimeError`` mentioning ``strict_cuda`` whatever the flag says
(optimized.py:51-55), and a missing library or device raises when the first operator is called.
GEMM-bearing operators compute in bf16 with fp32 accumulation (the reference's autocast arithmetic) and return
the input's dtype.
"""
from __future__ import annotations

import torch

from . import _abi as A
from .ops import CudaOps

STRICT_CUDA = True
REQUIRE_FLASH = True
_OPS: dict[int, CudaOps] = {}


# --------------------------------------------------------------------------- policy functions (optimized.py:12-49)
def set_strict_cuda(enabled: bool, *, require_flash: bool = True) -> None:
    """Recorded for `backend_status`; the kernels reject CPU tensors either way (there is nothing to fall back to)."""
    global STRICT_CUDA, REQUIRE_FLASH
    STRICT_CUDA, REQUIRE_FLASH = bool(enabled), bool(require_flash)


def triton_available() -> bool:
    """The reference's gate for its accelerated paths; here it reports whether the sm_100a library can run."""
    return torch.cuda.is_available()


def backend_status() -> dict[str, object]:
    cuda = torch.cuda.is_available()
    return {"mode": CudaOps.name if cuda else "unavailable", "strict_cuda": True, "require_flash": REQUIRE_FLASH,
            "cuda_available": cuda, "triton_available": False, "uses_reference_fallback": False}


def cuda_required() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is required for this optimized kernel path (rte_b200 has no CPU or Triton path)")


def _require_cuda_tensor(*tensors) -> None:
    if any(isinstance(t, torch.Tensor) and not t.is_cuda for t in tensors):
        raise RuntimeError("strict_cuda requires CUDA tensors in optimized hot-path kernels (rte_b200 has no fallback)")


def _ops_for(t: torch.Tensor) -> CudaOps:
    idx = t.device.index if t.device.index is not None else torch.cuda.current_device()
    if idx not in _OPS:
        _OPS[idx] = CudaOps(torch.device("cuda", idx))
    return _OPS[idx]


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(torch.bfloat16).contiguous()


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(torch.float32).contiguous()


def _check_gemm_dims(*dims: int) -> None:
    if any(v % 8 for v in dims):
        raise ValueError(f"rte_b200 GEMM operands need dimensions that are multiples of 8, got {dims}")


# --------------------------------------------------------------------------- RMSNorm (reference.py:9-17)
class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, eps):
        ops = _ops_for(x)
        y = _f32(x)
        if residual is not None:
            y = y.clone() if y.data_ptr() == x.data_ptr() else y
            ops.add_(y, _f32(residual))
        d = y.shape[-1]
        w = _f32(weight)
        out = torch.empty_like(y)
        rstd = torch.empty(y.numel() // d, dtype=torch.float32, device=y.device)
        ops.rmsnorm_fwd(y, w, None, rstd, y_f32=out, eps=eps)
        ctx.save_for_backward(y, w, rstd)
        ctx.has_residual = residual is not None
        ctx.in_dtypes = (x.dtype, weight.dtype, None if residual is None else residual.dtype)
        out_dtype = torch.result_type(x, weight)
        if residual is None:
            return out.to(out_dtype), None
        return out.to(out_dtype), y.to(torch.result_type(x, residual))

    @staticmethod
    def backward(ctx, d_out, d_sum):
        y, w, rstd = ctx.saved_tensors
        ops = _ops_for(y)
        d = y.shape[-1]
        rows = y.numel() // d
        dx = torch.empty_like(y)
        dw = torch.empty_like(w)
        partial = torch.empty(8 * ops.sm_count, d, dtype=torch.float32, device=y.device)
        dres = _f32(d_sum) if (ctx.has_residual and d_sum is not None) else None
        d_out = _f32(d_out) if d_out is not None else torch.zeros_like(y)
        ops.rmsnorm_bwd(y, w, rstd, d_out, dres, dx, None, dw, partial, rows=rows)
        xd, wd, rd = ctx.in_dtypes
        return dx.to(xd), dw.to(wd), (dx.to(rd) if ctx.has_residual else None), None


def k_fused_rmsnorm(x, weight, residual=None, eps: float = 1e-5):
    """(rmsnorm(x [+ residual]) * weight, x + residual | None), statistics in fp32 (reference.py:9-17)."""
    _require_cuda_tensor(x, weight, residual)
    if x.shape[-1] != weight.shape[-1]:
        raise ValueError("k_fused_rmsnorm: weight must match the last dimension of x")
    return _RmsNorm.apply(x, weight, residual, float(eps))


# --------------------------------------------------------------------------- rotary embedding (reference.py:20-28)
class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin):
        ops = _ops_for(q)
        S, hd = q.shape[-2], q.shape[-1]
        c, s = _f32(cos).reshape(S, hd), _f32(sin).reshape(S, hd)
        outs = []
        for t in (q, k):
            src = t.detach().contiguous()
            if src.dtype not in (torch.float32, torch.bfloat16):
                src = src.float()
            out = torch.empty_like(src)
            ops.rope_apply(src, c, s, out, rows=src.numel() // (S * hd), S=S, head_dim=hd)
            outs.append(out.to(t.dtype))
        ctx.save_for_backward(c, s)
        return tuple(outs)

    @staticmethod
    def backward(ctx, dq, dk):
        c, s = ctx.saved_tensors
        ops = _ops_for(c)
        S, hd = c.shape
        grads = []
        for g in (dq, dk):
            src = g.contiguous() if g.dtype in (torch.float32, torch.bfloat16) else g.float().contiguous()
            out = torch.empty_like(src)
            ops.rope_apply(src, c, s, out, rows=src.numel() // (S * hd), S=S, head_dim=hd, adjoint=True)
            grads.append(out.to(g.dtype))
        return grads[0], grads[1], None, None


def k_rope_apply(q, k, cos, sin):
    """q*cos + rotate_half(q)*sin on adjacent pairs, same for k; cos/sin [S, head_dim] (reference.py:20-28)."""
    _require_cuda_tensor(q, k, cos, sin)
    if q.shape[-2:] != k.shape[-2:] or cos.shape[-2:] != q.shape[-2:] or cos.numel() != q.shape[-2] * q.shape[-1]:
        raise ValueError("k_rope_apply: q/k [..., S, head_dim] with cos/sin [S, head_dim]")
    return _Rope.apply(q, k, cos, sin)


# --------------------------------------------------------------------------- causal attention (reference.py:40-41,54-55)
class _FlashCausal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v):
        ops = _ops_for(q)
        B, H, S, hd = q.shape
        # the kernels read one packed [B*S, 3*H*hd] buffer, columns (q | k | v), head-major inside each
        qkv = torch.stack([q.detach(), k.detach(), v.detach()], dim=0).to(torch.bfloat16)      # [3,B,H,S,hd]
        qkv = qkv.permute(1, 3, 0, 2, 4).contiguous().view(B * S, 3 * H * hd)
        y = torch.empty(B * S, H * hd, dtype=torch.bfloat16, device=q.device)
        lse = torch.empty(B * H * S, dtype=torch.float32, device=q.device)
        ops.attn_fwd(qkv, y, lse, B=B, S=S, n_heads=H, head_dim=hd, rope=ops.identity_rope_table(S, hd))
        ctx.save_for_backward(qkv, y, lse)
        ctx.dims = (B, H, S, hd)
        ctx.in_dtype = q.dtype
        return y.view(B, S, H, hd).permute(0, 2, 1, 3).to(q.dtype)

    @staticmethod
    def backward(ctx, d_out):
        qkv, y, lse = ctx.saved_tensors
        ops = _ops_for(qkv)
        B, H, S, hd = ctx.dims
        dy = d_out.permute(0, 2, 1, 3).to(torch.bfloat16).contiguous().view(B * S, H * hd)
        dqkv = torch.empty_like(qkv)
        ops.attn_bwd(qkv, y, dy, lse, dqkv, B=B, S=S, n_heads=H, head_dim=hd, rope=ops.identity_rope_table(S, hd))
        g = dqkv.view(B, S, 3, H, hd).permute(2, 0, 3, 1, 4).to(ctx.in_dtype)
        return g[0], g[1], g[2]


def k_flash_causal_dense(q, k, v):
    """softmax(q k^T / sqrt(head_dim), causal) v over [B, H, S, head_dim] (reference.py:40-41)."""
    _require_cuda_tensor(q, k, v)
    if q.ndim != 4 or q.shape != k.shape or q.shape != v.shape:
        raise ValueError("k_flash_causal_*: q, k, v must share the shape [B, H, S, head_dim]")
    if q.shape[2] > 256 or q.shape[3] not in (8, 16, 32, 64, 128):
        raise ValueError("k_flash_causal_*: S <= 256 and head_dim in {8,16,32,64,128}")
    return _FlashCausal.apply(q, k, v)


k_flash_causal_grouped = k_flash_causal_dense          # same arithmetic over the active heads (reference.py:54-55)


# --------------------------------------------------------------------------- GEMM-bearing operators
def _mm_io(ops: CudaOps, x16, w16, out_dtype):
    """x16 [M, in] @ w16 [in, out] (weight stored input-major, the banked layout of layers.py:690-696)."""
    M, K = x16.shape
    N = w16.shape[1]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x16.device)
    ops.gemm(x16, w16, out, M=M, N=N, K=K, b_mn=True)
    return out if out_dtype == torch.bfloat16 else out.to(out_dtype)


class _MatmulIO(torch.autograd.Function):
    """y = x @ w, w [in, out]."""

    @staticmethod
    def forward(ctx, x, w):
        ops = _ops_for(x)
        x16, w16 = _bf16(x).view(-1, x.shape[-1]), _bf16(w)
        _check_gemm_dims(x16.shape[1], w16.shape[1])
        ctx.save_for_backward(x16, w16)
        ctx.meta = (x.shape, x.dtype, w.dtype)
        return _mm_io(ops, x16, w16, x.dtype).view(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x16, w16 = ctx.saved_tensors
        ops = _ops_for(x16)
        xshape, xd, wd = ctx.meta
        M, K = x16.shape
        N = w16.shape[1]
        dy16 = _bf16(dy).view(M, N)
        dx = torch.empty(M, K, dtype=torch.float32, device=x16.device)
        ops.gemm(dy16, w16, dx, M=M, N=K, K=N, epilogue=A.EPI_F32)                 # dy [M,out] . w[in,out]^T
        dw = torch.empty(K, N, dtype=torch.float32, device=x16.device)
        ops.gemm_wgrad(x16, dy16, dw, M=K, N=N, K=M)                                # x^T dy, reduction over tokens
        return dx.view(xshape).to(xd), dw.to(wd)


class _MatmulOI(torch.autograd.Function):
    """y = x @ w^T, w [out, in] (nn.Linear / tied-embedding layout)."""

    @staticmethod
    def forward(ctx, x, w):
        ops = _ops_for(x)
        x16, w16 = _bf16(x).view(-1, x.shape[-1]), _bf16(w)
        _check_gemm_dims(x16.shape[1])
        M, K = x16.shape
        N = w16.shape[0]
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        ops.gemm(x16, w16, out, M=M, N=N, K=K)
        ctx.save_for_backward(x16, w16)
        ctx.meta = (x.shape, x.dtype, w.dtype)
        return out.to(x.dtype).view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x16, w16 = ctx.saved_tensors
        ops = _ops_for(x16)
        xshape, xd, wd = ctx.meta
        M, K = x16.shape
        N = w16.shape[0]
        _check_gemm_dims(N)
        dy16 = _bf16(dy).view(M, N)
        dx = torch.empty(M, K, dtype=torch.float32, device=x16.device)
        ops.gemm(dy16, w16, dx, M=M, N=K, K=N, b_mn=True, epilogue=A.EPI_F32)      # dy [M,out] . w[out,in]
        dw = torch.empty(N, K, dtype=torch.float32, device=x16.device)
        ops.gemm_wgrad(dy16, x16, dw, M=N, N=K, K=M)                                # dy^T x
        return dx.view(xshape).to(xd), dw.to(wd)


def k_qkv_dense(x, wq, wk, wv):
    """(x @ wq, x @ wk, x @ wv), weights [in, out] (reference.py:31-37)."""
    _require_cuda_tensor(x, wq, wk, wv)
    return _MatmulIO.apply(x, wq), _MatmulIO.apply(x, wk), _MatmulIO.apply(x, wv)


def k_logits_full(hidden, vocab_weight):
    """hidden @ vocab_weight^T (reference.py:137-138)."""
    _require_cuda_tensor(hidden, vocab_weight)
    if hidden.shape[-1] != vocab_weight.shape[-1]:
        raise ValueError("k_logits_full: hidden [..., d] against vocab_weight [V, d]")
    return _MatmulOI.apply(hidden, vocab_weight)


class _OutProjGrouped(torch.autograd.Function):
    """x @ wo[row_indices, :] with the selected rows gathered by the C-ABI row gather (reference.py:58-59)."""

    @staticmethod
    def forward(ctx, x, wo, row_indices):
        ops = _ops_for(x)
        idx = row_indices.detach().to(torch.int32).contiguous()
        n, dout = idx.numel(), wo.shape[1]
        _check_gemm_dims(n, dout)
        wo16 = _bf16(wo)
        sel = torch.empty(n, dout, dtype=torch.bfloat16, device=x.device)
        ops.gather_rows(wo16, idx, sel, n, dout * 2)
        x16 = _bf16(x).view(-1, n)
        ctx.save_for_backward(x16, sel, idx)
        ctx.meta = (x.shape, x.dtype, wo.dtype, wo.shape)
        return _mm_io(ops, x16, sel, x.dtype).view(*x.shape[:-1], dout)

    @staticmethod
    def backward(ctx, dy):
        x16, sel, idx = ctx.saved_tensors
        ops = _ops_for(x16)
        xshape, xd, wd, wshape = ctx.meta
        M, n = x16.shape
        dout = sel.shape[1]
        dy16 = _bf16(dy).view(M, dout)
        dx = torch.empty(M, n, dtype=torch.float32, device=x16.device)
        ops.gemm(dy16, sel, dx, M=M, N=n, K=dout, epilogue=A.EPI_F32)
        dsel = torch.empty(n, dout, dtype=torch.float32, device=x16.device)
        ops.gemm_wgrad(x16, dy16, dsel, M=n, N=dout, K=M)
        dwo = torch.zeros(wshape, dtype=torch.float32, device=x16.device)
        ops.scatter_add_rows(dwo, idx, dsel, n, dout)
        return dx.view(xshape).to(xd), dwo.to(wd), None


def k_out_proj_grouped(x, wo, row_indices):
    _require_cuda_tensor(x, wo, row_indices)
    if x.shape[-1] != row_indices.numel():
        raise ValueError("k_out_proj_grouped: x [..., len(row_indices)]")
    return _OutProjGrouped.apply(x, wo, row_indices)


# --------------------------------------------------------------------------- shortlist logits (reference.py:141-143)
class _LogitsShortlist(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, vocab_weight, shortlist):
        ops = _ops_for(hidden)
        d, K = hidden.shape[-1], shortlist.shape[-1]
        h16, w16 = _bf16(hidden).view(-1, d), _bf16(vocab_weight)
        ids = shortlist.detach().to(torch.int32).contiguous().view(-1, K)
        rows = h16.shape[0]
        logits = torch.empty(rows, K, dtype=torch.bfloat16, device=hidden.device)
        scratch = torch.empty(rows, dtype=torch.float32, device=hidden.device)
        ops.shortlist_ce(h16, w16, ids, None, 1, scratch, logits, None)
        ctx.save_for_backward(h16, w16, ids)
        ctx.meta = (hidden.shape, hidden.dtype, vocab_weight.dtype)
        return logits.to(hidden.dtype).view(*shortlist.shape)

    @staticmethod
    def backward(ctx, dlogits):
        h16, w16, ids = ctx.saved_tensors
        ops = _ops_for(h16)
        hshape, hd, wd = ctx.meta
        rows, d = h16.shape
        V, K = w16.shape[0], ids.shape[1]
        _check_gemm_dims(V)
        # gradient over shortlist slots -> otherwise-zero dense rows, so both products run on the tensor cores
        dense = torch.empty(rows, V, dtype=torch.bfloat16, device=h16.device)
        ops.scatter_cols(_bf16(dlogits).view(rows, K), ids, dense)
        dh = torch.empty(rows, d, dtype=torch.float32, device=h16.device)
        ops.gemm(dense, w16, dh, M=rows, N=d, K=V, b_mn=True, epilogue=A.EPI_F32)
        dw = torch.empty(V, d, dtype=torch.float32, device=h16.device)
        ops.gemm_wgrad(dense, h16, dw, M=V, N=d, K=rows)
        return dh.view(hshape).to(hd), dw.to(wd), None


def k_logits_shortlist(hidden, vocab_weight, shortlist):
    """(hidden[..., None, :] * vocab_weight[shortlist]).sum(-1); ids must be distinct within a row for the
    backward pass (they are: output.py:46-70)."""
    _require_cuda_tensor(hidden, vocab_weight, shortlist)
    if hidden.shape[:-1] != shortlist.shape[:-1]:
        raise ValueError("k_logits_shortlist: hidden [..., d] with shortlist [..., K]")
    return _LogitsShortlist.apply(hidden, vocab_weight, shortlist)


# --------------------------------------------------------------------------- cross entropy (reference.py:146-147)
class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        ops = _ops_for(logits)
        V = logits.shape[-1]
        lg = _bf16(logits).view(-1, V)
        tg = targets.detach().to(torch.int64).contiguous().view(-1)
        loss = torch.empty(lg.shape[0], dtype=torch.float32, device=logits.device)
        ops.ce_fwd_bwd(lg, tg, None, 1, loss, None)
        ctx.save_for_backward(lg, tg)
        ctx.meta = (logits.shape, logits.dtype)
        return loss.view_as(targets)

    @staticmethod
    def backward(ctx, dloss):
        lg, tg = ctx.saved_tensors
        ops = _ops_for(lg)
        shape, dt = ctx.meta
        dlogits = torch.empty_like(lg)
        scratch = torch.empty(lg.shape[0], dtype=torch.float32, device=lg.device)
        ops.ce_fwd_bwd(lg, tg, _f32(dloss).view(-1), 1, scratch, dlogits)          # (softmax - onehot) * dloss[row]
        return dlogits.view(shape).to(dt), None


def k_cross_entropy_unreduced(logits, targets):
    _require_cuda_tensor(logits, targets)
    if logits.shape[:-1] != targets.shape:
        raise ValueError("k_cross_entropy_unreduced: logits [..., V] with targets [...]")
    return _CrossEntropy.apply(logits, targets)


# --------------------------------------------------------------------------- host-side helpers of the table
def k_recurrent_exact_loop(step_fn, h, h0, depth: int, boundaries: set):
    """Control flow only (reference.py:127-134)."""
    states = {}
    for t in range(depth):
        h = step_fn(h, h0)
        if t + 1 in boundaries:
            states[t + 1] = h
    return h, states


def k_metrics_reduce(values: dict) -> dict:
    """One device-to-host read per key, as reference.py:156-157."""
    return {k: float(v.detach().float().mean().cpu()) for k, v in values.items()}


def k_sample_audit_mask(p, seed: int):
    """Bernoulli audit mask from a generator on p's device seeded with `seed` (reference.py:151-154): a host-side
    sampling decision, kept as the reference draws it so that the same seed gives the same mask."""
    gen = torch.Generator(device=p.device)
    gen.manual_seed(seed)
    return torch.bernoulli(p, generator=gen).bool()


class PackedByRecipe:
    """Result of `k_pack_by_recipe` (reference.py:81-88): same field names."""
    __slots__ = ("packed", "permutation", "inverse_permutation", "keys", "offsets", "unique_keys")

    def __init__(self, packed, permutation, inverse_permutation, keys, offsets, unique_keys):
        self.packed, self.permutation, self.inverse_permutation = packed, permutation, inverse_permutation
        self.keys, self.offsets, self.unique_keys = keys, offsets, unique_keys


class _GatherRows(torch.autograd.Function):
    """out[i] = src[index[i]] for a PERMUTATION `index` through the C-ABI row gather; the backward is the gather by
    the inverse permutation (no atomics)."""

    @staticmethod
    def forward(ctx, src, index, inverse):
        ops = _ops_for(src)
        flat = src.detach().contiguous().view(src.shape[0], -1)
        out = torch.empty_like(flat)
        ops.gather_rows(flat, index.to(torch.int32), out, flat.shape[0], flat.shape[1] * flat.element_size())
        ctx.save_for_backward(index, inverse)
        return out.view(src.shape)

    @staticmethod
    def backward(ctx, d_out):
        index, inverse = ctx.saved_tensors
        ops = _ops_for(d_out)
        flat = d_out.contiguous().view(d_out.shape[0], -1)
        out = torch.empty_like(flat)
        ops.gather_rows(flat, inverse.to(torch.int32), out, flat.shape[0], flat.shape[1] * flat.element_size())
        return out.view(d_out.shape), None, None


def _gather_ok(t: torch.Tensor) -> None:
    if (t[0].numel() * t.element_size()) % 16:
        raise ValueError("rte_b200 row gathers move 16-byte units: a row must be a multiple of 16 bytes")


def k_pack_by_recipe(hidden, recipe_ids, depth_ids, audit_flags=None):
    """Stable sort of the samples by (recipe, depth, audited) and the packed copy of `hidden` in that order
    (reference.py:91-104).  The keys are sorted on the device by torch (index bookkeeping); the rows move through
    rte_gather_rows."""
    _require_cuda_tensor(hidden, recipe_ids, depth_ids, audit_flags)
    audit = torch.zeros_like(recipe_ids) if audit_flags is None else audit_flags.long()
    keys = recipe_ids.long() * 1_000_000 + depth_ids.long() * 10 + audit
    sorted_keys, perm = torch.sort(keys, stable=True)
    inverse = torch.empty_like(perm)
    inverse[perm] = torch.arange(perm.numel(), device=perm.device)
    unique, counts = torch.unique_consecutive(sorted_keys, return_counts=True)
    offsets = torch.cat([counts.new_zeros(1), counts.cumsum(0)])
    _gather_ok(hidden)
    return PackedByRecipe(_GatherRows.apply(hidden, perm, inverse), perm, inverse, sorted_keys, offsets, unique)


def k_unpack_from_recipe(packed, inverse_permutation):
    """packed[inverse_permutation] (reference.py:107-108)."""
    _require_cuda_tensor(packed, inverse_permutation)
    _gather_ok(packed)
    perm = torch.empty_like(inverse_permutation)
    perm[inverse_permutation] = torch.arange(inverse_permutation.numel(), device=inverse_permutation.device)
    return _GatherRows.apply(packed, inverse_permutation, perm)


def k_qkv_grouped(x, wq, wk, wv, column_indices):
    """x @ w[:, column_indices] for the three projections (reference.py:44-51); the gathered columns are multiplied by
    the tcgen05 GEMM, autograd scatters their gradients back into the full weights."""
    _require_cuda_tensor(x, wq, wk, wv, column_indices)
    cols = column_indices.long()
    return k_qkv_dense(x, wq.index_select(1, cols), wk.index_select(1, cols), wv.index_select(1, cols))


def _swiglu_io(x, wu, wg, wd):
    """(x @ wu) * silu(x @ wg) @ wd with [in, out] weights through the packed SwiGLU FFN (GEMM + SiLU-gate + GEMM)."""
    wug = torch.cat([wu.t(), wg.t()], dim=0)            # [2M, d] = (up rows | gate rows)
    flat = x.reshape(-1, x.shape[-1])
    return packed_swiglu_ffn(flat, wug, wd).view(*x.shape[:-1], wd.shape[-1])


def k_swiglu_dense(x, wu, wg, wd):
    """reference.py:62-68."""
    _require_cuda_tensor(x, wu, wg, wd)
    return _swiglu_io(x, wu, wg, wd)


def k_swiglu_grouped(x, wu, wg, wd, slab_indices):
    """reference.py:71-78: SwiGLU over the hidden units `slab_indices` only."""
    _require_cuda_tensor(x, wu, wg, wd, slab_indices)
    idx = slab_indices.long()
    return _swiglu_io(x, wu.index_select(1, idx), wg.index_select(1, idx), wd.index_select(0, idx))


def k_macro_phi(h, h0, d_gain, v, u, bias, eps: float = 1e-5):
    """The operator table's simplified macro operator (reference.py:111-124): h + d_gain*h + silu(z @ v) @ u + bias with
    z = [rmsnorm(h) | mean_S rmsnorm(h) | h0].  (The model itself runs the bounded-residual form, rte_macro_phi_fwd.)
    Norm and both products run in the sm_100a kernels; concatenation and the element-wise tail are tensor glue."""
    _require_cuda_tensor(h, h0, d_gain, v, u, bias)
    normed, _ = k_fused_rmsnorm(h, torch.ones(h.shape[-1], device=h.device, dtype=h.dtype), None, eps)
    pooled = normed.mean(dim=1, keepdim=True).expand_as(normed)
    z = torch.cat([normed, pooled, h0], dim=-1)
    low = _MatmulIO.apply(torch.nn.functional.silu(_MatmulIO.apply(z, v)), u)
    return h + d_gain * h + low + bias


# --------------------------------------------------------------------------- packed SwiGLU FFN
class _PackedSwiGLUFFN(torch.autograd.Function):
    """(x @ wug^T -> (up | gate)) -> up * silu(gate) -> @ wdown_rows, saving (x, wug, wdown_rows, ug, z) in bf16
    exactly as the reference's _TritonPackedSwiGLUFFN does (kernels/active_swiglu_triton.py:62-108)."""

    @staticmethod
    def forward(ctx, x, wug, wdown_rows):
        ops = _ops_for(x)
        N, d = x.shape
        m = wug.shape[0] // 2
        x16, wug16, wd16 = _bf16(x), _bf16(wug), _bf16(wdown_rows)
        ug = torch.empty(N, 2 * m, dtype=torch.bfloat16, device=x.device)
        z = torch.empty(N, m, dtype=torch.bfloat16, device=x.device)
        y = torch.empty(N, d, dtype=torch.float32, device=x.device)
        if m % 64 == 0 and N <= 1024:        # small batches: SwiGLU fused into the GEMM epilogue
            ops.gemm(x16, wug16, z, M=N, N=2 * m, K=d, epilogue=A.EPI_SWIGLU_FWD, out2=ug, pair=m)
        else:                                # large batches: plain-store GEMM + one vectorised pass is faster
            ops.gemm(x16, wug16, ug, M=N, N=2 * m, K=d)
            ops.swiglu_fwd(ug, z, N, m)
        ops.gemm(z, wd16, y, M=N, N=d, K=m, b_mn=True, epilogue=A.EPI_F32)
        ctx.save_for_backward(x16, wug16, wd16, ug, z)
        ctx.dtypes = (x.dtype, wug.dtype, wdown_rows.dtype)
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x16, wug16, wd16, ug, z = ctx.saved_tensors
        ops = _ops_for(x16)
        N, d = x16.shape
        m = wd16.shape[0]
        dy16 = _bf16(dy)
        dz = torch.empty(N, m, dtype=torch.bfloat16, device=x16.device)
        dug = torch.empty(N, 2 * m, dtype=torch.bfloat16, device=x16.device)
        ops.gemm(dy16, wd16, dz, M=N, N=m, K=d)
        ops.swiglu_bwd(ug, dz, dug, N, m)
        dx = torch.empty(N, d, dtype=torch.float32, device=x16.device)
        ops.gemm(dug, wug16, dx, M=N, N=d, K=2 * m, b_mn=True, epilogue=A.EPI_F32)
        dwug = torch.empty(2 * m, d, dtype=torch.float32, device=x16.device)
        ops.gemm_wgrad(dug, x16, dwug, M=2 * m, N=d, K=N)
        dwd = torch.empty(m, d, dtype=torch.float32, device=x16.device)
        ops.gemm_wgrad(z, dy16, dwd, M=m, N=d, K=N)
        xd, ud, dd = ctx.dtypes
        return dx.to(xd), dwug.to(ud), dwd.to(dd)


def packed_swiglu_ffn(x, wug, wdown_rows):
    """Drop-in for ``triton_packed_swiglu_ffn`` (kernels/active_swiglu_triton.py:111-125; layers.py:90-116,284-339):
    x [tokens, d], wug [2*active_m, d] = (up rows | gate rows), wdown_rows [active_m, d].  Same shape errors."""
    _require_cuda_tensor(x, wug, wdown_rows)
    if x.ndim != 2 or wug.ndim != 2 or wdown_rows.ndim != 2:
        raise ValueError("expected x [N,D], wug [2M,D], wdown_rows [M,D]")
    if wug.shape[0] % 2 != 0:
        raise ValueError("wug first dimension must be 2M")
    if wdown_rows.shape[0] != wug.shape[0] // 2:
        raise ValueError("wdown_rows first dimension must match M")
    _check_gemm_dims(x.shape[1], wdown_rows.shape[0])
    return _PackedSwiGLUFFN.apply(x, wug, wdown_rows)


triton_packed_swiglu_ffn = packed_swiglu_ffn          # the symbol layers.py:12-22 imports


def active_union_swiglu(x, wug_weight, wd_weight, active_ids):
    """ActiveUnionSwiGLU.forward (layers.py:267-282): SwiGLU over the sorted unique `active_ids` only.
    wug_weight [2F, d], wd_weight [d, F]; the active rows are gathered by the C-ABI row gather."""
    _require_cuda_tensor(x, wug_weight, wd_weight, active_ids)
    ids = torch.unique(active_ids.reshape(-1).to(torch.int64), sorted=True)
    f = wd_weight.shape[1]
    rows = torch.cat([ids, ids + f]).to(torch.int32)
    # index_select keeps autograd's scatter of the row gradients into the dense weights
    wug_active = wug_weight.index_select(0, rows.long())
    wd_rows = wd_weight.t().index_select(0, ids)
    flat = x.reshape(-1, x.shape[-1])
    return packed_swiglu_ffn(flat, wug_active, wd_rows).view(*x.shape[:-1], -1)
