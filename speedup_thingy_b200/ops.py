"""Tensor-level operator table over the C ABI (``include/rte_b200.h``).

Every method takes preallocated ``torch`` CUDA tensors (used only as device memory), launches the
corresponding sm_100a kernel on the current CUDA stream and returns nothing (outputs are arguments).
This is the counterpart of the reference's ``kernels/optimized.py`` dispatch table: same operator
granularity, but a missing library or a CPU tensor is a hard error, never a fallback.
"""
from __future__ import annotations

import os

import ctypes as C

import torch

from . import _abi as A


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise A.RteError("strict_cuda: the rte_b200 kernels need CUDA tensors; CPU tensors are rejected "
                             "(no reference fallback)")


class CudaOps:
    """Launches the hand-written kernels.  One instance per device."""

    name = "cuda_sm100a_ext"

    def __init__(self, device: torch.device | str = "cuda:0"):
        if not torch.cuda.is_available():
            raise A.RteError("CUDA is required: rte_b200 has no CPU path")
        self.device = torch.device(device)
        self.lib = A.load()
        with torch.cuda.device(self.device):
            self.sm_count = int(self.lib.rte_device_sm_count())
        if self.sm_count <= 0:
            raise A.RteError("could not query the SM count")
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0          # kernels-entry calls issued (for bench accounting)
        self._split_ws: torch.Tensor | None = None
        self.small_gemm_rows = 256  # products with at most this many rows go to the few-row kernel (0: never)
        # ... and so can weight gradients over that few rows (RTE_SMALL_WGRAD=1).  Off by default: inside the training
        # step its hundreds of small CTAs on the replay's high-priority stream displace the hot pass (measured 2.04 ms
        # per step against 1.72 ms with these products on the tcgen05 kernel's 32 tiles).
        self.small_wgrad = os.environ.get("RTE_SMALL_WGRAD", "0") == "1"
        # RTE_SMALL_FUSED_REDUCE=1: split-K partials of a few-row product summed inside the launch by each tile's last
        # CTA (one launch less on the replay's chain per product).  Off by default: measured on one machine, the step
        # takes 1.774 ms with it against 1.754 ms with the separate reduction launch (the serial tail of the last CTA
        # costs more than the launch it saves).
        self.small_fused_reduce = os.environ.get("RTE_SMALL_FUSED_REDUCE", "0") == "1"
        self._split_counters = torch.zeros(1024, dtype=torch.int32, device=self.device)      # per-tile arrival counters
        self.few_rows_max_splits = int(os.environ.get("RTE_FEWROW_SPLITS", "4"))
        self.gemm_max_ctas = 0     # 0 = one persistent CTA per SM; smaller values leave SMs to kernels of other streams
        # tile hints passed to every tcgen05 GEMM (0 = the library's choice): RTE_GEMM_PAIR=0 keeps every tile on one
        # CTA (no cta_group::2 pairs), RTE_GEMM_TILE_N forces 128 or 256 columns per tile
        self.gemm_cta_pair = 1 if os.environ.get("RTE_GEMM_PAIR", "1") == "0" else 0
        self.gemm_tile_n = int(os.environ.get("RTE_GEMM_TILE_N", "0"))
        # When set, launches that only produce PARAMETER gradients (weight-gradient GEMMs with their split reduction,
        # column-sum reductions of the norm backward) go to this stream, ordered after the work issued so far on the
        # current one: a latency-bound backward chain then carries only the data-gradient launches.
        self.param_stream: torch.cuda.Stream | None = None
        self._rope_tables: dict[tuple[int, int], torch.Tensor] = {}

    # ------------------------------------------------------------------ helpers
    @property
    def stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def check_status(self) -> None:
        """Synchronises and raises if a kernel reported a device-side problem."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise A.RteError(f"device status {code}: {self.lib.rte_status_string(code).decode()}")

    def _deferred(self):
        import contextlib
        ps = self.param_stream
        if ps is None:
            return contextlib.nullcontext()
        ps.wait_stream(torch.cuda.current_stream(self.device))
        return torch.cuda.stream(ps)

    def _call(self, name: str, *args) -> None:
        self.launches += 1
        A.check(getattr(self.lib, name)(*args), name)

    def split_workspace(self, numel: int) -> torch.Tensor:
        if self._split_ws is None or self._split_ws.numel() < numel:
            self._split_ws = torch.empty(numel, dtype=torch.float32, device=self.device)
        return self._split_ws

    # ------------------------------------------------------------------ GEMM
    def gemm(self, a, b, out, *, M: int, N: int, K: int, a_mn: bool = False, b_mn: bool = False,
             epilogue: int = A.EPI_BF16, residual=None, out2=None, pair: int = 0, splits: int = 1,
             split_stride: int = 0, lda: int | None = None, ldb: int | None = None, ldc: int | None = None,
             ldr: int | None = None, ldc2: int | None = None, tile_group=None, n_groups: int = 0,
             b_group_stride: int = 0, split_kblocks=None, tile_n: int | None = None, cta_pair: int | None = None,
             split_reduce=None) -> None:
        """out[M,N] = a[M,K] @ b[N,K]^T with the stated epilogue (see rte_gemm_bf16).  `tile_group` switches on the
        grouped mode (B = stack of per-group matrices), `split_kblocks` the ragged split-K."""
        _require_cuda(a, b, out, residual, out2)
        args = A.GemmArgs()
        args.M, args.N, args.K = M, N, K
        args.A, args.lda, args.a_mn_major = a.data_ptr(), (lda if lda is not None else a.stride(0)), int(a_mn)
        args.B, args.ldb, args.b_mn_major = b.data_ptr(), (ldb if ldb is not None else b.stride(0)), int(b_mn)
        args.epilogue = epilogue
        args.C, args.ldc = out.data_ptr(), (ldc if ldc is not None else out.stride(-2))
        args.R = residual.data_ptr() if residual is not None else None
        args.ldr = (ldr if ldr is not None else residual.stride(-2)) if residual is not None else 0
        args.C2 = out2.data_ptr() if out2 is not None else None
        args.ldc2 = (ldc2 if ldc2 is not None else out2.stride(-2)) if out2 is not None else 0
        args.b_pair_offset = pair
        args.splits, args.split_stride = splits, split_stride
        args.max_ctas = self.gemm_max_ctas
        args.status = self.status.data_ptr()
        args.tile_group = tile_group.data_ptr() if tile_group is not None else None
        args.n_groups, args.b_group_stride = n_groups, b_group_stride
        args.split_kblocks = split_kblocks.data_ptr() if split_kblocks is not None else None
        args.tile_n = self.gemm_tile_n if tile_n is None else tile_n
        args.cta_pair = self.gemm_cta_pair if cta_pair is None else cta_pair
        if split_reduce is not None:          # (counters, final output, accumulate): the few-row kernel reduces its splits itself
            args.split_counters, args.split_out = split_reduce[0].data_ptr(), split_reduce[1].data_ptr()
            args.split_accumulate = int(split_reduce[2])
        # few output rows, or (weight gradient of a few rows: A and B stored [K, *]) a reduction over few rows
        few_rows = (epilogue in (A.EPI_BF16, A.EPI_F32) and tile_group is None and split_kblocks is None and K % 8 == 0
                    and (not b_mn or N % 8 == 0)
                    and ((not a_mn and M <= self.small_gemm_rows)
                         or (a_mn and b_mn and self.small_wgrad and K <= self.small_gemm_rows and epilogue == A.EPI_F32 and M % 8 == 0 and splits == 1)))
        self._call("rte_gemm_bf16_small" if few_rows else "rte_gemm_bf16", C.byref(args), self.stream)

    def pick_splits(self, M: int, N: int, K: int) -> int:
        """Split count for a reduction-heavy GEMM whose output has few tiles (weight gradients)."""
        args = A.GemmArgs()
        args.M, args.N, args.K, args.epilogue = M, N, K, A.EPI_F32
        args.max_ctas, args.tile_n, args.cta_pair = self.gemm_max_ctas, self.gemm_tile_n, self.gemm_cta_pair
        tm, tn, conc = C.c_int32(0), C.c_int32(0), C.c_int32(0)
        A.check(self.lib.rte_gemm_tile_plan(C.byref(args), C.byref(tm), C.byref(tn), C.byref(conc)), "rte_gemm_tile_plan")
        tiles = -(-M // tm.value) * -(-N // tn.value)
        kblocks = -(-K // 64)
        want = max(1, min(conc.value // max(tiles, 1), kblocks // 8 if kblocks >= 16 else 1, 16))
        while want > 1:
            per = -(-kblocks // want)
            if -(-kblocks // per) == want:
                break
            want -= 1
        return max(want, 1)

    def gemm_wgrad(self, a_t, b_t, out, *, M: int, N: int, K: int, accumulate: bool = False,
                   lda: int | None = None, ldb: int | None = None, ws=None) -> None:
        """out f32 [M,N] (+)= a_t^T @ b_t where a_t is stored [K,M] and b_t is stored [K,N]
        (both MN-major for the tensor core), split along K across SMs and reduced in fixed order."""
        splits = self.pick_splits(M, N, K)
        with self._deferred():
            if splits == 1:         # accumulation rides in the epilogue (residual = the output itself)
                self.gemm(a_t, b_t, out, M=M, N=N, K=K, a_mn=True, b_mn=True, epilogue=A.EPI_F32, lda=lda, ldb=ldb, ldc=N,
                          residual=out if accumulate else None)
                return
            if ws is None:
                ws = self.split_workspace(splits * M * N)
            elif ws.numel() < splits * M * N:
                raise A.RteError("split-K workspace too small")
            self.gemm(a_t, b_t, ws, M=M, N=N, K=K, a_mn=True, b_mn=True, epilogue=A.EPI_F32, splits=splits,
                      split_stride=M * N, lda=lda, ldb=ldb, ldc=N)
            self.reduce_splits(ws, splits, M * N, M * N, out, accumulate)

    def gemm_f32_few_rows(self, a, b, out, *, M: int, N: int, K: int, b_mn: bool, ws, accumulate: bool = False,
                          reduce: bool = True) -> tuple[int, int]:
        """out f32 [M,N] (+)= a @ b^T for a GEMM with few rows and a long reduction (the audit replay's chain): one or
        two output tiles would run their k-blocks one after another on one or two SMs, so the reduction is split
        across up to 16 CTAs per tile and summed in fixed order.  `reduce=False` leaves the partials in `ws` for a
        consumer that sums them itself; returns (splits, stride between partials) -- (1, 0) when `out` holds the result."""
        kb = -(-K // 64)
        splits = 1
        if M <= 256 and kb >= 16 and K % 64 == 0:
            splits = max(s for s in range(1, self.few_rows_max_splits + 1) if kb % s == 0 and kb // s >= 2)
        if splits == 1 or ws is None or ws.numel() < splits * M * N:
            self.gemm(a, b, out, M=M, N=N, K=K, b_mn=b_mn, epilogue=A.EPI_F32, residual=out if accumulate else None)
            return (1, 0)
        if not reduce and not accumulate and (M * N) % 4 == 0:
            self.gemm(a, b, ws, M=M, N=N, K=K, b_mn=b_mn, epilogue=A.EPI_F32, splits=splits, split_stride=M * N, ldc=N)
            return (splits, M * N)
        if self.small_fused_reduce and M <= self.small_gemm_rows and -(-N // 32) * -(-M // 64) <= 1024 and out.is_contiguous():
            # one launch: the last CTA of every output tile sums the tile's partials (fixed order)
            self.gemm(a, b, ws, M=M, N=N, K=K, b_mn=b_mn, epilogue=A.EPI_F32, splits=splits, split_stride=M * N, ldc=N,
                      split_reduce=(self._split_counters, out, accumulate))
            return (1, 0)
        self.gemm(a, b, ws, M=M, N=N, K=K, b_mn=b_mn, epilogue=A.EPI_F32, splits=splits, split_stride=M * N, ldc=N)
        self.reduce_splits(ws, splits, M * N, M * N, out, accumulate)
        return (1, 0)

    def reduce_splits(self, ws, splits: int, stride: int, n: int, out, accumulate: bool) -> None:
        self._call("rte_reduce_splits", _ptr(ws), splits, stride, n, _ptr(out), int(accumulate), self.stream)

    # ------------------------------------------------------------------ embedding / norm / CE
    def embed_fwd(self, tokens, table, out) -> None:
        _require_cuda(tokens, table, out)
        self._call("rte_embed_fwd", _ptr(tokens), _ptr(table), _ptr(out), tokens.numel(), table.shape[1],
                   table.shape[0], _ptr(self.status), self.stream)

    def embed_bwd(self, tokens, dx, dtable, accum) -> None:
        """`accum`: int64 scratch of dtable.numel() elements (fixed-point meeting place of the scatter-add)."""
        if accum.dtype != torch.int64 or accum.numel() < dtable.numel():
            raise ValueError("embed_bwd: accum must be int64 with at least dtable.numel() elements")
        self._call("rte_embed_bwd", _ptr(tokens), _ptr(dx), _ptr(dtable), _ptr(accum), tokens.numel(), dtable.shape[1],
                   dtable.shape[0], _ptr(self.status), self.stream)

    def rmsnorm_fwd(self, x, w, y_bf16, rstd, *, y_f32=None, film_gamma=None, film_beta=None, eps: float = 1e-5,
                    rows: int | None = None) -> None:
        _require_cuda(x, w)
        d = x.shape[-1]
        rows = rows if rows is not None else x.numel() // d
        self._call("rte_rmsnorm_fwd", _ptr(x), _ptr(w), _ptr(film_gamma), _ptr(film_beta), _ptr(y_bf16), _ptr(y_f32),
                   _ptr(rstd), rows, d, eps, self.stream)

    def residual_rmsnorm_fwd(self, base, branch, scale, x_out, w, y_bf16, rstd, *, S: int, active=None, passthrough=None,
                             add2=None, scale2=None, x1_out=None, film_gamma=None, film_beta=None, eps: float = 1e-5,
                             branch_splits: tuple[int, int] = (1, 0), branch_out=None) -> None:
        """x1 = active ? base + scale*branch : passthrough; x = x1 (+ scale2*add2); y = rmsnorm(x)*w (FiLM).
        `branch_splits` = (count, stride): `branch` holds split-K partials, summed in the launch (sum kept in `branch_out`)."""
        d = base.shape[-1]
        self._call("rte_residual_rmsnorm_fwd_splits", _ptr(base), _ptr(branch), branch_splits[0], branch_splits[1],
                   _ptr(branch_out), _ptr(scale), _ptr(active), _ptr(passthrough), S, _ptr(add2), _ptr(scale2), _ptr(x1_out),
                   _ptr(x_out), _ptr(w), _ptr(film_gamma), _ptr(film_beta), _ptr(y_bf16), _ptr(rstd), base.numel() // d, d,
                   eps, self.stream)

    def rmsnorm_bwd(self, x, w, rstd, dy, dres, dx_f32, dx_bf16, dw_out, partial, *, film_gamma=None,
                    dgamma_out=None, dbeta_out=None, partial_g=None, partial_b=None, accumulate_dw: bool = False,
                    accumulate_film: bool = False, rows: int | None = None, dy_splits: tuple[int, int] = (1, 0)) -> None:
        """dx = rmsnorm_backward(dy) + dres; dw_out (+)= column sums (two-stage, deterministic).
        `dy_splits` = (count, stride): `dy` (fp32) holds split-K partials of the gradient, summed in the launch."""
        d = x.shape[-1]
        rows = rows if rows is not None else x.numel() // d
        n_part = C.c_int32(0)
        dy16 = dy if dy.dtype == torch.bfloat16 else None
        dy32 = dy if dy.dtype == torch.float32 else None
        max_partials = partial.shape[0] if partial is not None else 0
        self._call("rte_rmsnorm_bwd_splits", _ptr(x), _ptr(w), _ptr(film_gamma), _ptr(rstd), _ptr(dy16), _ptr(dy32),
                   dy_splits[0], dy_splits[1],
                   _ptr(dres), _ptr(dx_f32), _ptr(dx_bf16), _ptr(partial if dw_out is not None else None),
                   _ptr(partial_g), _ptr(partial_b), rows, d, max_partials, C.byref(n_part), self.stream)
        if dw_out is None and dgamma_out is None:
            return
        jobs = []
        if dw_out is not None:
            jobs.append((partial, dw_out, accumulate_dw))
        if dgamma_out is not None:
            jobs += [(partial_g, dgamma_out, accumulate_film), (partial_b, dbeta_out, accumulate_film)]
        with self._deferred():
            if len(jobs) == 1:
                self._call("rte_colsum_partials", _ptr(jobs[0][0]), n_part.value, d, _ptr(jobs[0][1]), int(jobs[0][2]), self.stream)
            else:                   # norm weight and the two FiLM vectors: one launch
                k = len(jobs)
                parts = (C.c_void_p * k)(*[j[0].data_ptr() for j in jobs])
                outs = (C.c_void_p * k)(*[j[1].data_ptr() for j in jobs])
                acc = (C.c_int32 * k)(*[int(j[2]) for j in jobs])
                self._call("rte_colsum_partials3", parts, outs, acc, k, n_part.value, d, self.stream)

    def ce_fwd_bwd(self, logits, targets, row_weight, S: int, loss_tok, dlogits) -> None:
        rows, V = logits.shape
        self._call("rte_ce_fwd_bwd", _ptr(logits), logits.stride(0), _ptr(targets), _ptr(row_weight), S,
                   _ptr(loss_tok), _ptr(dlogits), rows, V, _ptr(self.status), self.stream)

    def segment_sum(self, src, out, n_seg: int, seg_len: int) -> None:
        self._call("rte_segment_sum", _ptr(src), _ptr(out), n_seg, seg_len, self.stream)

    # ------------------------------------------------------------------ attention
    def rope_table(self, S: int, head_dim: int) -> torch.Tensor:
        """(cos, sin) table [S, head_dim/2, 2] for the attention kernels, built once per (S, head_dim)."""
        key = (S, head_dim)
        if key not in self._rope_tables:
            out = torch.empty(S, head_dim // 2, 2, dtype=torch.float32, device=self.device)
            self._call("rte_rope_table", _ptr(out), S, head_dim, self.stream)
            self._rope_tables[key] = out
        return self._rope_tables[key]

    def identity_rope_table(self, S: int, head_dim: int) -> torch.Tensor:
        """(cos, sin) = (1, 0): attention over q and k that already carry their positions (k_flash_causal_*)."""
        key = (-S, head_dim)
        if key not in self._rope_tables:
            out = torch.zeros(S, head_dim // 2, 2, dtype=torch.float32, device=self.device)
            out[..., 0] = 1.0
            self._rope_tables[key] = out
        return self._rope_tables[key]

    def attn_fwd(self, qkv, y, lse, *, B: int, S: int, n_heads: int, head_dim: int, sec: int | None = None,
                 rope=None) -> None:
        sec = sec if sec is not None else n_heads * head_dim
        rope = rope if rope is not None else self.rope_table(S, head_dim)
        self._call("rte_attn_fwd", _ptr(qkv), qkv.stride(0), sec, _ptr(y), y.stride(0), _ptr(lse),
                   _ptr(rope), B, S, n_heads, head_dim, self.stream)

    def attn_fwd_masked(self, qkv, y, y_masked, lse, mask_row, mask_table, *, B: int, S: int, n_heads: int, head_dim: int,
                        sec: int | None = None, rope=None) -> None:
        """Attention forward plus y_masked = y * mask_table[mask_row[sample]] (one launch on the tensor-core path)."""
        sec = sec if sec is not None else n_heads * head_dim
        rope = rope if rope is not None else self.rope_table(S, head_dim)
        self._call("rte_attn_fwd_masked", _ptr(qkv), qkv.stride(0), sec, _ptr(y), _ptr(y_masked), y.stride(0), _ptr(lse),
                   _ptr(rope), _ptr(mask_row), _ptr(mask_table), B, S, n_heads, head_dim, self.stream)

    def attn_bwd(self, qkv, y, dy, lse, dqkv, *, B: int, S: int, n_heads: int, head_dim: int,
                 sec: int | None = None, rope=None) -> None:
        sec = sec if sec is not None else n_heads * head_dim
        rope = rope if rope is not None else self.rope_table(S, head_dim)
        self._call("rte_attn_bwd", _ptr(qkv), qkv.stride(0), sec, _ptr(y), _ptr(dy), y.stride(0), _ptr(lse),
                   _ptr(dqkv), _ptr(rope), B, S, n_heads, head_dim, self.stream)

    def attn_bwd_masked(self, qkv, y, dy, lse, dqkv, mask_row, mask_table, *, B: int, S: int, n_heads: int, head_dim: int,
                        sec: int | None = None, rope=None) -> None:
        """Attention backward for the upstream gradient dy * mask_table[mask_row[sample]] (dy may be masked in place)."""
        sec = sec if sec is not None else n_heads * head_dim
        rope = rope if rope is not None else self.rope_table(S, head_dim)
        self._call("rte_attn_bwd_masked", _ptr(qkv), qkv.stride(0), sec, _ptr(y), _ptr(dy), y.stride(0), _ptr(lse),
                   _ptr(dqkv), _ptr(rope), _ptr(mask_row), _ptr(mask_table), B, S, n_heads, head_dim, self.stream)

    def rope_apply(self, x, cos, sin, out, *, rows: int, S: int, head_dim: int, adjoint: bool = False) -> None:
        _require_cuda(x, cos, sin, out)
        self._call("rte_rope_apply", _ptr(x), _ptr(cos), _ptr(sin), _ptr(out), rows, S, head_dim,
                   int(x.dtype == torch.bfloat16), int(adjoint), self.stream)

    # ------------------------------------------------------------------ router
    @staticmethod
    def _router_weights(w: dict) -> A.RouterWeights:
        s = A.RouterWeights()
        for name in ("r_w0", "r_b0", "r_w2", "r_b2", "d_w0", "d_b0", "d_w2", "d_b2", "pass_recipe_bias"):
            setattr(s, name, w[name].data_ptr())
        return s

    @staticmethod
    def _router_out(o: dict) -> A.RouterOut:
        s = A.RouterOut()
        for name, _ in A.RouterOut._fields_:
            setattr(s, name, o[name].data_ptr())
        return s

    def router_fwd(self, h0, w: dict, depth_values, out: dict, *, B, S, d, hid, R, K, T, fixed_recipe, fixed_depth_id):
        sw, so = self._router_weights(w), self._router_out(out)
        self._call("rte_router_fwd", _ptr(h0), C.byref(sw), _ptr(depth_values), C.byref(so), B, S, d, hid, R, K, T,
                   -1 if fixed_recipe is None else fixed_recipe, -1 if fixed_depth_id is None else fixed_depth_id,
                   self.stream)

    def router_aux_bwd(self, w: dict, fwd: dict, depth_values, lambda_load, lambda_depth, aux, grads: dict, dh0,
                       scratch, *, B, S, d, hid, R, K, mean_prob=None):
        """`mean_prob` (device f32 [R], optional): the recipe probabilities' mean over the GLOBAL batch (all
        data-parallel shards) to use instead of this batch's own (see rte_router_aux_bwd_data)."""
        sw, so = self._router_weights(w), self._router_out(fwd)
        sg = A.RouterGrads()
        for name, _ in A.RouterGrads._fields_:
            setattr(sg, name, grads[name].data_ptr())
        if mean_prob is None:
            self._call("rte_router_aux_bwd", C.byref(sw), C.byref(so), _ptr(depth_values), lambda_load, lambda_depth,
                       _ptr(aux), C.byref(sg), _ptr(dh0), _ptr(scratch), B, S, d, hid, R, K, self.stream)
            return
        self._call("rte_router_aux_bwd_data", C.byref(sw), C.byref(so), _ptr(depth_values), lambda_load, lambda_depth,
                   _ptr(aux), _ptr(dh0), _ptr(scratch), _ptr(mean_prob), B, S, d, hid, R, K, self.stream)
        self._call("rte_router_aux_bwd_params", C.byref(so), C.byref(sg), _ptr(scratch), B, d, hid, R, K, self.stream)

    def router_mean_prob(self, recipe_probs, out, scale: float, *, B, R) -> None:
        """out[r] = scale * sum_b recipe_probs[b, r] (this rank's share of the global batch mean)."""
        self._call("rte_router_mean_prob", _ptr(recipe_probs), _ptr(out), scale, B, R, self.stream)

    def router_aux_bwd_split(self, w: dict, fwd: dict, depth_values, lambda_load, lambda_depth, aux, grads: dict, dh0,
                             scratch, *, B, S, d, hid, R, K, mean_prob=None):
        """The same backward with the weight gradients on `param_stream` when one is set."""
        sw, so = self._router_weights(w), self._router_out(fwd)
        sg = A.RouterGrads()
        for name, _ in A.RouterGrads._fields_:
            setattr(sg, name, grads[name].data_ptr())
        self._call("rte_router_aux_bwd_data", C.byref(sw), C.byref(so), _ptr(depth_values), lambda_load, lambda_depth,
                   _ptr(aux), _ptr(dh0), _ptr(scratch), _ptr(mean_prob), B, S, d, hid, R, K, self.stream)
        with self._deferred():
            self._call("rte_router_aux_bwd_params", C.byref(so), C.byref(sg), _ptr(scratch), B, d, hid, R, K, self.stream)

    def router_aux_bwd_early(self, w: dict, fwd: dict, depth_values, lambda_load, lambda_depth, aux, grads: dict, scratch, *,
                             B, S, d, hid, R, K, mean_prob=None):
        """Everything of the auxiliary-loss backward except the add into dh0 (no upstream gradient is involved, so
        this may run right after the router's forward); `router_aux_add_dh0` finishes it."""
        sw, so = self._router_weights(w), self._router_out(fwd)
        sg = A.RouterGrads()
        for name, _ in A.RouterGrads._fields_:
            setattr(sg, name, grads[name].data_ptr())
        self._call("rte_router_aux_bwd_data", C.byref(sw), C.byref(so), _ptr(depth_values), lambda_load, lambda_depth,
                   _ptr(aux), None, _ptr(scratch), _ptr(mean_prob), B, S, d, hid, R, K, self.stream)
        self._call("rte_router_aux_bwd_params", C.byref(so), C.byref(sg), _ptr(scratch), B, d, hid, R, K, self.stream)

    def router_aux_add_dh0(self, dh0, scratch, *, B, S, d, hid, R, K) -> None:
        self._call("rte_router_aux_add_dh0", _ptr(dh0), _ptr(scratch), B, S, d, hid, R, K, self.stream)

    def topk_lowest_index(self, scores, k: int, idx, vals=None) -> None:
        rows, n = scores.shape
        self._call("rte_topk_lowest_index", _ptr(scores), scores.stride(0), rows, n, k, _ptr(idx), _ptr(vals), self.stream)

    # ------------------------------------------------------------------ macro operator
    @staticmethod
    def _phi_params(p: dict) -> A.PhiParams:
        s = A.PhiParams()
        for name in ("gain", "v", "u", "bias", "scale"):
            setattr(s, name, p[name].data_ptr())
        wt = p.get("wt")
        s.wt = wt.data_ptr() if wt is not None else None
        s.n_keys = p["gain"].shape[0] * p["gain"].shape[1] if wt is not None else 0
        return s

    def macro_phi_prepare(self, p: dict) -> None:
        """Refreshes p["wt"] (transposed v and u) for the tensor-core forward; call after the parameters changed."""
        R, K, d = p["gain"].shape
        m = p["u"].shape[2]
        if p["wt"].numel() < R * K * (3 * d * m + m * d):
            raise ValueError("macro_phi_prepare: wt too small")
        self._call("rte_macro_phi_prepare", _ptr(p["v"]), _ptr(p["u"]), _ptr(p["wt"]), R * K, d, m, self.stream)

    def macro_phi_fwd(self, h0, p: dict, recipe_id, stride_id, s_cfg, out, rstd, pooled, act, *, B, S, d, m, K):
        sp = self._phi_params(p)
        self._call("rte_macro_phi_fwd", _ptr(h0), C.byref(sp), _ptr(recipe_id), _ptr(stride_id), s_cfg, _ptr(out),
                   _ptr(rstd), _ptr(pooled), _ptr(act), B, S, d, m, K, 1e-5, self.stream)

    def macro_phi_bwd(self, h0, dout, p: dict, recipe_id, stride_id, s_cfg, rstd, pooled, act, dh0, grads: dict,
                      scratch, *, B, S, d, m, R, K):
        sp = self._phi_params(p)
        sg = A.PhiGrads()
        for name, _ in A.PhiGrads._fields_:
            setattr(sg, name, grads[name].data_ptr())
        self._call("rte_macro_phi_bwd", _ptr(h0), _ptr(dout), C.byref(sp), _ptr(recipe_id), _ptr(stride_id), s_cfg,
                   _ptr(rstd), _ptr(pooled), _ptr(act), _ptr(dh0), C.byref(sg), _ptr(scratch), B, S, d, m, R, K,
                   1e-5, self.stream)

    def macro_phi_fwd_hx(self, h, h0, p: dict, recipe_id, stride_id, s_cfg, out, rstd, pooled, act, *, B, S, d, m, K):
        """Phi applied to a state `h` other than the injected `h0` (the consistency term's second application)."""
        sp = self._phi_params(p)
        self._call("rte_macro_phi_fwd_hx", _ptr(h), _ptr(h0), C.byref(sp), _ptr(recipe_id), _ptr(stride_id), s_cfg, _ptr(out),
                   _ptr(rstd), _ptr(pooled), _ptr(act), B, S, d, m, K, 1e-5, self.stream)

    def macro_phi_bwd_hx(self, h, h0, dout, p: dict, recipe_id, stride_id, s_cfg, rstd, pooled, act, dh, dh0, grads: dict,
                         scratch, *, B, S, d, m, R, K):
        """Backward of `macro_phi_fwd_hx`: `dh` overwritten, `dh0` accumulated into, parameter gradients overwritten."""
        sp = self._phi_params(p)
        sg = A.PhiGrads()
        for name, _ in A.PhiGrads._fields_:
            setattr(sg, name, grads[name].data_ptr())
        self._call("rte_macro_phi_bwd_hx", _ptr(h), _ptr(h0), _ptr(dout), C.byref(sp), _ptr(recipe_id), _ptr(stride_id), s_cfg,
                   _ptr(rstd), _ptr(pooled), _ptr(act), _ptr(dh), _ptr(dh0), C.byref(sg), _ptr(scratch), B, S, d, m, R, K,
                   self.stream)

    def sqdiff_grad(self, a, b, coef: float, g, partial, sum_out, accumulate: bool) -> None:
        """g = coef * (a - b); sum_out (+)= sum (a - b)^2 (fixed order)."""
        self._call("rte_sqdiff_grad", _ptr(a), _ptr(b), a.numel(), float(coef), _ptr(g), _ptr(partial), _ptr(sum_out),
                   int(accumulate), self.stream)

    def macro_phi_bwd_split(self, h0, dout, p: dict, recipe_id, stride_id, s_cfg, rstd, pooled, act, dh0, grads: dict,
                            scratch, *, B, S, d, m, R, K):
        """The same backward with its parameter-gradient half on `param_stream` when one is set (nothing downstream
        in backward reads those gradients); the data-gradient half stays on the current stream."""
        sp = self._phi_params(p)
        sg = A.PhiGrads()
        for name, _ in A.PhiGrads._fields_:
            setattr(sg, name, grads[name].data_ptr())
        self._call("rte_macro_phi_bwd_data", _ptr(h0), _ptr(dout), C.byref(sp), _ptr(recipe_id), _ptr(stride_id), s_cfg,
                   _ptr(rstd), _ptr(act), _ptr(dh0), _ptr(scratch), B, S, d, m, K, self.stream)
        with self._deferred():
            self._call("rte_macro_phi_bwd_params", _ptr(h0), _ptr(recipe_id), _ptr(stride_id), _ptr(rstd), _ptr(pooled),
                       _ptr(act), C.byref(sg), _ptr(scratch), B, S, d, m, R, K, self.stream)

    @staticmethod
    def phi_bwd_scratch_floats(B, S, d, m) -> int:
        return B * S * d + B * S * m + 3 * B * d + B * m * d + B * 3 * d * m

    # ------------------------------------------------------------------ vocabulary shortlist
    def shortlist_build(self, targets, top_clusters, random_negs, shortlist, dup_count, *, V, C, TC, HN, RN, K) -> None:
        self._call("rte_shortlist_build", _ptr(targets), _ptr(top_clusters), _ptr(random_negs), _ptr(shortlist),
                   _ptr(dup_count), shortlist.shape[0], V, C, TC, HN, RN, K, _ptr(self.status), self.stream)

    def shortlist_ce(self, hidden, W, shortlist, row_weight, S, loss_tok, logits_out, dlogits_dense) -> None:
        rows, K = shortlist.shape
        self._call("rte_shortlist_ce", _ptr(hidden), _ptr(W), _ptr(shortlist), _ptr(row_weight), S, _ptr(loss_tok),
                   _ptr(logits_out), _ptr(dlogits_dense), rows, hidden.shape[-1], W.shape[0], K, self.stream)

    def shortlist_ce_from_logits(self, logits, shortlist, row_weight, S, loss_tok) -> None:
        """Shortlist cross entropy read from full logits [rows, V]; the row becomes the dense gradient in place."""
        rows, K = shortlist.shape
        self._call("rte_shortlist_ce_from_logits", _ptr(logits), _ptr(shortlist), _ptr(row_weight), S, _ptr(loss_tok), rows,
                   logits.shape[-1], K, self.stream)

    def scatter_cols(self, vals, ids, dense) -> None:
        rows, K = ids.shape
        self._call("rte_scatter_cols_bf16", _ptr(vals), _ptr(ids), _ptr(dense), rows, dense.shape[-1], K, self.stream)

    def random_tokens(self, out, vocab: int, seed) -> None:
        self._call("rte_random_tokens", _ptr(out), out.numel(), vocab, _ptr(seed), self.stream)

    # ------------------------------------------------------------------ exact-audit replay helpers
    def gather_rows(self, src, idx, dst, n: int, row_bytes: int) -> None:
        self._call("rte_gather_rows", _ptr(src), _ptr(idx), _ptr(dst), n, row_bytes, self.stream)

    def scatter_add_rows(self, dst, idx, src, n: int, row_elems: int) -> None:
        self._call("rte_scatter_add_rows_f32", _ptr(dst), _ptr(idx), _ptr(src), n, row_elems, self.stream)

    def audit_route(self, by_pass, depth, idx, rid_out, active_out, n: int, T: int) -> None:
        self._call("rte_audit_route", _ptr(by_pass), _ptr(depth), _ptr(idx), _ptr(rid_out), _ptr(active_out), n, T, self.stream)

    def colmask_mul(self, x, rid, table, S: int, out, rows: int, cols: int) -> None:
        self._call("rte_colmask_mul_bf16", _ptr(x), _ptr(rid), _ptr(table), S, _ptr(out), rows, cols, self.stream)

    def swiglu_masked_fwd(self, ug, rid, table, S: int, z, rows: int, F: int) -> None:
        self._call("rte_swiglu_masked_fwd", _ptr(ug), _ptr(rid), _ptr(table), S, _ptr(z), rows, F, self.stream)

    def swiglu_masked_bwd(self, ug, dz, rid, table, S: int, dug, rows: int, F: int) -> None:
        self._call("rte_swiglu_masked_bwd", _ptr(ug), _ptr(dz), _ptr(rid), _ptr(table), S, _ptr(dug), rows, F, self.stream)

    def scaled_residual_fwd(self, base, branch, scale, active, passthrough, out, n: int, sample_elems: int) -> None:
        self._call("rte_scaled_residual_fwd", _ptr(base), _ptr(branch), _ptr(scale), _ptr(active), _ptr(passthrough),
                   _ptr(out), n, sample_elems, self.stream)

    def scaled_residual_bwd(self, dout, branch, scale, active, dbase, dbranch_bf16, dbranch_f32_accum, dpassthrough,
                            dscale_partial, n: int, sample_elems: int, frozen_active=None, frozen_src=None) -> int:
        """Returns how many per-CTA partial sums of d(scale) were written to `dscale_partial`."""
        n_part = C.c_int32(0)
        cap = dscale_partial.numel() if dscale_partial is not None else 0
        self._call("rte_scaled_residual_bwd", _ptr(dout), _ptr(branch), _ptr(scale), _ptr(active), _ptr(dbase),
                   _ptr(dbranch_bf16), _ptr(dbranch_f32_accum), _ptr(dpassthrough), _ptr(dscale_partial), cap,
                   C.byref(n_part), _ptr(frozen_active), _ptr(frozen_src), n, sample_elems, self.stream)
        return n_part.value

    def macro_distill(self, hot, exact, h0, l_dir, l_rms, l_normed, l_raw, terms, dhot, n: int, S: int, d: int) -> None:
        self._call("rte_macro_distill", _ptr(hot), _ptr(exact), _ptr(h0), l_dir, l_rms, l_normed, l_raw, _ptr(terms),
                   _ptr(dhot), n, S, d, self.stream)

    def kl_distill(self, hot_logits, exact_logits, temp, coef, idx, S: int, dlogits_hot, kl_rows, rows: int, V: int) -> None:
        self._call("rte_kl_distill", _ptr(hot_logits), _ptr(exact_logits), temp, coef, _ptr(idx), S, _ptr(dlogits_hot),
                   dlogits_hot.stride(0), _ptr(kl_rows), rows, V, self.stream)

    def kl_distill_grad(self, hot_logits, exact_logits, temp, coef, dgrad, kl_rows, rows: int, V: int, kl1_rows=None) -> None:
        self._call("rte_kl_distill_grad", _ptr(hot_logits), _ptr(exact_logits), temp, coef, _ptr(dgrad), _ptr(kl_rows),
                   _ptr(kl1_rows), rows, V, self.stream)

    def add_rows_to_bf16(self, dst_bf16, idx, S: int, src_f32, rows: int, V: int) -> None:
        self._call("rte_add_rows_f32_to_bf16", _ptr(dst_bf16), dst_bf16.stride(0), _ptr(idx), S, _ptr(src_f32), rows, V,
                   self.stream)

    def audit_clip(self, hot_loss, exact_loss, idx, n: int, inv_p: float, clip: float, f_hot, f_exact, inv_p_slot=None) -> None:
        self._call("rte_audit_clip", _ptr(hot_loss), _ptr(exact_loss), _ptr(idx), n, float(inv_p),
                   _ptr(inv_p_slot) if inv_p_slot is not None else None, float(clip), _ptr(f_hot), _ptr(f_exact), self.stream)

    def audit_sample_bernoulli(self, entropy, recipe_id, u, perm_table, ema, recent, prm: dict, idx, idx_scatter, valid, inv_p,
                               dist_scale, row_weight, row_weight_a, stats, none_audited=None) -> None:
        """audit.py:62-132 on the device; `prm`: the fields of rte_audit_sample_params."""
        sp = A.AuditSampleParams()
        for k, v in prm.items():
            setattr(sp, k, v)
        self._call("rte_audit_sample_bernoulli", _ptr(entropy), _ptr(recipe_id), _ptr(u),
                   _ptr(perm_table) if perm_table is not None else None, _ptr(ema), _ptr(recent), C.byref(sp), _ptr(idx),
                   _ptr(idx_scatter), _ptr(valid), _ptr(inv_p), _ptr(dist_scale), _ptr(row_weight), _ptr(row_weight_a), _ptr(stats),
                   _ptr(none_audited) if none_audited is not None else None, C.c_void_p(self.status.data_ptr()), self.stream)

    def audit_alignment_sums(self, hot_end, exact_end, h0, n: int, row_len: int, out) -> None:
        self._call("rte_audit_alignment_sums", _ptr(hot_end), _ptr(exact_end), _ptr(h0), n, row_len, _ptr(out), self.stream)

    def scale_rows_f32(self, x, factor, n: int, row_len: int) -> None:
        self._call("rte_scale_rows_f32", _ptr(x), _ptr(factor), n, row_len, self.stream)

    def audit_recent_residual(self, hot_end, exact_end, valid, n: int, row_len: int, cos_scratch, recent) -> None:
        self._call("rte_audit_recent_residual", _ptr(hot_end), _ptr(exact_end), _ptr(valid), n, row_len, _ptr(cos_scratch),
                   _ptr(recent), self.stream)

    def scale_rows_bf16(self, x_bf16, idx, S: int, scale, rows: int, V: int) -> None:
        """x[rows of the samples idx (or the first rows // S samples), :V] *= scale[sample]."""
        self._call("rte_scale_rows_bf16", _ptr(x_bf16), x_bf16.stride(0), _ptr(idx) if idx is not None else None, S, _ptr(scale),
                   rows, V, self.stream)

    # ------------------------------------------------------------------ cluster-pool FFN helpers
    def cluster_route(self, q, centers, assignments, scores=None) -> None:
        n, W = q.shape
        self._call("rte_cluster_route", _ptr(q), q.stride(0), _ptr(centers), _ptr(assignments), _ptr(scores), n, W,
                   centers.shape[0], self.stream)

    def cluster_pack(self, assignments, n_clusters: int, perm, pos, counts, offsets, tile_group, kblocks) -> None:
        self._call("rte_cluster_pack", _ptr(assignments), assignments.numel(), n_clusters, perm.numel(), _ptr(perm),
                   _ptr(pos), _ptr(counts), _ptr(offsets), _ptr(tile_group), _ptr(kblocks), _ptr(self.status), self.stream)

    def gather_rows_convert(self, src, idx, dst) -> None:
        _require_cuda(src, idx, dst)
        self._call("rte_gather_rows_convert", _ptr(src), int(src.dtype == torch.bfloat16), _ptr(idx), _ptr(dst),
                   int(dst.dtype == torch.bfloat16), idx.numel(), dst.shape[-1], self.stream)

    def csr_row_reduce(self, src, row_ptr, rows, dense, accumulate: bool = False) -> None:
        self._call("rte_csr_row_reduce_f32", _ptr(src), _ptr(row_ptr), _ptr(rows), _ptr(dense), dense.shape[0],
                   dense.shape[1], int(accumulate), self.stream)

    def transpose(self, src, dst, accumulate: bool = False) -> None:
        rows, cols = src.shape
        self._call("rte_transpose_f32", _ptr(src), _ptr(dst), rows, cols, int(dst.dtype == torch.bfloat16),
                   int(accumulate), self.stream)

    # ------------------------------------------------------------------ SVD-factor sparse FFN helpers
    def svd_ffn_select(self, hats, ug, wd_norm, z_masked, selected, cand_count, *, up_m, gate_m, product_m, top_k) -> None:
        rows, F = z_masked.shape
        self._call("rte_svd_ffn_select", _ptr(hats), _ptr(ug), _ptr(wd_norm), _ptr(z_masked), _ptr(selected),
                   _ptr(cand_count), rows, F, up_m, gate_m, product_m, top_k, self.stream)

    def svd_ffn_swiglu_bwd(self, ug, dz, selected, dug) -> None:
        rows, F = dz.shape
        self._call("rte_svd_ffn_swiglu_bwd", _ptr(ug), _ptr(dz), _ptr(selected), _ptr(dug), rows, F, self.stream)

    def row_norm(self, w, out) -> None:
        self._call("rte_row_norm_f32", _ptr(w), _ptr(out), w.shape[0], w.shape[1], self.stream)

    def swiglu_fwd(self, ug, z, rows: int, F: int) -> None:
        self._call("rte_swiglu_fwd", _ptr(ug), _ptr(z), rows, F, self.stream)

    def swiglu_bwd(self, ug, dz, dug, rows: int, F: int) -> None:
        self._call("rte_swiglu_bwd", _ptr(ug), _ptr(dz), _ptr(dug), rows, F, self.stream)

    # ------------------------------------------------------------------ small vector ops
    def cast_bf16(self, src, dst) -> None:
        self._call("rte_cast_f32_bf16", _ptr(src), _ptr(dst), src.numel(), self.stream)

    def fill_(self, dst, value: float) -> None:
        self._call("rte_fill_f32", _ptr(dst), value, dst.numel(), self.stream)

    def add_(self, dst, src) -> None:
        self._call("rte_add_f32", _ptr(dst), _ptr(src), dst.numel(), self.stream)

    def axpy_rows(self, dst, vec, alpha: float, rows: int, seg: int, d: int) -> None:
        self._call("rte_axpy_rows_f32", _ptr(dst), _ptr(vec), alpha, rows, seg, d, self.stream)

    # ------------------------------------------------------------------ optimiser
    def adamw(self, plan: "AdamWPlan", beta1, beta2, eps, weight_decay, grad_scale=None, *, skip=None,
              metric_out=None, absent_flag=None, absent_mask=None) -> None:
        """One fused AdamW launch over the plan's tensors.  `skip` (device int32): non-zero drops the update;
        `metric_out` f32 [plan.n_metric_groups, 2]: per-group sums of grad^2 and param^2 (see rte_adamw_multi_tensor_ex);
        `absent_flag` (device int32) + `absent_mask` (device uint8 per plan tensor): tensors without a gradient this step."""
        if skip is None and metric_out is None and absent_flag is None:
            self._call("rte_adamw_multi_tensor", _ptr(plan.table), plan.n_tensors, plan.total_chunks,
                       _ptr(plan.chunk_tensor), _ptr(plan.chunk_index), _ptr(plan.lr_table), _ptr(plan.step_count),
                       beta1, beta2, eps, weight_decay, _ptr(grad_scale), self.stream)
            return
        ex = A.AdamWExtras()
        ex.skip = skip.data_ptr() if skip is not None else None
        if absent_flag is not None:
            ex.absent_flag, ex.absent_mask = absent_flag.data_ptr(), absent_mask.data_ptr()
        if metric_out is not None:
            ex.metric_partial, ex.metric_group = plan.metric_partial.data_ptr(), plan.metric_group.data_ptr()
            ex.metric_out, ex.n_metric_groups = metric_out.data_ptr(), plan.n_metric_groups
        self._call("rte_adamw_multi_tensor_ex", _ptr(plan.table), plan.n_tensors, plan.total_chunks,
                   _ptr(plan.chunk_tensor), _ptr(plan.chunk_index), _ptr(plan.lr_table), _ptr(plan.step_count),
                   beta1, beta2, eps, weight_decay, _ptr(grad_scale), C.byref(ex), self.stream)

    def nonfinite_guard(self, ranges, skip, flag_out=None) -> None:
        """skip[0] = 1 when any element of the (up to three) f32 tensors in `ranges` is NaN or infinite, else 0."""
        r = [t for t in ranges if t is not None and t.numel() > 0][:3]
        r += [None] * (3 - len(r))
        args = []
        for t in r:
            args += [_ptr(t), t.numel() if t is not None else 0]
        self._call("rte_nonfinite_guard", *args, _ptr(skip), _ptr(flag_out), self.stream)

    def add_guarded_(self, dst, src, skip) -> None:
        self._call("rte_add_f32_guarded", _ptr(dst), _ptr(src), dst.numel(), _ptr(skip), self.stream)

    def grad_norm(self, plan: "AdamWPlan", partial, sumsq, max_norm: float, clip_coef) -> None:
        self._call("rte_grad_norm_multi_tensor", _ptr(plan.table), plan.total_chunks, _ptr(plan.chunk_tensor),
                   _ptr(plan.chunk_index), _ptr(partial), _ptr(sumsq), max_norm, _ptr(clip_coef), self.stream)

    def grad_norm_static(self, plan: "AdamWPlan", sumsq, max_norm: float, clip_coef) -> None:
        """Gradient norm through the entry point that uses the library's built-in scratch array (no buffer
        from the caller, no allocation).  Calls on one device must not overlap; see include/rte_b200.h."""
        self._call("rte_grad_norm_multi_tensor_static", _ptr(plan.table), plan.total_chunks, _ptr(plan.chunk_tensor),
                   _ptr(plan.chunk_index), _ptr(sumsq), max_norm, _ptr(clip_coef), self.stream)


class AdamWPlan:
    """Device-resident description of the tensors one fused AdamW launch updates."""

    def __init__(self, entries: list[dict], lr_groups: int, device, n_metric_groups: int = 0):
        """entries: dicts with p, g, m, v (f32 tensors), shadow (bf16 tensor or None), lr_group (int) and, with
        `n_metric_groups` > 0, metric_group (int): the group whose gradient / parameter norms the tensor counts towards."""
        n = len(entries)
        table = (A.AdamWTensor * n)()
        chunk_tensor: list[int] = []
        chunk_index: list[int] = []
        for i, e in enumerate(entries):
            t = table[i]
            t.p, t.g, t.m, t.v = e["p"].data_ptr(), e["g"].data_ptr(), e["m"].data_ptr(), e["v"].data_ptr()
            t.bf16_shadow = e["shadow"].data_ptr() if e.get("shadow") is not None else None
            t.n, t.lr_group, t.step_slot = e["p"].numel(), e["lr_group"], i
            chunks = -(-e["p"].numel() // A.ADAMW_CHUNK)
            chunk_tensor += [i] * chunks
            chunk_index += list(range(chunks))
        raw = bytes(table)
        self.table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
        self.n_tensors = n
        self.total_chunks = len(chunk_tensor)
        self.chunk_tensor = torch.tensor(chunk_tensor, dtype=torch.int32, device=device)
        self.chunk_index = torch.tensor(chunk_index, dtype=torch.int32, device=device)
        self.lr_table = torch.zeros(max(lr_groups, 1), dtype=torch.float32, device=device)
        self.step_count = torch.zeros(n, dtype=torch.int32, device=device)
        self.entries = entries
        self.n_metric_groups = n_metric_groups
        if n_metric_groups > 0:
            self.metric_group = torch.tensor([e["metric_group"] for e in entries], dtype=torch.int32, device=device)
            self.metric_partial = torch.zeros(self.total_chunks, 2, dtype=torch.float32, device=device)
