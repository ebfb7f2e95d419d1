"""TEST-ONLY stand-in for ``speedup_thingy_b200.ops.CudaOps``.

Implements each operator of the C ABI with plain PyTorch on the CPU, following the contract written in
``include/rte_b200.h`` (same argument meaning, same output dtypes, same saved tensors).  It exists so
that the host-side step sequencing in ``engine.py`` -- the hand-written backward pass, buffer reuse,
optimiser plan -- can be checked against the oracle on a machine without a GPU.  It is never imported
by the package; the product path constructs ``CudaOps`` and fails without CUDA.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

EPI_BF16, EPI_F32, EPI_SWIGLU_FWD, EPI_SWIGLU_BWD = 0, 1, 2, 3


def _rope_tables(S, hd):
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
    fr = torch.outer(torch.arange(S, dtype=torch.float32), inv)
    return fr.cos(), fr.sin()          # [S, hd/2]


def _rope(x, cos, sin):               # x [B,H,S,hd] f32, adjacent pairs
    a, b = x[..., ::2], x[..., 1::2]
    return torch.stack((a * cos - b * sin, b * cos + a * sin), dim=-1).flatten(-2)


def _unrope(g, cos, sin):
    a, b = g[..., ::2], g[..., 1::2]
    return torch.stack((a * cos + b * sin, -a * sin + b * cos), dim=-1).flatten(-2)


class EmulOps:
    name = "cpu_emulation_for_tests"

    def __init__(self, device="cpu", sm_count=148):
        self.device = torch.device(device)
        self.sm_count = sm_count
        self.launches = 0
        self._ws = None

    def check_status(self):
        pass

    def split_workspace(self, numel):
        if self._ws is None or self._ws.numel() < numel:
            self._ws = torch.empty(numel, dtype=torch.float32)
        return self._ws

    def pick_splits(self, M, N, K):
        bn = 256 if N >= 192 else 128
        tiles = -(-M // 128) * -(-N // bn)
        kblocks = -(-K // 64)
        want = max(1, min(self.sm_count // max(tiles, 1), kblocks // 8 if kblocks >= 16 else 1, 16))
        while want > 1:
            per = -(-kblocks // want)
            if -(-kblocks // per) == want:
                break
            want -= 1
        return max(want, 1)

    # ---------------------------------------------------------------- GEMM
    def gemm(self, a, b, out, *, M, N, K, a_mn=False, b_mn=False, epilogue=EPI_BF16, residual=None, out2=None,
             pair=0, splits=1, split_stride=0, lda=None, ldb=None, ldc=None, ldr=None, ldc2=None):
        self.launches += 1
        A_ = (a.reshape(K, -1)[:, :M].t() if a_mn else a.reshape(-1, a.shape[-1])[:M, :K]).float()
        B_ = (b.reshape(K, -1)[:, :N].t() if b_mn else b.reshape(-1, b.shape[-1])[:N, :K]).float()
        acc = A_ @ B_.t()
        if epilogue == EPI_BF16:
            out.view(M, -1)[:, :N] = acc.to(torch.bfloat16)
        elif epilogue == EPI_F32:
            if splits > 1:
                ws = out[: splits * split_stride].view(splits, split_stride)
                ws.zero_()
                ws[0, : M * N] = acc.flatten()          # emulation: whole sum in partial 0
            else:
                res = acc if residual is None else acc + residual.view(M, N)
                out.view(-1)[: M * N] = res.flatten()
        elif epilogue == EPI_SWIGLU_FWD:
            f = pair
            up = acc[:, :f].to(torch.bfloat16).float()
            gate = acc[:, f:].to(torch.bfloat16).float()
            out2[:, :f] = up.to(torch.bfloat16)
            out2[:, f:] = gate.to(torch.bfloat16)
            out[:, :f] = (up * F.silu(gate)).to(torch.bfloat16)
        else:
            f = pair
            up, gate = residual[:, :f].float(), residual[:, f:].float()
            sg = torch.sigmoid(gate)
            out[:, :f] = (acc * gate * sg).to(torch.bfloat16)
            out[:, f:] = (acc * up * sg * (1 + gate * (1 - sg))).to(torch.bfloat16)

    def gemm_wgrad(self, a_t, b_t, out, *, M, N, K, accumulate=False, lda=None, ldb=None, ws=None):
        self.launches += 1
        res = a_t.reshape(K, -1)[:, :M].float().t() @ b_t.reshape(K, -1)[:, :N].float()
        if accumulate:
            out.view(M, N).add_(res)
        else:
            out.view(M, N).copy_(res)

    def gemm_f32_few_rows(self, a, b, out, *, M, N, K, b_mn, ws, accumulate=False, reduce=True):
        if not reduce and not accumulate and ws is not None and ws.numel() >= 2 * M * N and K >= 2 and (M * N) % 4 == 0:
            # two partials over the halves of the reduction, left for the consumer to sum (as the split-K launch does)
            self.launches += 1
            A_ = a.reshape(-1, a.shape[-1])[:M, :K].float()
            B_ = (b.reshape(K, -1)[:, :N].t() if b_mn else b.reshape(-1, b.shape[-1])[:N, :K]).float()
            h = K // 2
            ws.view(-1)[: M * N] = (A_[:, :h] @ B_[:, :h].t()).flatten()
            ws.view(-1)[M * N: 2 * M * N] = (A_[:, h:] @ B_[:, h:].t()).flatten()
            return (2, M * N)
        self.gemm(a, b, out, M=M, N=N, K=K, b_mn=b_mn, epilogue=EPI_F32, residual=out if accumulate else None)
        return (1, 0)

    def reduce_splits(self, ws, splits, stride, n, out, accumulate):
        res = ws[: splits * stride].view(splits, stride)[:, :n].sum(0)
        out.view(-1)[:n] = res + (out.view(-1)[:n] if accumulate else 0)

    # ---------------------------------------------------------------- embedding / norm / CE
    def embed_fwd(self, tokens, table, out):
        self.launches += 1
        out.copy_(table[tokens.view(-1)])

    def embed_bwd(self, tokens, dx, dtable, accum=None):
        self.launches += 1
        dtable.index_add_(0, tokens.view(-1), dx)

    def rmsnorm_fwd(self, x, w, y_bf16, rstd, *, y_f32=None, film_gamma=None, film_beta=None, eps=1e-5, rows=None):
        self.launches += 1
        d = x.shape[-1]
        xr = x.reshape(-1, d)
        r = torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + eps)
        y = xr * r
        if w is not None:
            y = y * w
        if film_gamma is not None:
            y = y * (1 + film_gamma) + film_beta
        if rstd is not None:
            rstd.view(-1)[: xr.shape[0]] = r.view(-1)
        if y_bf16 is not None:
            y_bf16.view(-1, d).copy_(y.to(torch.bfloat16))
        if y_f32 is not None:
            y_f32.view(-1, d).copy_(y)

    def residual_rmsnorm_fwd(self, base, branch, scale, x_out, w, y_bf16, rstd, *, S, active=None, passthrough=None,
                             add2=None, scale2=None, x1_out=None, film_gamma=None, film_beta=None, eps=1e-5,
                             branch_splits=(1, 0), branch_out=None):
        d = base.shape[-1]
        if branch_splits[0] > 1:
            n = base.numel()
            parts = branch.view(-1)[: branch_splits[0] * branch_splits[1]].view(branch_splits[0], branch_splits[1])[:, :n]
            branch = parts[0].clone()
            for s in range(1, branch_splits[0]):
                branch = branch + parts[s]
            if branch_out is not None:
                branch_out.view(-1)[:n] = branch
        x1 = base.reshape(-1, d) + scale.reshape(()) * branch.reshape(-1, d)
        if active is not None:
            on = active.bool().repeat_interleave(S)[:, None]
            x1 = torch.where(on, x1, passthrough.reshape(-1, d))
        if x1_out is not None:
            x1_out.copy_(x1.view_as(x1_out))
        x = x1 if add2 is None else x1 + scale2.reshape(()) * add2.reshape(-1, d)
        x_out.copy_(x.view_as(x_out))
        self.rmsnorm_fwd(x_out, w, y_bf16, rstd, film_gamma=film_gamma, film_beta=film_beta, eps=eps)

    def rmsnorm_bwd(self, x, w, rstd, dy, dres, dx_f32, dx_bf16, dw_out, partial, *, film_gamma=None,
                    dgamma_out=None, dbeta_out=None, partial_g=None, partial_b=None, accumulate_dw=False,
                    accumulate_film=False, rows=None, dy_splits=(1, 0)):
        self.launches += 1
        d = x.shape[-1]
        if dy_splits[0] > 1:
            n = x.numel()
            parts = dy.view(-1)[: dy_splits[0] * dy_splits[1]].view(dy_splits[0], dy_splits[1])[:, :n]
            dy = parts[0].clone()
            for s in range(1, dy_splits[0]):
                dy = dy + parts[s]
        xr = x.reshape(-1, d)
        r = rstd.view(-1)[: xr.shape[0]].unsqueeze(-1)
        xh = xr * r
        dyf = dy.reshape(-1, d).float()
        ww = w if w is not None else torch.ones(d)
        f1 = 1 + film_gamma if film_gamma is not None else torch.ones(d)
        g = dyf * f1 * ww
        dx = r * (g - xh * (g * xh).mean(-1, keepdim=True))
        if dres is not None:
            dx = dx + dres.reshape(-1, d)
        if dw_out is not None:
            val = (dyf * f1 * xh).sum(0)
            dw_out.copy_(val + (dw_out if accumulate_dw else 0))
        if dgamma_out is not None:
            dgamma_out.copy_((dyf * xh * ww).sum(0) + (dgamma_out if accumulate_film else 0))
            dbeta_out.copy_(dyf.sum(0) + (dbeta_out if accumulate_film else 0))
        if dx_f32 is not None:
            dx_f32.view(-1, d).copy_(dx)
        if dx_bf16 is not None:
            dx_bf16.view(-1, d).copy_(dx.to(torch.bfloat16))

    def ce_fwd_bwd(self, logits, targets, row_weight, S, loss_tok, dlogits):
        self.launches += 1
        lf = logits.float()
        lse = torch.logsumexp(lf, dim=-1)
        tgt = targets.view(-1)
        loss_tok.copy_(lse - lf.gather(1, tgt[:, None]).squeeze(1))
        if dlogits is not None:
            pr = torch.exp(lf - lse[:, None])
            pr[torch.arange(pr.shape[0]), tgt] -= 1.0
            wgt = row_weight.repeat_interleave(S)[:, None]
            dlogits.copy_((pr * wgt).to(torch.bfloat16))

    def segment_sum(self, src, out, n_seg, seg_len):
        self.launches += 1
        out.view(-1)[:n_seg] = src.view(-1)[: n_seg * seg_len].view(n_seg, seg_len).sum(-1)

    # ---------------------------------------------------------------- attention
    def _split_heads(self, qkv, B, S, H, hd, sec):
        rows = qkv.reshape(B * S, -1).float()
        pick = lambda off: rows[:, off: off + H * hd].view(B, S, H, hd).transpose(1, 2)  # noqa: E731
        return pick(0), pick(sec), pick(2 * sec)

    def attn_fwd(self, qkv, y, lse, *, B, S, n_heads, head_dim, sec=None):
        self.launches += 1
        sec = sec if sec is not None else n_heads * head_dim
        q, k, v = self._split_heads(qkv, B, S, n_heads, head_dim, sec)
        cos, sin = _rope_tables(S, head_dim)
        q = _rope(q, cos, sin).to(torch.bfloat16).float()
        k = _rope(k, cos, sin).to(torch.bfloat16).float()
        sc = (q @ k.transpose(-1, -2)) / math.sqrt(head_dim)
        sc = sc.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
        l = torch.logsumexp(sc, dim=-1)
        out = torch.exp(sc - l[..., None]) @ v
        y.view(B * S, -1)[:, : n_heads * head_dim] = out.transpose(1, 2).reshape(B * S, -1).to(torch.bfloat16)
        lse.view(-1)[: B * n_heads * S] = l.reshape(-1)

    def attn_bwd(self, qkv, y, dy, lse, dqkv, *, B, S, n_heads, head_dim, sec=None):
        self.launches += 1
        sec = sec if sec is not None else n_heads * head_dim
        H, hd = n_heads, head_dim
        q, k, v = self._split_heads(qkv, B, S, H, hd, sec)
        cos, sin = _rope_tables(S, hd)
        q = _rope(q, cos, sin).to(torch.bfloat16).float()
        k = _rope(k, cos, sin).to(torch.bfloat16).float()
        do = dy.reshape(B * S, -1)[:, : H * hd].float().view(B, S, H, hd).transpose(1, 2)
        o = y.reshape(B * S, -1)[:, : H * hd].float().view(B, S, H, hd).transpose(1, 2)
        scale = 1.0 / math.sqrt(hd)
        sc = (q @ k.transpose(-1, -2)) * scale
        mask = torch.ones(S, S, dtype=torch.bool).tril()
        p = torch.exp(sc - lse.view(-1)[: B * H * S].view(B, H, S, 1)).masked_fill(~mask, 0.0)
        dp = do @ v.transpose(-1, -2)
        D = (do * o).sum(-1, keepdim=True)
        ds = p * (dp - D)
        dq = _unrope((ds @ k) * scale, cos, sin)
        dk = _unrope((ds.transpose(-1, -2) @ q) * scale, cos, sin)
        dv = p.transpose(-1, -2) @ do
        rows = dqkv.view(B * S, -1)
        flat = lambda t: t.transpose(1, 2).reshape(B * S, H * hd).to(torch.bfloat16)  # noqa: E731
        rows[:, 0: H * hd] = flat(dq)
        rows[:, sec: sec + H * hd] = flat(dk)
        rows[:, 2 * sec: 2 * sec + H * hd] = flat(dv)

    # ---------------------------------------------------------------- router
    def router_fwd(self, h0, w, depth_values, out, *, B, S, d, hid, R, K, T, fixed_recipe, fixed_depth_id):
        self.launches += 1
        pooled = h0.view(B, S, d).mean(1)
        out["pooled"].copy_(pooled)
        rpre = pooled @ w["r_w0"].t() + w["r_b0"]
        dpre = pooled @ w["d_w0"].t() + w["d_b0"]
        out["r_hidden_pre"].copy_(rpre)
        out["d_hidden_pre"].copy_(dpre)
        rl = F.silu(rpre) @ w["r_w2"].t() + w["r_b2"]
        dl = F.silu(dpre) @ w["d_w2"].t() + w["d_b2"]
        rp, dp = torch.softmax(rl, -1), torch.softmax(dl, -1)
        out["recipe_logits"].copy_(rl)
        out["recipe_probs"].copy_(rp)
        out["depth_probs"].copy_(dp)
        dv = depth_values.float()
        out["expected_depth"].copy_((dp * dv).sum(-1))
        ent = lambda p: -(p.clamp_min(1e-9).log() * p).sum(-1)  # noqa: E731
        out["router_entropy"].copy_(ent(rp) + ent(dp))

        def amax(x):
            mx = x.max(-1, keepdim=True).values
            idx = torch.arange(x.shape[-1]).expand_as(x)
            return torch.where(x == mx, idx, torch.full_like(idx, x.shape[-1])).min(-1).values

        if fixed_recipe is None:
            out["recipe_id"].copy_(amax(rp))
            out["recipe_id_by_pass"].copy_(amax(torch.softmax(rl[:, None, :] + w["pass_recipe_bias"][None], -1)))
        else:
            out["recipe_id"].fill_(fixed_recipe)
            out["recipe_id_by_pass"].fill_(fixed_recipe)
        if fixed_depth_id is None:
            out["depth_id"].copy_(amax(dp))
        else:
            out["depth_id"].fill_(fixed_depth_id)
        out["depth"].copy_(depth_values[out["depth_id"].long()])

    def router_aux_bwd_split(self, *args, **kw):
        self.router_aux_bwd(*args, **kw)

    def router_mean_prob(self, recipe_probs, out, scale, *, B, R):
        out[:R] = recipe_probs.sum(0) * scale

    def router_aux_bwd(self, w, fwd, depth_values, lambda_load, lambda_depth, aux, grads, dh0, scratch, *, B, S, d, hid, R, K,
                       mean_prob=None):
        self.launches += 1
        rp, dp = fwd["recipe_probs"], fwd["depth_probs"]
        mean = rp.mean(0) if mean_prob is None else mean_prob[:R].clone()
        aux[0] = lambda_load * (R * mean.square().sum() - 1.0)
        aux[1] = lambda_depth * fwd["expected_depth"].mean()
        dprob_r = (lambda_load * R * 2.0 * mean / B).expand(B, R)
        dprob_d = (lambda_depth * depth_values.float() / B).expand(B, K)
        dlr = rp * (dprob_r - (rp * dprob_r).sum(-1, keepdim=True))
        dld = dp * (dprob_d - (dp * dprob_d).sum(-1, keepdim=True))

        def back(dlog, pre, w2):
            sg = torch.sigmoid(pre)
            return (dlog @ w2) * sg * (1 + pre * (1 - sg))

        dpr = back(dlr, fwd["r_hidden_pre"], w["r_w2"])
        dpd = back(dld, fwd["d_hidden_pre"], w["d_w2"])
        grads["r_w2"].copy_(dlr.t() @ F.silu(fwd["r_hidden_pre"]))
        grads["r_b2"].copy_(dlr.sum(0))
        grads["d_w2"].copy_(dld.t() @ F.silu(fwd["d_hidden_pre"]))
        grads["d_b2"].copy_(dld.sum(0))
        grads["r_w0"].copy_(dpr.t() @ fwd["pooled"])
        grads["r_b0"].copy_(dpr.sum(0))
        grads["d_w0"].copy_(dpd.t() @ fwd["pooled"])
        grads["d_b0"].copy_(dpd.sum(0))
        dpooled = dpr @ w["r_w0"] + dpd @ w["d_w0"]
        if dh0 is None:
            scratch.view(-1)[:B * d].copy_(dpooled.reshape(-1))
        else:
            dh0.view(B, S, d).add_(dpooled[:, None, :] / S)

    def router_aux_bwd_early(self, w, fwd, depth_values, lambda_load, lambda_depth, aux, grads, scratch, *, B, S, d, hid, R, K,
                             mean_prob=None):
        self.router_aux_bwd(w, fwd, depth_values, lambda_load, lambda_depth, aux, grads, None, scratch, B=B, S=S, d=d,
                            hid=hid, R=R, K=K, mean_prob=mean_prob)

    def router_aux_add_dh0(self, dh0, scratch, *, B, S, d, hid, R, K):
        self.launches += 1
        dh0.view(B, S, d).add_(scratch.view(-1)[:B * d].view(B, 1, d) / S)

    def topk_lowest_index(self, scores, k, idx, vals=None):
        order = torch.sort(-scores.double(), dim=-1, stable=True).indices[:, :k]
        if idx is not None:
            idx.copy_(order)
        if vals is not None:
            vals.copy_(torch.gather(scores, -1, order))

    def swiglu_fwd(self, ug, z, rows, F):
        self.launches += 1
        up, gate = ug[:rows, :F].float(), ug[:rows, F:].float()
        z[:rows] = (up * torch.nn.functional.silu(gate)).to(torch.bfloat16)

    def swiglu_bwd(self, ug, dz, dug, rows, F):
        self.launches += 1
        up, gate, d = ug[:rows, :F].float(), ug[:rows, F:].float(), dz[:rows].float()
        sg = torch.sigmoid(gate)
        dug[:rows, :F] = (d * gate * sg).to(torch.bfloat16)
        dug[:rows, F:] = (d * up * sg * (1 + gate * (1 - sg))).to(torch.bfloat16)

    # ---------------------------------------------------------------- vocabulary shortlist
    def shortlist_build(self, targets, top_clusters, random_negs, shortlist, dup_count, *, V, C, TC, HN, RN, K):
        self.launches += 1
        rows, mpc = shortlist.shape[0], -(-V // C)
        tg = targets.view(-1).tolist()
        for r in range(rows):
            seq = [tg[r]]
            for c in top_clusters[r].tolist():
                seq += [(c + j * C) if c + j * C < V else 0 for j in range(mpc)]
            seq += [p % V for p in range(HN)] + random_negs[r, :RN].tolist() + [p % V for p in range(K)]
            seq += [(tg[r] + p) % V for p in range(2 * K)]
            uniq = list(dict.fromkeys(seq))
            shortlist[r] = torch.tensor(uniq[:K], dtype=shortlist.dtype)
            if dup_count is not None:
                dup_count[r] = len(seq) - len(uniq)

    def shortlist_ce(self, hidden, W, shortlist, row_weight, S, loss_tok, logits_out, dlogits_dense):
        self.launches += 1
        rows, K = shortlist.shape
        lg = torch.einsum("rd,rkd->rk", hidden.float(), W.float()[shortlist.long()]).to(torch.bfloat16).float()
        lse = torch.logsumexp(lg, dim=-1)
        loss_tok.copy_(lse - lg[:, 0])
        if logits_out is not None:
            logits_out.copy_(lg.to(torch.bfloat16))
        if dlogits_dense is not None:
            g = torch.exp(lg - lse[:, None])
            g[:, 0] -= 1.0
            g = g * row_weight.repeat_interleave(S)[:, None]
            dlogits_dense.zero_()
            dlogits_dense.scatter_(1, shortlist.long(), g.to(torch.bfloat16))

    def shortlist_ce_from_logits(self, logits, shortlist, row_weight, S, loss_tok):
        self.launches += 1
        lg = torch.gather(logits.float(), 1, shortlist.long())
        lse = torch.logsumexp(lg, dim=-1)
        loss_tok.copy_(lse - lg[:, 0])
        g = torch.exp(lg - lse[:, None])
        g[:, 0] -= 1.0
        g = g * row_weight.repeat_interleave(S)[:, None]
        logits.zero_()
        logits.scatter_(1, shortlist.long(), g.to(torch.bfloat16))

    # ---------------------------------------------------------------- macro operator (via autograd here)
    def _phi(self, h0, p, rid, sid, s_cfg, B, S, d, m, hx=None):
        h = h0.view(B, S, d)
        hx = h if hx is None else hx.view(B, S, d)
        r, s = rid.long(), sid.long()
        gain, v, u, bias, scale = (p[k][r, s] for k in ("gain", "v", "u", "bias", "scale"))
        rstd = torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5)
        normed = h * rstd
        pooled = normed.mean(1, keepdim=True)
        z = torch.cat([normed, pooled.expand_as(normed), hx], -1)
        act = torch.bmm(z, v)
        low = torch.bmm(F.silu(act), u)
        out = h + s_cfg * scale[:, None] * torch.tanh(gain[:, None] * h + low + bias[:, None])
        return out, rstd, pooled, act

    def macro_phi_fwd(self, h0, p, recipe_id, stride_id, s_cfg, out, rstd, pooled, act, *, B, S, d, m, K):
        self.launches += 1
        o, r, pl, a = self._phi(h0, p, recipe_id, stride_id, s_cfg, B, S, d, m)
        out.view(B, S, d).copy_(o)
        rstd.view(-1)[: B * S] = r.reshape(-1)
        pooled.view(-1)[: B * d] = pl.reshape(-1)
        act.view(B, S, m).copy_(a)

    def macro_phi_bwd_split(self, *args, **kw):
        self.macro_phi_bwd(*args, **kw)

    def sqdiff_grad(self, a, b, coef, g, partial, sum_out, accumulate):
        self.launches += 1
        dv = a.reshape(-1) - b.reshape(-1)
        g.view(-1)[: dv.numel()] = coef * dv
        sum_out[0] = (sum_out[0] if accumulate else 0.0) + dv.double().pow(2).sum().float()

    def macro_phi_fwd_hx(self, h, h0, p, recipe_id, stride_id, s_cfg, out, rstd, pooled, act, *, B, S, d, m, K):
        self.launches += 1
        o, r, pl, a = self._phi(h, p, recipe_id, stride_id, s_cfg, B, S, d, m, hx=h0)
        out.view(B, S, d).copy_(o)
        rstd.view(-1)[: B * S] = r.reshape(-1)
        pooled.view(-1)[: B * d] = pl.reshape(-1)
        act.view(B, S, m).copy_(a)

    def macro_phi_bwd_hx(self, h, h0, dout, p, recipe_id, stride_id, s_cfg, rstd, pooled, act, dh, dh0, grads, scratch, *,
                         B, S, d, m, R, K):
        self.launches += 1
        leaves = {k: p[k].detach().clone().requires_grad_(k != "scale") for k in p if k != "wt"}
        hh, hz = h.detach().clone().requires_grad_(True), h0.detach().clone().requires_grad_(True)
        o, *_ = self._phi(hh, leaves, recipe_id, stride_id, s_cfg, B, S, d, m, hx=hz)
        o.backward(dout.view(B, S, d))
        dh.view(B, S, d).copy_(hh.grad.view(B, S, d))
        dh0.view(B, S, d).add_(hz.grad.view(B, S, d))
        for k in ("gain", "v", "u", "bias"):
            grads[k].copy_(leaves[k].grad if leaves[k].grad is not None else torch.zeros_like(grads[k]))

    def macro_phi_bwd(self, h0, dout, p, recipe_id, stride_id, s_cfg, rstd, pooled, act, dh0, grads, scratch, *, B, S, d, m, R, K):
        self.launches += 1
        leaves = {k: p[k].detach().clone().requires_grad_(k != "scale") for k in p if k != "wt"}
        hh = h0.detach().clone().requires_grad_(True)
        o, *_ = self._phi(hh, leaves, recipe_id, stride_id, s_cfg, B, S, d, m)
        o.backward(dout.view(B, S, d))
        dh0.view(B, S, d).copy_(hh.grad.view(B, S, d))
        for k in ("gain", "v", "u", "bias"):
            grads[k].copy_(leaves[k].grad if leaves[k].grad is not None else torch.zeros_like(grads[k]))

    @staticmethod
    def phi_bwd_scratch_floats(B, S, d, m):
        return 8

    # ---------------------------------------------------------------- exact-audit replay helpers
    def gather_rows(self, src, idx, dst, n, row_bytes):
        self.launches += 1
        per = row_bytes // src.element_size()
        dst.view(-1)[: n * per].view(n, per).copy_(src.reshape(-1, per)[idx[:n].long()])

    def scatter_add_rows(self, dst, idx, src, n, row_elems):
        self.launches += 1
        keep = idx[:n] >= 0
        dst.view(-1, row_elems).index_add_(0, idx[:n][keep].long(), src.view(-1)[: n * row_elems].view(n, row_elems)[keep])

    def audit_route(self, by_pass, depth, idx, rid_out, active_out, n, T):
        self.launches += 1
        ii = idx[:n].long()
        rid_out.view(T, n).copy_(by_pass.view(-1, T)[ii].t())
        active_out.view(T, n).copy_((depth[ii][None, :] > torch.arange(T)[:, None]).int())

    def colmask_mul(self, x, rid, table, S, out, rows, cols):
        self.launches += 1
        m = table.view(-1, cols)[rid.long()].repeat_interleave(S, 0)[:rows]
        out.view(rows, cols).copy_((x.view(rows, cols).float() * m).to(torch.bfloat16))

    def swiglu_masked_fwd(self, ug, rid, table, S, z, rows, F_):
        self.launches += 1
        m = table.view(-1, F_)[rid.long()].repeat_interleave(S, 0)[:rows]
        u, g = ug.view(rows, 2 * F_)[:, :F_].float(), ug.view(rows, 2 * F_)[:, F_:].float()
        z.view(rows, F_).copy_((u * F.silu(g) * m).to(torch.bfloat16))

    def swiglu_masked_bwd(self, ug, dz, rid, table, S, dug, rows, F_):
        self.launches += 1
        m = table.view(-1, F_)[rid.long()].repeat_interleave(S, 0)[:rows]
        u, g = ug.view(rows, 2 * F_)[:, :F_].float(), ug.view(rows, 2 * F_)[:, F_:].float()
        d = dz.view(rows, F_).float() * m
        sg = torch.sigmoid(g)
        dug.view(rows, 2 * F_)[:, :F_] = (d * g * sg).to(torch.bfloat16)
        dug.view(rows, 2 * F_)[:, F_:] = (d * u * sg * (1 + g * (1 - sg))).to(torch.bfloat16)

    def scaled_residual_fwd(self, base, branch, scale, active, passthrough, out, n, sample_elems):
        self.launches += 1
        res = base.view(n, -1) + float(scale) * branch.view(n, -1)
        if active is not None:
            res = torch.where(active.view(n, 1) != 0, res, passthrough.view(n, -1))
        out.view(n, -1).copy_(res)

    def scaled_residual_bwd(self, dout, branch, scale, active, dbase, dbranch_bf16, dbranch_f32_accum, dpassthrough,
                            dscale_partial, n, sample_elems, frozen_active=None, frozen_src=None):
        self.launches += 1
        on = torch.ones(n, 1, dtype=torch.bool) if active is None else (active.view(n, 1) != 0)
        g = dout.view(n, -1).clone()
        s = float(scale)
        if dscale_partial is not None:
            dscale_partial.zero_()
            dscale_partial[0] = (torch.where(on, g, torch.zeros_like(g)) * branch.view(n, -1)).sum()
        if dpassthrough is not None:
            dpassthrough.view(n, -1).add_(torch.where(on, torch.zeros_like(g), g))
        if dbranch_bf16 is not None:
            dbranch_bf16.view(n, -1).copy_(torch.where(on, s * g, torch.zeros_like(g)).to(torch.bfloat16))
        if dbranch_f32_accum is not None:
            dbranch_f32_accum.view(n, -1).add_(torch.where(on, s * g, torch.zeros_like(g)))
        if dbase is not None:
            base = torch.where(on, g, torch.zeros_like(g))
            if frozen_src is not None:
                frozen = frozen_active.view(n, 1) == 0
                base = base + torch.where(frozen, frozen_src.view(n, -1), torch.zeros_like(g))
            dbase.view(n, -1).copy_(base)
        return 1

    def macro_distill(self, hot, exact, h0, l_dir, l_rms, l_normed, l_raw, terms, dhot, n, S, d):
        self.launches += 1
        h = hot.view(n, S, d).detach().clone().requires_grad_(True)
        e, z = exact.view(n, S, d), h0.view(n, S, d)
        dp, de = h - z, e - z
        cos = F.cosine_similarity(dp.flatten(1), de.flatten(1), dim=-1, eps=1e-8)
        rms = lambda x: x.pow(2).mean(dim=(1, 2)).sqrt().clamp_min(1e-8)  # noqa: E731
        diff2 = (torch.log(rms(dp)) - torch.log(rms(de))).square()
        nrm = lambda x: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)  # noqa: E731
        sl_n = F.smooth_l1_loss(nrm(h), nrm(e), reduction="none").sum(dim=(1, 2))
        sl_r = F.smooth_l1_loss(h, e, reduction="none").sum(dim=(1, 2))
        total = l_dir * (1 - cos).mean() + l_rms * diff2.mean() + (l_normed * sl_n.sum() + l_raw * sl_r.sum()) / (n * S * d)
        total.backward()
        terms.view(n, 4).copy_(torch.stack([1 - cos, diff2, sl_n, sl_r], dim=1).detach())
        dhot.view(n, S, d).copy_(h.grad)

    def kl_distill(self, hot_logits, exact_logits, temp, coef, idx, S, dlogits_hot, kl_rows, rows, V):
        self.launches += 1
        lh = torch.log_softmax(hot_logits.view(rows, V).float() / temp, -1)
        le = torch.log_softmax(exact_logits.view(rows, V).float() / temp, -1)
        kl_rows.view(-1)[:rows] = (le.exp() * (le - lh)).sum(-1)
        n = rows // S
        tgt = (idx[:n].long()[:, None] * S + torch.arange(S)[None, :]).reshape(-1)
        cur = dlogits_hot[tgt, :V].float()
        dlogits_hot[tgt, :V] = (cur + coef * (lh.exp() - le.exp())).to(torch.bfloat16)

    def attn_bwd_masked(self, qkv, y, dy, lse, dqkv, mask_row, mask_table, *, B, S, n_heads, head_dim, sec=None, rope=None):
        self.colmask_mul(dy, mask_row, mask_table, S, dy, B * S, n_heads * head_dim)
        self.attn_bwd(qkv, y, dy, lse, dqkv, B=B, S=S, n_heads=n_heads, head_dim=head_dim, sec=sec)

    def attn_fwd_masked(self, qkv, y, y_masked, lse, mask_row, mask_table, *, B, S, n_heads, head_dim, sec=None, rope=None):
        self.attn_fwd(qkv, y, lse, B=B, S=S, n_heads=n_heads, head_dim=head_dim, sec=sec)
        self.colmask_mul(y, mask_row, mask_table, S, y_masked, B * S, n_heads * head_dim)

    def macro_phi_prepare(self, p):
        pass

    def kl_distill_grad(self, hot_logits, exact_logits, temp, coef, dgrad, kl_rows, rows, V, kl1_rows=None):
        self.launches += 1
        lh = torch.log_softmax(hot_logits.view(rows, V).float() / temp, -1)
        le = torch.log_softmax(exact_logits.view(rows, V).float() / temp, -1)
        kl_rows.view(-1)[:rows] = (le.exp() * (le - lh)).sum(-1)
        if dgrad is not None:
            dgrad.view(rows, V).copy_(coef * (lh.exp() - le.exp()))
        if kl1_rows is not None:
            lh1 = torch.log_softmax(hot_logits.view(rows, V).float(), -1)
            le1 = torch.log_softmax(exact_logits.view(rows, V).float(), -1)
            kl1_rows.view(-1)[:rows] = (le1.exp() * (le1 - lh1)).sum(-1)

    def add_rows_to_bf16(self, dst_bf16, idx, S, src_f32, rows, V):
        self.launches += 1
        n = rows // S
        keep = (idx[:n] >= 0).repeat_interleave(S)
        tgt = (idx[:n].long()[:, None] * S + torch.arange(S)[None, :]).reshape(-1)[keep]
        dst_bf16[tgt, :V] = (dst_bf16[tgt, :V].float() + src_f32.view(rows, V)[keep]).to(torch.bfloat16)

    def audit_clip(self, hot_loss, exact_loss, idx, n, inv_p, clip, f_hot, f_exact, inv_p_slot=None):
        self.launches += 1
        r = exact_loss[:n] - hot_loss[idx[:n].long()]
        inside = r.abs() <= clip
        ip = inv_p_slot[:n] if inv_p_slot is not None else torch.full_like(r, inv_p)
        f_hot[:n] = torch.where(inside, 1.0 - ip, torch.ones_like(r))
        f_exact[:n] = inside.float()

    def audit_sample_bernoulli(self, entropy, recipe_id, u, perm_table, ema, recent, prm, idx, idx_scatter, valid, inv_p,
                               dist_scale, row_weight, row_weight_a, stats, none_audited=None):
        self.launches += 1
        B, R, cap, n_cap = prm["B"], prm["R"], prm["cap"], prm["n_cap"]
        rid = recipe_id[:B].long()
        deficit = (prm["coverage_min"] - ema[rid]).clamp_min(0.0) / max(prm["coverage_min"], 1e-12)
        p = prm["p_min"] + prm["alpha"] * (entropy[:B] * prm["inv_r_plus_k"]) + prm["beta"] * recent[0] + prm["gamma"] * deficit
        p = p.clamp(prm["p_min"], prm["p_max"])
        mask = u[:B] < p
        cand = int(mask.sum())
        p_inc = p.clone()
        if cap >= 0 and cand > cap:
            sel = mask.nonzero().flatten()
            perm = perm_table.view(-1, cap)[cand - cap - 1].long()
            mask = torch.zeros_like(mask)
            mask[sel[perm]] = True
            p_inc = p * (float(cap) / float(cand))
        chosen = mask.nonzero().flatten()
        a = int(chosen.numel())
        if a > n_cap:
            if not hasattr(self, "status"):
                raise RuntimeError("device status 202: more audited samples than the replay's capacity")
            self.status[0] = 202
            chosen, a = chosen[:n_cap], n_cap
        ip = 1.0 / p_inc.clamp_min(1e-12)
        idx.zero_(); idx_scatter.fill_(-1); valid.zero_(); inv_p.zero_(); dist_scale.zero_(); row_weight_a.zero_()
        idx[:a] = chosen.int(); idx_scatter[:a] = chosen.int(); valid[:a] = 1.0; inv_p[:a] = ip[chosen]
        dist_scale[:a] = float(n_cap) / max(a, 1)
        row_weight_a[:a] = prm["w0"] * ip[chosen]
        row_weight[:B] = prm["w0"]
        if prm["weight_mode"] == 1:
            row_weight[chosen] = prm["w0"] * (1.0 - ip[chosen])
        counts = torch.bincount(rid[mask], minlength=R).float()
        ema[:R] = ema[:R] * prm["coverage_beta"] + counts / max(float(mask.sum()), 1.0) * (1.0 - prm["coverage_beta"])
        stats[0], stats[1], stats[2], stats[3] = float(cand), float(mask.sum()), float(p.mean()), float(p_inc.mean())
        if none_audited is not None:
            none_audited[0] = int(a == 0)

    def audit_alignment_sums(self, hot_end, exact_end, h0, n, row_len, out):
        self.launches += 1
        a, b, z = (t.reshape(-1)[: n * row_len].view(n, row_len).double() for t in (hot_end, exact_end, h0))
        o = out.view(-1)[: n * 8].view(n, 8)
        cols = [(a * b), (a * a), (b * b), (a - b) ** 2, (a - z) ** 2, (b - z) ** 2, (a - z) * (b - z)]
        for k, c in enumerate(cols):
            o[:, k] = c.sum(-1).float()             # (column 7 is the caller's)

    def scale_rows_f32(self, x, factor, n, row_len):
        self.launches += 1
        x.view(-1)[: n * row_len].view(n, row_len).mul_(factor[:n, None])

    def audit_recent_residual(self, hot_end, exact_end, valid, n, row_len, cos_scratch, recent):
        self.launches += 1
        a, b = hot_end.view(-1)[: n * row_len].view(n, row_len), exact_end.view(-1)[: n * row_len].view(n, row_len)
        cos = F.cosine_similarity(a, b, dim=-1, eps=1e-8)
        cos_scratch[:n] = cos
        if float(valid[:n].sum()) > 0:
            recent[0] = (1.0 - (valid[:n] * cos).sum() / valid[:n].sum()).clamp_min(0.0)

    def scale_rows_bf16(self, x_bf16, idx, S, scale, rows, V):
        self.launches += 1
        n = rows // S
        base = idx[:n].long() if idx is not None else torch.arange(n)
        keep = (base >= 0).repeat_interleave(S)
        tgt = (base[:, None] * S + torch.arange(S)[None, :]).reshape(-1)[keep]
        f = scale[:n].repeat_interleave(S)[keep][:, None]
        x_bf16[tgt, :V] = (x_bf16[tgt, :V].float() * f).to(torch.bfloat16)

    # ---------------------------------------------------------------- small vector ops
    def cast_bf16(self, src, dst):
        self.launches += 1
        dst.copy_(src.to(torch.bfloat16))

    def fill_(self, dst, value):
        dst.fill_(value)

    def add_(self, dst, src):
        dst.add_(src)

    def axpy_rows(self, dst, vec, alpha, rows, seg, d):
        dst.view(rows, d).add_(vec.view(-1, d).repeat_interleave(seg, 0)[:rows] * alpha)

    # ---------------------------------------------------------------- optimiser
    def nonfinite_guard(self, ranges, skip, flag_out=None):
        bad = any(t is not None and t.numel() and not bool(torch.isfinite(t).all()) for t in ranges)
        skip[0] = int(bad)
        if flag_out is not None:
            flag_out[0] = float(bad)

    def add_guarded_(self, dst, src, skip):
        if int(skip[0]) == 0:
            dst.add_(src)

    def adamw(self, plan, beta1, beta2, eps, weight_decay, grad_scale=None, *, skip=None, metric_out=None, absent_flag=None,
              absent_mask=None):
        self.launches += 1
        if skip is not None and int(skip[0]) != 0:
            if metric_out is not None:
                metric_out.zero_()
            return
        gs = float(grad_scale) if grad_scale is not None else 1.0
        if metric_out is not None:
            metric_out.zero_()
            for i, e in enumerate(plan.entries):
                if absent_flag is not None and int(absent_flag[0]) and int(absent_mask[i]):
                    continue
                metric_out[e["metric_group"], 0] += float((e["g"] * gs).double().pow(2).sum())
                metric_out[e["metric_group"], 1] += float(e["p"].double().pow(2).sum())
        for i, e in enumerate(plan.entries):
            if absent_flag is not None and int(absent_flag[0]) and int(absent_mask[i]):
                continue                      # no gradient this step: torch.optim.AdamW leaves the tensor alone
            lr = float(plan.lr_table[e["lr_group"]])
            step = int(plan.step_count[i]) + 1
            g = e["g"] * gs
            e["p"].mul_(1 - lr * weight_decay)
            e["m"].mul_(beta1).add_(g, alpha=1 - beta1)
            e["v"].mul_(beta2).addcmul_(g, g, value=1 - beta2)
            bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
            e["p"].addcdiv_(e["m"], e["v"].sqrt() / math.sqrt(bc2) + eps, value=-lr / bc1)
            if e.get("shadow") is not None:
                e["shadow"].copy_(e["p"].to(torch.bfloat16))
            plan.step_count[i] = step

    def grad_norm(self, plan, partial, sumsq, max_norm, clip_coef):
        self.launches += 1
        s = sum(float(e["g"].double().pow(2).sum()) for e in plan.entries)
        sumsq[0] = s
        if clip_coef is not None:
            clip_coef[0] = min(1.0, max_norm / (math.sqrt(s) + 1e-6)) if max_norm > 0 else 1.0
