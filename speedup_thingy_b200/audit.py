"""Exact-audit replay of the `recursive_macro` step, kept on the device.

Reference: ``AuditEngine.correction`` (audit.py:245-387) with the fixed-count sampler (audit.py:99-116),
``RecursiveModel.forward_exact_subset`` -> ``forward_exact_from_h0`` (models.py:605-679, 416-512),
``BankedRecursiveCore.forward_step`` / ``step_group`` (layers.py:831-870), ``macro_distill_loss``
(macro.py:394-469, delta objective) and the control variate ``hot + (exact - hot) / p``.

The audited samples (k per batch, chosen on the host with the same seeded CPU permutation the reference
draws) are replayed through the banked core for ``t_max`` passes.  A recipe selects heads / FFN slabs /
banks; here every pass computes all columns of every bank and multiplies by the recipe's column mask looked
up on the device from the router's per-pass choice, so tensor shapes never depend on routing and the replay
is part of the step's CUDA graph.  The replay's gradients flow into the core, the coda, the tied embedding
and -- through the cached h0 -- the prelude, exactly as under ``audit_mode: gradient_corrected``.
"""
from __future__ import annotations

import math

import torch

from . import _abi as A


def next_fixed_count(tr, current: int, metrics: dict, batch_size: int, state: dict) -> int:
    """The fixed-count schedule's decision (audit.py:137-185) from the metrics of a step that audited somebody: halve
    the count (not below `audit_schedule_min_count`, default batch // 128) when the loss residual, the endpoints'
    cosine, mse, delta-RMS ratio and norm and the residual variance all pass their thresholds and -- where asked --
    mse and norm did not rise since the last such step (`state`); double it, up to the batch, otherwise.  A metric
    that is missing fails its test."""
    if not tr.audit_schedule_enabled or current <= 0:
        return current
    get = lambda key, default: float(metrics.get(key, default))            # noqa: E731
    floor = tr.audit_schedule_min_count if tr.audit_schedule_min_count is not None else max(1, batch_size // 128)
    # (the reference looks the loss gap up in the audit's own metrics, where only `loss_residual` exists at that point:
    #  the mean of exact - hot over the audited samples' summed token losses, before any clip)
    gap = abs(get("loss_residual", math.inf))
    mse, norm = get("hidden_mse_exact_macro", math.inf), get("macro_norm", math.inf)
    limit = tr.audit_schedule_macro_norm_threshold
    if limit is None:
        limit = tr.audit_schedule_macro_norm_threshold_mult * get("exact_norm", 0.0)
    rising_mse = state.get("mse") is not None and mse - state["mse"] > 0
    rising_norm = state.get("norm") is not None and norm - state["norm"] > 0
    state["mse"], state["norm"] = mse, norm
    ratio = get("delta_rms_ratio", math.inf)
    tracked = (gap <= tr.audit_schedule_nll_gap_threshold
               and get("hidden_cosine_exact_macro", 0.0) >= tr.audit_schedule_hidden_cosine_threshold
               and tr.audit_schedule_delta_rms_ratio_min <= ratio <= tr.audit_schedule_delta_rms_ratio_max
               and mse <= tr.audit_schedule_hidden_mse_threshold and norm <= limit
               and get("audit_residual_var", math.inf) <= tr.audit_schedule_residual_var_threshold
               and not (tr.audit_schedule_require_negative_mse_slope and rising_mse)
               and not (tr.audit_schedule_require_negative_norm_slope and rising_norm))
    return max(floor, current // 2) if tracked else min(batch_size, current * 2)


def build_recipes(cfg) -> list[dict]:
    """Static recipe templates (recipes.py:65-100): recipe 0 = dense fallback over all banks and groups."""
    out = [dict(attn_banks=tuple(range(cfg.attn_banks)), ffn_banks=tuple(range(cfg.ffn_banks)),
                head_groups=tuple(range(cfg.head_groups)), ffn_groups=tuple(range(cfg.ffn_groups)))]
    head_slots = max(1, cfg.head_groups // cfg.active_head_groups)
    ffn_slots = max(1, cfg.ffn_groups // cfg.active_ffn_groups)
    for idx in range(cfg.recipe_count - 1):
        hs = (idx % head_slots) * cfg.active_head_groups
        fs = (idx % ffn_slots) * cfg.active_ffn_groups
        out.append(dict(attn_banks=((idx // head_slots) % cfg.attn_banks,), ffn_banks=((idx // ffn_slots) % cfg.ffn_banks,),
                        head_groups=tuple((hs + j) % cfg.head_groups for j in range(cfg.active_head_groups)),
                        ffn_groups=tuple((fs + j) % cfg.ffn_groups for j in range(cfg.active_ffn_groups))))
    return out


def recipe_mask_tables(cfg, device) -> tuple[torch.Tensor, torch.Tensor]:
    """head_tab [attn_banks, R, d] and ffn_tab [ffn_banks, R, F]: 1/len(banks of the recipe) on the columns the
    recipe activates in a bank it uses, 0 elsewhere (layers.py:673-700,728,744-763,779)."""
    d, f, hd = cfg.d_model, cfg.d_ff, cfg.d_model // cfg.n_heads
    hpg, slab = cfg.n_heads // cfg.head_groups, cfg.d_ff // cfg.ffn_groups
    recipes = build_recipes(cfg)
    head = torch.zeros(cfg.attn_banks, len(recipes), d)
    ffn = torch.zeros(cfg.ffn_banks, len(recipes), f)
    for r, rec in enumerate(recipes):
        for bank in rec["attn_banks"]:
            for grp in rec["head_groups"]:
                head[bank, r, grp * hpg * hd:(grp + 1) * hpg * hd] = 1.0 / len(rec["attn_banks"])
        for bank in rec["ffn_banks"]:
            for grp in rec["ffn_groups"]:
                ffn[bank, r, grp * slab:(grp + 1) * slab] = 1.0 / len(rec["ffn_banks"])
    return head.to(device), ffn.to(device)


CORE_PARAMS = ["core.pass_gamma1", "core.pass_beta1", "core.pass_gamma2", "core.pass_beta2", "core.pass_attn_scale",
               "core.pass_mlp_scale", "core.alpha_inj", "core.norm1.weight", "core.attn.wqkv", "core.attn.wo",
               "core.norm2.weight", "core.mlp.wug", "core.mlp.wd"]
CORE_SHADOWED = ["core.attn.wqkv", "core.attn.wo", "core.mlp.wug", "core.mlp.wd"]


class AuditReplay:
    """Buffers and launch sequences of the replay; owned by ``TrainEngine`` (``eng``)."""

    def __init__(self, eng, k: int, direct_grads: bool = False):
        """`direct_grads`: write the gradients of final norm / coda / embedding straight into the engine's buffers
        (the `recursive_exact` mode, where no hot pass shares them) instead of a private mirror."""
        from .engine import _Block, _Temps

        self.eng, self.k = eng, k
        self._stage = None
        self._prepared = None
        self._prelude_copied = None
        self._core_fwd_done = self.distill_done = None
        self.fixed_rid = None                        # [T, n] int32 when `recursive_exact` runs a fixed recipe schedule
        self.deferred_depth = 0                      # branches of the grouped block (recursive_deferred_grouped_exact)
        cfg, dev = eng.cfg, eng.device
        self.n, self.S, self.T = k, eng.S, cfg.t_max
        self.Ma = k * eng.S
        n, S, T, Ma, d, f, V = self.n, self.S, self.T, self.Ma, cfg.d_model, cfg.d_ff, cfg.vocab_size
        f32, bf, i32 = torch.float32, torch.bfloat16, torch.int32
        e = lambda *shape, dtype=f32: torch.zeros(*shape, dtype=dtype, device=dev)  # noqa: E731
        self.p_inc = float(k) / float(eng.B)                              # inclusion probability k/n (audit.py:116)
        # Bernoulli sampler (audit.py:79-132): the subset is drawn ON THE DEVICE from this step's routing; `k` is then
        # the capacity of the replay's buffers, slots beyond the audited count carry weight 0
        self.bernoulli = (not direct_grads) and getattr(eng, "audit_bernoulli", False)
        # Fixed-count schedule (audit.py:137-185): the host draws the subset as for a fixed count, but the count changes
        # between steps; `k` is again a capacity, and the host stages what the Bernoulli kernel writes on the device
        self.scheduled = (not direct_grads) and getattr(eng, "audit_scheduled", False)
        self.padded = self.bernoulli or self.scheduled       # slots beyond the step's audited count carry weight 0
        self.grad = direct_grads or eng.tr.audit_mode == "gradient_corrected"      # does the replay carry gradients
        self.clip = eng.tr.audit_residual_clip if (self.grad and not direct_grads) else None
        # (the reported control variate is clipped in every audit mode, audit.py:311-318; `clip` is the device side)
        self.clip_reported = None if direct_grads else eng.tr.audit_residual_clip
        self.f_hot, self.f_exact = e(n), e(n)                             # residual clip: per-sample gradient factors
        self.align = e(n, 8)                                              # alignment sums (the engine points it at the results)
        self.idx = e(n, dtype=i32)
        self.head_tab, self.ffn_tab = recipe_mask_tables(cfg, dev)
        self.rid, self.active = e(T, n, dtype=i32), e(T, n, dtype=i32)
        self.h0a, self.targets_a = e(Ma, d), e(Ma, dtype=torch.int64)
        self.h = [self.h0a] + [e(Ma, d) for _ in range(T)]                 # h[0] = the gathered h0 rows, h[t+1] = after pass t
        self.ht, self.u = [e(Ma, d) for _ in range(T)], [e(Ma, d) for _ in range(T)]
        # With one attention and one FFN bank, what the weight-gradient products of the T passes read is laid out pass
        # after pass in one tensor each, so that a weight's gradient is ONE product over T * Ma rows after the last
        # pass instead of T products that each rewrite the whole fp32 gradient (RTE_REPLAY_FUSED_WGRAD=0: per pass).
        import os
        self.fused_wgrad = (cfg.attn_banks == 1 and cfg.ffn_banks == 1 and os.environ.get("RTE_REPLAY_FUSED_WGRAD", "1") != "0")
        self._stacked: dict[str, torch.Tensor] = {}
        # the norm launches behind the core's split-K few-row products sum the partials themselves (one dependent
        # launch less per product; RTE_REPLAY_SPLIT_FEED=0: a separate reduction launch)
        self.split_feed = os.environ.get("RTE_REPLAY_SPLIT_FEED", "1") != "0"

        def per_pass(name: str, cols: int) -> list[torch.Tensor]:
            if not self.fused_wgrad:
                return [e(Ma, cols, dtype=bf) for _ in range(T)]
            self._stacked[name] = e(T * Ma, cols, dtype=bf)
            return [self._stacked[name][t * Ma:(t + 1) * Ma] for t in range(T)]

        self.n1, self.n2 = per_pass("n1", d), per_pass("n2", d)
        self.rstd1, self.rstd2 = [e(Ma) for _ in range(T)], [e(Ma) for _ in range(T)]
        self.attn_acc, self.mlp_acc = [e(Ma, d) for _ in range(T)], [e(Ma, d) for _ in range(T)]
        ab, fb, H = cfg.attn_banks, cfg.ffn_banks, cfg.n_heads
        self.qkv = [[e(Ma, 3 * d, dtype=bf) for _ in range(ab)] for _ in range(T)]
        self.y = [[e(Ma, d, dtype=bf) for _ in range(ab)] for _ in range(T)]
        self.ym = [[x] for x in per_pass("ym", d)] if self.fused_wgrad else [[e(Ma, d, dtype=bf) for _ in range(ab)] for _ in range(T)]
        self.lse = [[e(n * H * S) for _ in range(ab)] for _ in range(T)]
        self.ug = [[e(Ma, 2 * f, dtype=bf) for _ in range(fb)] for _ in range(T)]
        self.zm = [[x] for x in per_pass("zm", f)] if self.fused_wgrad else [[e(Ma, f, dtype=bf) for _ in range(fb)] for _ in range(T)]
        self.coda = [_Block(f"coda.{i}@audit", Ma, cfg, n, S, dev) for i in range(cfg.n_coda)]
        self.tmp = _Temps(Ma, cfg, dev)
        self.hidden16, self.rstd_f = e(Ma, d, dtype=bf), e(Ma)
        self.logits, self.hot_logits = e(Ma, V, dtype=bf), e(Ma, V, dtype=bf)
        self.loss_tok, self.exact_loss = e(Ma), e(n)
        self.hot_end = e(Ma, d)
        self.terms, self.dhot_extra, self.kl_rows, self.kl_sum = e(n, 4), e(Ma, d), e(Ma), e(1)
        self.kl1_rows = e(Ma)
        self.dkl = e(Ma, V)
        self.row_weight_a = torch.full((n,), 1.0 / (eng.B * eng.S * eng.loss_div) / self.p_inc, dtype=f32, device=dev)
        self.idx_scatter = self.idx                    # padded subsets: a second index list with -1 on unused slots
        if self.scheduled:
            # one staging copy fills: idx_scatter | valid | dist_scale | the replay's loss weights
            self.sched_pack = e(4 * n)
            self.idx_scatter = self.sched_pack[0:n].view(i32)
            self.valid, self.dist_scale, self.row_weight_a = (self.sched_pack[j * n:(j + 1) * n] for j in (1, 2, 3))
            self.count = int(eng.audit_count0)         # this step's count; `update_schedule` sets the next one
            self.schedule_state: dict = {}             # mse and norm of the last audited step (the slope tests)
        if self.bernoulli:
            tr, B = eng.tr, eng.B
            self.cap = None if tr.audit_cap is None else int(tr.audit_cap)
            self.idx_scatter = e(n, dtype=i32)
            self.valid, self.dist_scale, self.cos = e(n), e(n), e(n)
            self.u_dev = e(B)
            self.perm_dev = e(max((B - self.cap) * self.cap, 1), dtype=i32) if (self.cap is not None and self.cap < B) else None
            self.audit_ema = e(cfg.recipe_count)       # recipe_audit_ema (audit.py:62-77), starts at zero
            self.recent = e(1)                         # recent_residual (audit.py:213-218)
        # backward scratch
        self.dn_f32, self.dh0_acc, self.dcur, self.dalt = e(Ma, d), e(Ma, d), e(Ma, d), e(Ma, d)
        self.d16b = e(Ma, d, dtype=bf)
        self.dz16 = e(Ma, f, dtype=bf)
        # inputs of the weight-gradient launches are kept per pass: those launches run on their own stream and may
        # trail the data-gradient chain, which therefore must not reuse what they still have to read
        self.d16_mlp, self.d16_attn = per_pass("d16_mlp", d), per_pass("d16_attn", d)
        self.dug16, self.dqkv16 = per_pass("dug16", 2 * f), per_pass("dqkv16", 3 * d)
        PR = 128
        self.partials = [[(e(PR, d), e(PR, d), e(PR, d)) for _ in range(2)] for _ in range(T)]
        self.coda_tmps = [_Temps(Ma, cfg, dev) for _ in range(cfg.n_coda)]
        self.dx16_alt = e(Ma, d, dtype=bf)
        self.P = 64
        self.part_alpha, self.part_attn, self.part_mlp = e(T * self.P), e(T * self.P), e(T * self.P)
        # The replay runs on its own stream beside the hot pass, so the gradients it contributes to parameters the
        # hot pass also touches (final norm, coda, tied embedding) are written to a private mirror of those slices of
        # the flat gradient buffer and added after the join; likewise it owns a split-K workspace.
        names = ["final_norm.weight"] + [n for n in eng.grads if n.startswith("coda.")]
        lo = min(eng._grad_offsets[nm] for nm in names)
        hi = max(eng._grad_offsets[nm] + -(-eng.params[nm].numel() // 64) * 64 for nm in names)
        self.shared_range = (lo, hi)
        self.shared_flat = e(hi - lo)
        self.g_shared = {nm: self.shared_flat[eng._grad_offsets[nm] - lo: eng._grad_offsets[nm] - lo + eng.params[nm].numel()]
                         .view(eng.params[nm].shape) for nm in names}
        self.g_embed = e(*eng.params["embed.weight"].shape)
        self.g_shared["embed.weight"] = self.g_embed
        # The replay also carries the gradient of ITS h0 rows back through the prelude and the embedding on its own
        # stream (few-row launches over copies of the hot pass's saved activations), so the hot backward never waits
        # for the replay before its own prelude backward; the two shares meet just before the optimiser.
        # (gather_rows moves 16-byte units: the per-sample rows of rstd / lse need S % 4 == 0.)
        self.own_prelude = (not direct_grads) and len(eng.prelude) > 0 and S % 4 == 0
        if self.own_prelude:
            pnames = [nm for nm in eng.grads if nm.startswith("prelude.")]
            plo = min(eng._grad_offsets[nm] for nm in pnames)
            phi = max(eng._grad_offsets[nm] + -(-eng.params[nm].numel() // 64) * 64 for nm in pnames)
            self.prelude_range = (plo, phi)
            self.prelude_flat = e(phi - plo)
            for nm in pnames:
                o0 = eng._grad_offsets[nm] - plo
                self.g_shared[nm] = self.prelude_flat[o0:o0 + eng.params[nm].numel()].view(eng.params[nm].shape)
            self.prelude_a = [_Block(f"prelude.{i}@audit", Ma, cfg, n, S, dev) for i in range(len(eng.prelude))]
            self.prelude_x_in = [e(Ma, d) for _ in eng.prelude]
            self.prelude_tmps = [_Temps(Ma, cfg, dev) for _ in eng.prelude]
            self.tokens_a = e(Ma, dtype=torch.int64)
            self.dpre, self.dpre_u = e(Ma, d), e(Ma, d)
            self.dpre16 = [e(Ma, d, dtype=bf) for _ in range(len(eng.prelude) + 1)]
            self.embed_accum = torch.zeros(V * d, dtype=torch.int64, device=dev)
        if direct_grads:
            self.g_shared = eng.grads
        big = max(eng.ops.pick_splits(mm, nn, Ma) * mm * nn
                  for mm, nn in ((V, d), (2 * f, d), (d, 2 * f), (3 * d, d), (d, 3 * d), (d, d), (f, d), (d, f)))
        if self.fused_wgrad:
            big = max(big, max(eng.ops.pick_splits(mm, nn, T * Ma) * mm * nn for mm, nn in ((f, d), (d, 2 * f), (d, d), (d, 3 * d))))
        self.ws = e(big)
        self.ws_chain = e(16 * Ma * d)          # split-K partials of the chain's own few-row GEMMs

    # ------------------------------------------------------------------ host side, once per step
    def prepare(self, step_seed: int) -> None:
        """Host half of `choose` for a coming step: the seeded permutation and the control-variate weights, written to
        a pinned staging pair.  Three pairs rotate: with up to two steps queued on the device, the pair written here for
        step i+2 is the one step i-1 used, whose copy has completed by the time that step was collected."""
        eng = self.eng
        if self.bernoulli:
            return self._prepare_bernoulli(step_seed)
        if self.scheduled:
            return self._prepare_scheduled(step_seed)
        if self._stage is None:
            pin = eng.device.type == "cuda"
            self._stage = [(torch.empty(self.k, dtype=torch.int32, pin_memory=pin),
                            torch.empty(eng.B, dtype=torch.float32, pin_memory=pin)) for _ in range(3)]
            self._stage_next = 0
        gen = torch.Generator().manual_seed(step_seed)
        chosen = torch.sort(torch.randperm(eng.B, generator=gen)[: self.k]).values
        h_idx, h_rw = self._stage[self._stage_next]
        w0 = 1.0 / (eng.B * eng.S * eng.loss_div)
        h_idx.copy_(chosen)
        h_rw.fill_(w0)
        if self.grad and self.clip is None:
            h_rw[chosen] = w0 * (1.0 - 1.0 / self.p_inc)                 # d corrected / d hot on audited samples
        # (with a residual clip the factor depends on the losses: `clip_hot` applies it on the device;
        #  without gradient correction the audited samples keep their plain weight)
        self._prepared = (step_seed, chosen, h_idx, h_rw)
        self._stage_next = (self._stage_next + 1) % 3

    def _prepare_bernoulli(self, step_seed: int) -> None:
        """Host half of the Bernoulli sampler: the uniforms `torch.bernoulli(p, generator)` compares p with (the same
        CPU generator stream as `torch.rand`), and -- with a cap -- for every possible candidate count above the cap the
        first `cap` entries of the permutation the reference would draw next from that generator (audit.py:117-131)."""
        eng, B = self.eng, self.eng.B
        if self._stage is None:
            pin = eng.device.type == "cuda"
            rows = max((B - self.cap) * self.cap, 1) if (self.cap is not None and self.cap < B) else 1
            self._stage = [(torch.empty(B, dtype=torch.float32, pin_memory=pin),
                            torch.zeros(rows, dtype=torch.int32, pin_memory=pin)) for _ in range(3)]
            self._stage_next = 0
        gen = torch.Generator().manual_seed(step_seed)
        h_u, h_perm = self._stage[self._stage_next]
        h_u.copy_(torch.rand(B, generator=gen))
        if self.perm_dev is not None:
            state = gen.get_state()
            table = h_perm.view(B - self.cap, self.cap)
            for count in range(self.cap + 1, B + 1):
                g2 = torch.Generator()
                g2.set_state(state)
                table[count - self.cap - 1].copy_(torch.randperm(count, generator=g2)[: self.cap])
        self._prepared = (step_seed, None, h_u, h_perm)
        self._stage_next = (self._stage_next + 1) % 3

    def _prepare_scheduled(self, step_seed: int) -> None:
        """Count schedule: the subset is the fixed-count sampler's (audit.py:99-116) for the current count; the host
        writes what `rte_audit_sample_bernoulli` writes on the device for a drawn subset -- slot lists padded to the
        capacity, per-slot 1/p, the rescaling of the distillation means, both sets of loss weights, the statistics."""
        eng, n, B = self.eng, self.n, self.eng.B
        k = min(self.count, B)
        if k > n:
            raise RuntimeError(f"the audit schedule asks for {k} audited samples, the replay was built for {n} "
                               "(TrainEngine(audit_capacity=...))")
        if self._stage is None:
            pin = eng.device.type == "cuda"
            self._stage = [(torch.zeros(2 * n + 4, dtype=torch.float32, pin_memory=pin),
                            torch.zeros(4 * n, dtype=torch.float32, pin_memory=pin),
                            torch.zeros(B, dtype=torch.float32, pin_memory=pin),
                            torch.zeros(1, dtype=torch.int32, pin_memory=pin)) for _ in range(3)]
            self._stage_next = 0
        h_blk, h_pack, h_rw, h_none = self._stage[self._stage_next]
        gen = torch.Generator().manual_seed(step_seed)
        chosen = torch.sort(torch.randperm(B, generator=gen)[:k]).values.to(torch.int32)
        p = float(k) / float(B)
        ip = 1.0 / max(p, 1e-12)
        w0 = 1.0 / (B * eng.S * eng.loss_div)
        idx, inv_p, stats = h_blk[0:n].view(torch.int32), h_blk[n:2 * n], h_blk[2 * n:]
        idx_scatter, valid, dist_scale, rw_a = h_pack[0:n].view(torch.int32), h_pack[n:2 * n], h_pack[2 * n:3 * n], h_pack[3 * n:]
        idx.zero_(); idx_scatter.fill_(-1)                                                       # noqa: E702
        for t in (inv_p, valid, dist_scale, rw_a):
            t.zero_()
        idx[:k], idx_scatter[:k] = chosen, chosen
        inv_p[:k], valid[:k], rw_a[:k] = ip, 1.0, w0 * ip
        if k:
            dist_scale[:k] = float(n) / float(k)
        stats.copy_(torch.tensor([float(k), float(k), p, p]))
        h_rw.fill_(w0)
        if k and self.grad and self.clip is None:
            h_rw[chosen.long()] = w0 * (1.0 - ip)              # d corrected / d hot on audited samples
        h_none.fill_(0 if k else 1)
        self.p_inc = max(p, 1e-12)
        self._prepared = (step_seed, chosen.long(), h_blk, h_pack, h_rw, h_none)
        self._stage_next = (self._stage_next + 1) % 3

    def update_schedule(self, metrics: dict) -> int:
        """audit.py:137-185, called with the metrics of a step that audited somebody: sets the next step's count."""
        self.count = next_fixed_count(self.eng.tr, self.count, metrics, self.eng.B, self.schedule_state)
        return self.count

    def sample(self) -> None:
        """Device half of the Bernoulli sampler, after the router: audit probabilities, the subset, its per-sample
        inclusion probabilities, the loss weights of the hot rows and of the replay, the coverage average."""
        eng = self.eng
        tr, cfg = eng.tr, eng.cfg
        w0 = 1.0 / (eng.B * eng.S * eng.loss_div)
        prm = dict(p_min=tr.audit_p_min, p_max=tr.audit_p_max, alpha=tr.audit_alpha, beta=tr.audit_beta, gamma=tr.audit_gamma,
                   coverage_min=tr.coverage_min, coverage_beta=tr.coverage_beta,
                   inv_r_plus_k=1.0 / (cfg.recipe_count + len(cfg.depth_choices)), w0=w0, B=eng.B, R=cfg.recipe_count,
                   cap=-1 if (self.cap is None or self.cap >= eng.B) else self.cap, n_cap=self.n,      # (a cap of B or more never engages)
                   weight_mode=1 if (self.grad and self.clip is None) else 0)
        eng.ops.audit_sample_bernoulli(eng.route["router_entropy"], eng.route["recipe_id"], self.u_dev, self.perm_dev,
                                       self.audit_ema, self.recent, prm, self.idx, self.idx_scatter, self.valid, self.inv_p,
                                       self.dist_scale, eng.row_weight, self.row_weight_a, self.stats,
                                       none_audited=eng._none_audited)
        if eng._core_absent is not None:
            eng._core_absent.mul_(eng._none_audited)      # stays 1 only while nobody has been audited in this cycle

    def choose(self, step_seed: int) -> None:
        """Fixed-count sampler: first k entries of a seeded CPU permutation (audit.py:99-116); writes the subset
        indices and the control-variate weights of the hot rows."""
        eng = self.eng
        if self._prepared is None or self._prepared[0] != step_seed:
            self.prepare(step_seed)
        if self.bernoulli:
            _, _, h_u, h_perm = self._prepared
            self._prepared = None
            self.u_dev.copy_(h_u, non_blocking=True)
            if self.perm_dev is not None:
                self.perm_dev.copy_(h_perm, non_blocking=True)
            self.last_chosen = None
            return
        if self.scheduled:
            _, chosen, h_blk, h_pack, h_rw, h_none = self._prepared
            self._prepared = None
            self.sampler_block.copy_(h_blk, non_blocking=True)
            self.sched_pack.copy_(h_pack, non_blocking=True)
            eng.row_weight.copy_(h_rw, non_blocking=True)
            if eng._none_audited is not None:
                eng._none_audited.copy_(h_none, non_blocking=True)
            self.last_chosen = chosen
            return
        _, chosen, h_idx, h_rw = self._prepared
        self._prepared = None
        self.idx.copy_(h_idx, non_blocking=True)
        eng.row_weight.copy_(h_rw, non_blocking=True)
        self.last_chosen = chosen

    # ------------------------------------------------------------------ forward
    def forward_replay_head(self, h0: torch.Tensor) -> None:
        """The part of the replay's forward that needs h0 but no routing decision yet: the gathers, the first norm and
        the first pass's QKV product and attention (the recipe's column mask only enters after the attention), so it
        can run beside the router."""
        eng = self.eng
        o, cfg, p, sh = eng.ops, eng.cfg, eng.params, eng.shadow
        n, S, Ma, d = self.n, self.S, self.Ma, cfg.d_model
        o.gather_rows(h0, self.idx, self.h0a, n, S * d * 4)
        if not self.own_prelude:             # (own_prelude: `gather_prelude` copies the targets too, off this chain)
            o.gather_rows(eng.targets, self.idx, self.targets_a, n, S * 8)
        alpha = p["core.alpha_inj"].view(1)
        o.residual_rmsnorm_fwd(self.h[0], self.h0a, alpha, self.ht[0], p["core.norm1.weight"], self.n1[0], self.rstd1[0],
                               S=S, film_gamma=p["core.pass_gamma1"][0], film_beta=p["core.pass_beta1"][0])
        for bk in range(cfg.attn_banks):
            o.gemm(self.n1[0], sh["core.attn.wqkv"][bk], self.qkv[0][bk], M=Ma, N=3 * d, K=d, b_mn=True)
            o.attn_fwd(self.qkv[0][bk], self.y[0][bk], self.lse[0][bk], B=n, S=S, n_heads=cfg.n_heads, head_dim=cfg.head_dim)

    def forward_replay(self, h0: torch.Tensor, head_done: bool = False) -> None:
        """Everything of the replay's forward that needs only h0 and the routing decisions (`head_done`: the caller
        has already issued `forward_replay_head`)."""
        eng = self.eng
        o, cfg, p, sh = eng.ops, eng.cfg, eng.params, eng.shadow
        n, S, T, Ma, d, f, V = self.n, self.S, self.T, self.Ma, cfg.d_model, cfg.d_ff, cfg.vocab_size
        if not head_done:
            self.forward_replay_head(h0)
        o.audit_route(eng.route["recipe_id_by_pass"], eng.route["depth"], self.idx, self.rid, self.active, n, T)
        if self.fixed_rid is not None:               # a fixed per-pass recipe schedule overrides the routed recipes
            self.rid.copy_(self.fixed_rid)
        alpha = p["core.alpha_inj"].view(1)
        # The residual updates ride in front of the norms (one launch each instead of two or three):
        #   ht = h + alpha*h0 -> norm1;   u = ht + s_attn*attn -> norm2;
        #   h' = active ? u + s_mlp*mlp : h, then ht' = h' + alpha*h0 -> next pass's norm1
        film1 = lambda t: dict(film_gamma=p["core.pass_gamma1"][t], film_beta=p["core.pass_beta1"][t])  # noqa: E731
        for t in range(T):
            rid = self.rid[t]
            for bk in range(cfg.attn_banks):
                if t > 0:           # pass 0's attention was issued by forward_replay_head (before the routing was known)
                    o.gemm(self.n1[t], sh["core.attn.wqkv"][bk], self.qkv[t][bk], M=Ma, N=3 * d, K=d, b_mn=True)
                    o.attn_fwd_masked(self.qkv[t][bk], self.y[t][bk], self.ym[t][bk], self.lse[t][bk], rid, self.head_tab[bk],
                                      B=n, S=S, n_heads=cfg.n_heads, head_dim=cfg.head_dim)
                else:
                    o.colmask_mul(self.y[t][bk], rid, self.head_tab[bk], S, self.ym[t][bk], Ma, d)
                o.gemm(self.ym[t][bk], sh["core.attn.wo"][bk], self.attn_acc[t], M=Ma, N=d, K=d, b_mn=True,
                       epilogue=A.EPI_F32, residual=self.attn_acc[t] if bk > 0 else None)
            o.residual_rmsnorm_fwd(self.ht[t], self.attn_acc[t], p["core.pass_attn_scale"][t:t + 1], self.u[t],
                                   p["core.norm2.weight"], self.n2[t], self.rstd2[t], S=S,
                                   film_gamma=p["core.pass_gamma2"][t], film_beta=p["core.pass_beta2"][t])
            for bk in range(cfg.ffn_banks):
                o.gemm(self.n2[t], sh["core.mlp.wug"][bk], self.ug[t][bk], M=Ma, N=2 * f, K=d, b_mn=True)
                o.swiglu_masked_fwd(self.ug[t][bk], rid, self.ffn_tab[bk], S, self.zm[t][bk], Ma, f)
                # (one bank, another pass to come: the split-K partials go straight into the norm launch below, which
                #  sums them in split order and keeps the sum in mlp_acc for the backward pass)
                sp = o.gemm_f32_few_rows(self.zm[t][bk], sh["core.mlp.wd"][bk], self.mlp_acc[t], M=Ma, N=d, K=f, b_mn=True,
                                         ws=self.ws_chain, accumulate=bk > 0,
                                         reduce=not (self.split_feed and cfg.ffn_banks == 1 and t + 1 < T))
            if t + 1 < T:
                split = sp[0] > 1
                o.residual_rmsnorm_fwd(self.u[t], self.ws_chain if split else self.mlp_acc[t],
                                       p["core.pass_mlp_scale"][t:t + 1], self.ht[t + 1],
                                       p["core.norm1.weight"], self.n1[t + 1], self.rstd1[t + 1], S=S,
                                       active=self.active[t], passthrough=self.h[t], add2=self.h0a, scale2=alpha,
                                       x1_out=self.h[t + 1], branch_splits=sp, branch_out=self.mlp_acc[t] if split else None,
                                       **film1(t + 1))
            else:
                o.scaled_residual_fwd(self.u[t], self.mlp_acc[t], p["core.pass_mlp_scale"][t:t + 1], self.active[t],
                                      self.h[t], self.h[t + 1], n, S * d)
        x = self.h[T]
        self._core_fwd_done = None                  # the exact endpoint h[T] exists: the distillation terms can start
        if eng._side_stream is not None:
            self._core_fwd_done = torch.cuda.Event()
            self._core_fwd_done.record(torch.cuda.current_stream(eng.device))
        for blk in self.coda:
            x = eng._block_fwd(blk, x)
        self.x_last = x
        o.rmsnorm_fwd(x, p["final_norm.weight"], self.hidden16, self.rstd_f)
        o.gemm(self.hidden16, sh["embed.weight"], self.logits, M=Ma, N=V, K=d)

    def forward_distill(self, h_phi: torch.Tensor) -> None:
        """Distillation terms between the macro output and the replay's endpoint (the hot side receives the
        gradient, the exact side is a constant: macro.py:413-415).  Issued by the hot pass once the macro operator has
        run.  The terms need the replay's endpoint h[T] but not its coda or logits, and the hot pass needs their
        gradient only when its backward reaches the macro operator (`distill_done`): they run on the replay's
        weight-gradient stream, idle during forward, beside the replay's coda instead of in front of its KL term."""
        eng = self.eng
        o, cfg = eng.ops, eng.cfg
        n, S, T, d = self.n, self.S, self.T, cfg.d_model
        tr, w = eng.tr, 1.0 / eng.loss_div
        ps, main = eng._param_stream, None
        self.distill_done = None
        if ps is not None and self._core_fwd_done is not None:
            main = torch.cuda.current_stream(eng.device)
            ps.wait_stream(main)                        # h_phi
            ps.wait_event(self._core_fwd_done)          # h[T], h0a, idx
            ctx = torch.cuda.stream(ps)
        else:
            eng._side_wait_main()
            ctx = eng._on_side()
        with ctx:
            o.gather_rows(h_phi, self.idx, self.hot_end, n, S * d * 4)
            o.macro_distill(self.hot_end, self.h[T], self.h0a, tr.lambda_delta_dir * w, tr.lambda_delta_rms * w,
                            tr.lambda_endpoint_normed * w, tr.lambda_endpoint_raw * w, self.terms, self.dhot_extra, n, S, d)
            if self.padded:
                # the kernel averaged over all n slots: n / audited on the audited samples' rows, 0 on the others
                o.scale_rows_f32(self.dhot_extra, self.dist_scale, n, S * d)
            if main is not None:
                self.distill_done = torch.cuda.Event()
                self.distill_done.record(ps)

    def forward_kl(self) -> None:
        """KL-distillation term between the saved hot logits of the audited rows and the replay's logits; its gradient
        goes to `self.dkl` (the hot pass adds it to its dlogits with `add_kl_grad` once its own cross-entropy kernel
        has written them, so this launch can run beside that kernel)."""
        eng = self.eng
        o, cfg, tr, w = eng.ops, eng.cfg, eng.tr, 1.0 / eng.loss_div
        n, Ma, V = self.n, self.Ma, cfg.vocab_size
        temp = max(float(tr.distill_temperature), 1e-6)
        if not eng.shortlist:      # the shortlist head keeps no full hot logits, so the KL term is absent (models.py:698-703)
            # (the temperature-1 KL of logit_kl_exact_macro, macro.py:538-543 / metrics.py:119-124, is a by-product of the
            #  same launch: the replay's logits are overwritten by its cross entropy right afterwards)
            o.kl_distill_grad(self.hot_logits, self.logits, temp, tr.lambda_kl * w * temp / n, self.dkl, self.kl_rows, Ma, V,
                              kl1_rows=self.kl1_rows if temp != 1.0 else None)
            if self.padded:
                o.scale_rows_f32(self.dkl, self.dist_scale, n, self.S * V)

    def report(self) -> None:
        """Everything of the replay's forward that the step only REPORTS (or that the next step's sampler reads): the
        alignment sums, the summed KL rows, the temperature-1 KL, the sampler's last residual.  The hot pass waits
        for none of it, so it is issued after the event the hot pass waits on, and -- when the replay goes on with a
        backward pass -- on the replay's weight-gradient stream (idle until that backward's first weight gradient, and
        joined before the optimiser), so that it delays neither the hot pass nor the replay's own chain."""
        import contextlib
        eng = self.eng
        o, cfg, tr = eng.ops, eng.cfg, eng.tr
        n, S, T, Ma, d, V = self.n, self.S, self.T, self.Ma, cfg.d_model, cfg.vocab_size
        ps = eng._param_stream if self.grad else None
        ctx = contextlib.nullcontext()
        if ps is not None:
            ps.wait_stream(torch.cuda.current_stream(eng.device))
            ctx = torch.cuda.stream(ps)
        elif self.distill_done is not None:
            torch.cuda.current_stream(eng.device).wait_event(self.distill_done)     # hot_end is written there
        with ctx:
            o.audit_alignment_sums(self.hot_end, self.h[T], self.h0a, n, S * d, self.align)
            if self.bernoulli:
                o.audit_recent_residual(self.hot_end, self.h[T], self.valid, n, S * d, self.cos, self.recent)
            if eng.shortlist:
                return
            if self.padded:
                o.scale_rows_f32(self.kl_rows, self.valid, n, S)
            o.segment_sum(self.kl_rows, self.kl_sum, 1, Ma)
            if max(float(tr.distill_temperature), 1e-6) != 1.0:
                # the temperature-1 KL's sum over the audited rows rides in the free eighth column of the alignment sums
                if self.padded:
                    o.scale_rows_f32(self.kl1_rows, self.valid, n, S)
                o.segment_sum(self.kl1_rows, self.align.view(-1)[7:8], 1, Ma)

    def add_kl_grad(self) -> None:
        """Hot-pass side of `forward_kl`: dlogits[audited rows] += dkl."""
        eng = self.eng
        if not eng.shortlist:
            eng.ops.add_rows_to_bf16(eng.logits, self.idx_scatter, self.S, self.dkl, self.Ma, eng.cfg.vocab_size)

    def forward_ce(self) -> None:
        """The replay's own cross entropy (its logits become dlogits in place)."""
        eng = self.eng
        o, n, S = eng.ops, self.n, self.S
        if self.own_prelude and eng._param_stream is not None:
            # what `gather_prelude` queued on the weight-gradient stream during forward is read by this backward
            # (its event, not the whole stream: `report` may still be running there)
            if self._prelude_copied is not None:
                torch.cuda.current_stream(eng.device).wait_event(self._prelude_copied)
            else:
                torch.cuda.current_stream(eng.device).wait_stream(eng._param_stream)
        o.ce_fwd_bwd(self.logits, self.targets_a, self.row_weight_a, S, self.loss_tok, self.logits)
        ps = eng._param_stream
        if self.grad and self.clip is None and ps is not None:
            # the per-sample sums are only reported (a residual clip would read them): off the backward's chain
            ps.wait_stream(torch.cuda.current_stream(eng.device))
            with torch.cuda.stream(ps):
                o.segment_sum(self.loss_tok, self.exact_loss, n, S)
        else:
            o.segment_sum(self.loss_tok, self.exact_loss, n, S)

    def clip_exact(self) -> None:
        """Residual clip (audit.py:306-321), replay side: decides per audited sample whether exact - hot lies inside the
        clip and removes the replay's cross-entropy gradient (written with weight 1/p) where it does not."""
        eng = self.eng
        o = eng.ops
        o.audit_clip(eng.loss_per_sample, self.exact_loss, self.idx, self.n, 1.0 / self.p_inc, float(self.clip),
                     self.f_hot, self.f_exact, inv_p_slot=self.inv_p if self.padded else None)
        o.scale_rows_bf16(self.logits, None, self.S, self.f_exact, self.Ma, eng.cfg.vocab_size)

    def clip_hot(self) -> None:
        """Hot side of `clip_exact`: the audited rows of the hot dlogits (written with weight 1) get 1 - 1/p inside the
        clip and keep 1 outside."""
        eng = self.eng
        eng.ops.scale_rows_bf16(eng.logits, self.idx_scatter, self.S, self.f_hot, self.Ma, eng.cfg.vocab_size)

    def save_hot_logits(self) -> None:
        """Copies the audited rows of the hot logits before the cross-entropy kernel overwrites them."""
        V = self.eng.cfg.vocab_size
        self.eng.ops.gather_rows(self.eng.logits, self.idx, self.hot_logits, self.n, self.S * V * 2)

    # ------------------------------------------------------------------ backward
    def backward_head(self) -> torch.Tensor:
        """Logits, final norm and coda of the replay (weight gradients are ADDED to the hot pass's).
        Returns the gradient wrt the last recurrent state h[T]."""
        eng = self.eng
        o, cfg, p, sh, g = eng.ops, eng.cfg, eng.params, eng.shadow, eng.grads
        Ma, d, V = self.Ma, cfg.d_model, cfg.vocab_size
        t = self.tmp
        self._defer_param_grads(True)
        o.gemm(self.logits, sh["embed.weight"], t.dn16, M=Ma, N=d, K=V, b_mn=True)
        gs = self.g_shared
        o.gemm_wgrad(self.logits, self.hidden16, gs["embed.weight"], M=V, N=d, K=Ma, ws=self.ws)
        o.rmsnorm_bwd(self.x_last, p["final_norm.weight"], self.rstd_f, t.dn16, None, t.dxa, t.dx16,
                      gs["final_norm.weight"], t.partial)
        dcur, dalt = t.dxa, t.dxb
        in16, out16 = t.dx16, self.dx16_alt          # distinct: the deferred wd gradient still reads the block's input
        for i, blk in enumerate(reversed(self.coda)):
            eng._block_bwd(blk, dcur, in16, dalt, out16, t.dxc, tmp=self.coda_tmps[i], mark_ready=False, grads=gs, ws=self.ws)
            dcur, dalt = dalt, dcur
            in16, out16 = out16, in16
        self._defer_param_grads(False)
        # the head's weight gradients are queued: `merge_head` may add them to the hot pass's from here on
        self.head_w_done = None
        if eng._param_stream is not None and eng.device.type == "cuda":
            self.head_w_done = torch.cuda.Event()
            self.head_w_done.record(eng._param_stream)
        return dcur

    def _defer_param_grads(self, on: bool) -> None:
        """Routes the replay's weight-gradient launches to the parameter-gradient stream (see CudaOps.param_stream)."""
        eng = self.eng
        if eng._param_stream is not None and hasattr(eng.ops, "param_stream"):
            eng.ops.param_stream = eng._param_stream if on else None

    def backward_core(self, dh_last: torch.Tensor) -> None:
        """Backward through the t_max banked passes (the subset's h0 gradient is folded in by `merge`)."""
        eng = self.eng
        o, cfg, p, sh, g = eng.ops, eng.cfg, eng.params, eng.shadow, eng.grads
        n, S, T, Ma, d, f, P = self.n, self.S, self.T, self.Ma, cfg.d_model, cfg.d_ff, self.P
        alpha = p["core.alpha_inj"].view(1)
        if not self.own_prelude:          # (own_prelude: cleared during forward, off the chain, by `gather_prelude`)
            o.fill_(self.dh0_acc, 0.0)
        # With several banks the per-bank buffers are reused inside a pass, so everything stays on the chain (after
        # the head's deferred launches, which share the split-K workspace, have finished); the single-bank case (the
        # usual one) defers its weight gradients.
        defer = cfg.ffn_banks == 1 and cfg.attn_banks == 1
        fused = self.fused_wgrad            # the four weight-gradient products once, over all passes, after the loop
        if not defer and eng._param_stream is not None:
            torch.cuda.current_stream(eng.device).wait_stream(eng._param_stream)
        self._defer_param_grads(defer)
        dnext, dthis = dh_last, (self.dcur if dh_last is not self.dcur else self.dalt)
        for t in reversed(range(T)):
            rid, first = self.rid[t], t == T - 1
            acc = not first
            d16m, d16a, dug16, dqkv16 = self.d16_mlp[t], self.d16_attn[t], self.dug16[t], self.dqkv16[t]
            (pw2, pg2, pb2), (pw1, pg1, pb1) = self.partials[t]
            du, dht = self.tmp.dxc, self.tmp.dxb if dnext is not self.tmp.dxb else self.tmp.dxa
            if du is dnext:
                du = self.tmp.dxa if dht is not self.tmp.dxa else self.tmp.dxb
            # out = active ? u + s_mlp * mlp : h_in
            o.scaled_residual_bwd(dnext, self.mlp_acc[t], p["core.pass_mlp_scale"][t:t + 1], self.active[t], du,
                                          d16m, None, None, self.part_mlp[t * P:(t + 1) * P], n, S * d)
            for bk in range(cfg.ffn_banks):
                o.gemm(d16m, sh["core.mlp.wd"][bk], self.dz16, M=Ma, N=f, K=d)
                if not fused:
                    o.gemm_wgrad(self.zm[t][bk], d16m, g["core.mlp.wd"][bk], M=f, N=d, K=Ma, accumulate=acc, ws=self.ws)
                o.swiglu_masked_bwd(self.ug[t][bk], self.dz16, rid, self.ffn_tab[bk], S, dug16, Ma, f)
                sp2 = o.gemm_f32_few_rows(dug16, sh["core.mlp.wug"][bk], self.dn_f32, M=Ma, N=d, K=2 * f, b_mn=False,
                                          ws=self.ws_chain, accumulate=bk > 0, reduce=cfg.ffn_banks > 1 or not self.split_feed)
                if not fused:
                    o.gemm_wgrad(self.n2[t], dug16, g["core.mlp.wug"][bk], M=d, N=2 * f, K=Ma, accumulate=acc, ws=self.ws)
            # (one bank: the norm backward sums the product's split-K partials itself, in split order)
            o.rmsnorm_bwd(self.u[t], p["core.norm2.weight"], self.rstd2[t], self.ws_chain if sp2[0] > 1 else self.dn_f32,
                          du, du, None, g["core.norm2.weight"], pw2, film_gamma=p["core.pass_gamma2"][t],
                          dgamma_out=g["core.pass_gamma2"][t], dbeta_out=g["core.pass_beta2"][t],
                          partial_g=pg2, partial_b=pb2, accumulate_dw=acc, dy_splits=sp2)
            # u = ht + s_attn * attn
            o.scaled_residual_bwd(du, self.attn_acc[t], p["core.pass_attn_scale"][t:t + 1], None, dht, d16a, None, None,
                                  self.part_attn[t * P:(t + 1) * P], n, S * d)
            for bk in range(cfg.attn_banks):
                o.gemm(d16a, sh["core.attn.wo"][bk], self.d16b, M=Ma, N=d, K=d)
                if not fused:
                    o.gemm_wgrad(self.ym[t][bk], d16a, g["core.attn.wo"][bk], M=d, N=d, K=Ma, accumulate=acc, ws=self.ws)
                o.attn_bwd_masked(self.qkv[t][bk], self.y[t][bk], self.d16b, self.lse[t][bk], dqkv16, rid, self.head_tab[bk],
                                  B=n, S=S, n_heads=cfg.n_heads, head_dim=cfg.head_dim)
                sp1 = o.gemm_f32_few_rows(dqkv16, sh["core.attn.wqkv"][bk], self.dn_f32, M=Ma, N=d, K=3 * d, b_mn=False,
                                          ws=self.ws_chain, accumulate=bk > 0, reduce=cfg.attn_banks > 1 or not self.split_feed)
                if not fused:
                    o.gemm_wgrad(self.n1[t], dqkv16, g["core.attn.wqkv"][bk], M=d, N=3 * d, K=Ma, accumulate=acc, ws=self.ws)
            o.rmsnorm_bwd(self.ht[t], p["core.norm1.weight"], self.rstd1[t], self.ws_chain if sp1[0] > 1 else self.dn_f32,
                          dht, dht, None, g["core.norm1.weight"], pw1, film_gamma=p["core.pass_gamma1"][t],
                          dgamma_out=g["core.pass_gamma1"][t], dbeta_out=g["core.pass_beta1"][t],
                          partial_g=pg1, partial_b=pb1, accumulate_dw=acc, dy_splits=sp1)
            # ht = h_in + alpha * h0
            # (samples that were frozen in this pass hand their gradient `dnext` straight through: same launch)
            o.scaled_residual_bwd(dht, self.h0a, alpha, None, dthis, None, self.dh0_acc, None,
                                  self.part_alpha[t * P:(t + 1) * P], n, S * d, frozen_active=self.active[t],
                                  frozen_src=dnext)
            dnext, dthis = dthis, (self.dalt if dthis is self.dcur else self.dcur)
        self.dh_first = dnext
        if fused:
            st, K = self._stacked, T * Ma
            o.gemm_wgrad(st["zm"], st["d16_mlp"], g["core.mlp.wd"][0], M=f, N=d, K=K, ws=self.ws)
            o.gemm_wgrad(st["n2"], st["dug16"], g["core.mlp.wug"][0], M=d, N=2 * f, K=K, ws=self.ws)
            o.gemm_wgrad(st["ym"], st["d16_attn"], g["core.attn.wo"][0], M=d, N=d, K=K, ws=self.ws)
            o.gemm_wgrad(st["n1"], st["dqkv16"], g["core.attn.wqkv"][0], M=d, N=3 * d, K=K, ws=self.ws)
        self._defer_param_grads(False)
        if not self.own_prelude:                      # (own_prelude: `finish_core` does this off the chain)
            self._scalar_grads()
            if eng._param_stream is not None:         # the replay's stream ends only when its weight gradients have
                torch.cuda.current_stream(eng.device).wait_stream(eng._param_stream)

    # ------------------------------------------------------------------ the grouped block (recursive_deferred_grouped_exact)
    def forward_deferred(self, h0: torch.Tensor) -> None:
        """`BankedRecursiveCore.deferred_grouped_block` (layers.py:872-912) over the whole batch, then coda and logits:
        ONE block whose attention half and MLP half each sum the branches of the `deferred_depth` scheduled recipes;
        every branch reads the same normed input under its own pass's FiLM and enters with its own pass's scale.
        Pass t's buffers hold branch t (one bank each; `fixed_rid` holds the schedule)."""
        eng = self.eng
        o, cfg, p, sh = eng.ops, eng.cfg, eng.params, eng.shadow
        n, S, T, Ma, d, f, V, D = self.n, self.S, self.T, self.Ma, cfg.d_model, cfg.d_ff, cfg.vocab_size, self.deferred_depth
        o.gather_rows(h0, self.idx, self.h0a, n, S * d * 4)
        o.gather_rows(eng.targets, self.idx, self.targets_a, n, S * 8)
        self.rid.copy_(self.fixed_rid)
        alpha = p["core.alpha_inj"].view(1)
        film = lambda k, t: dict(film_gamma=p[f"core.pass_gamma{k}"][t], film_beta=p[f"core.pass_beta{k}"][t])      # noqa: E731
        ht, u, out = self.ht[0], self.u[0], self.h[T]
        # ht = h0 + alpha * h0 (the block starts from h = h0), normed once per branch under that branch's FiLM
        o.residual_rmsnorm_fwd(self.h0a, self.h0a, alpha, ht, p["core.norm1.weight"], self.n1[0], self.rstd1[0], S=S, **film(1, 0))
        for t in range(D):
            if t:
                o.rmsnorm_fwd(ht, p["core.norm1.weight"], self.n1[t], self.rstd1[t], **film(1, t))
            o.gemm(self.n1[t], sh["core.attn.wqkv"][0], self.qkv[t][0], M=Ma, N=3 * d, K=d, b_mn=True)
            o.attn_fwd_masked(self.qkv[t][0], self.y[t][0], self.ym[t][0], self.lse[t][0], self.rid[t], self.head_tab[0],
                              B=n, S=S, n_heads=cfg.n_heads, head_dim=cfg.head_dim)
            o.gemm(self.ym[t][0], sh["core.attn.wo"][0], self.attn_acc[t], M=Ma, N=d, K=d, b_mn=True, epilogue=A.EPI_F32)
            o.scaled_residual_fwd(ht if t == 0 else u, self.attn_acc[t], p["core.pass_attn_scale"][t:t + 1], None, None, u,
                                  n, S * d)                                   # u = ht + sum_t s_attn[t] * attn_t
        for t in range(D):
            o.rmsnorm_fwd(u, p["core.norm2.weight"], self.n2[t], self.rstd2[t], **film(2, t))
            o.gemm(self.n2[t], sh["core.mlp.wug"][0], self.ug[t][0], M=Ma, N=2 * f, K=d, b_mn=True)
            o.swiglu_masked_fwd(self.ug[t][0], self.rid[t], self.ffn_tab[0], S, self.zm[t][0], Ma, f)
            o.gemm_f32_few_rows(self.zm[t][0], sh["core.mlp.wd"][0], self.mlp_acc[t], M=Ma, N=d, K=f, b_mn=True,
                                ws=self.ws_chain)
            o.scaled_residual_fwd(u if t == 0 else out, self.mlp_acc[t], p["core.pass_mlp_scale"][t:t + 1], None, None, out,
                                  n, S * d)                                   # out = u + sum_t s_mlp[t] * mlp_t
        x = out
        for blk in self.coda:
            x = eng._block_fwd(blk, x)
        self.x_last = x
        o.rmsnorm_fwd(x, p["final_norm.weight"], self.hidden16, self.rstd_f)
        o.gemm(self.hidden16, sh["embed.weight"], self.logits, M=Ma, N=V, K=d)

    def backward_deferred(self, dh_last: torch.Tensor) -> None:
        """Backward of `forward_deferred` from the gradient wrt the block's output: every MLP branch sends its share
        through norm2 into d u, every attention branch through norm1 into d ht; leaves `dh_first` (the part of d h0
        through h) and `dh0_acc` (the part through alpha * h0) like `backward_core`."""
        eng = self.eng
        o, cfg, p, sh, g = eng.ops, eng.cfg, eng.params, eng.shadow, eng.grads
        n, S, T, Ma, d, f, P, D = self.n, self.S, self.T, self.Ma, cfg.d_model, cfg.d_ff, self.P, self.deferred_depth
        alpha = p["core.alpha_inj"].view(1)
        fused = self.fused_wgrad
        self._defer_param_grads(True)
        du, dht = [b for b in (self.dcur, self.dalt, self.tmp.dxa, self.tmp.dxb) if b is not dh_last][:2]
        for t in range(D):
            d16m, dug16, acc = self.d16_mlp[t], self.dug16[t], t > 0
            (pw2, pg2, pb2), _ = self.partials[t]
            o.scaled_residual_bwd(dh_last, self.mlp_acc[t], p["core.pass_mlp_scale"][t:t + 1], None, None, d16m, None, None,
                                  self.part_mlp[t * P:(t + 1) * P], n, S * d)
            o.gemm(d16m, sh["core.mlp.wd"][0], self.dz16, M=Ma, N=f, K=d)
            if not fused:
                o.gemm_wgrad(self.zm[t][0], d16m, g["core.mlp.wd"][0], M=f, N=d, K=Ma, accumulate=acc, ws=self.ws)
            o.swiglu_masked_bwd(self.ug[t][0], self.dz16, self.rid[t], self.ffn_tab[0], S, dug16, Ma, f)
            o.gemm_f32_few_rows(dug16, sh["core.mlp.wug"][0], self.dn_f32, M=Ma, N=d, K=2 * f, b_mn=False, ws=self.ws_chain)
            if not fused:
                o.gemm_wgrad(self.n2[t], dug16, g["core.mlp.wug"][0], M=d, N=2 * f, K=Ma, accumulate=acc, ws=self.ws)
            # d u = d out + sum_t norm2-backward of branch t (the running sum rides in as the residual gradient)
            o.rmsnorm_bwd(self.u[0], p["core.norm2.weight"], self.rstd2[t], self.dn_f32, dh_last if t == 0 else du, du, None,
                          g["core.norm2.weight"], pw2, film_gamma=p["core.pass_gamma2"][t],
                          dgamma_out=g["core.pass_gamma2"][t], dbeta_out=g["core.pass_beta2"][t],
                          partial_g=pg2, partial_b=pb2, accumulate_dw=acc)
        for t in range(D):
            d16a, dqkv16, acc = self.d16_attn[t], self.dqkv16[t], t > 0
            _, (pw1, pg1, pb1) = self.partials[t]
            o.scaled_residual_bwd(du, self.attn_acc[t], p["core.pass_attn_scale"][t:t + 1], None, None, d16a, None, None,
                                  self.part_attn[t * P:(t + 1) * P], n, S * d)
            o.gemm(d16a, sh["core.attn.wo"][0], self.d16b, M=Ma, N=d, K=d)
            if not fused:
                o.gemm_wgrad(self.ym[t][0], d16a, g["core.attn.wo"][0], M=d, N=d, K=Ma, accumulate=acc, ws=self.ws)
            o.attn_bwd_masked(self.qkv[t][0], self.y[t][0], self.d16b, self.lse[t][0], dqkv16, self.rid[t], self.head_tab[0],
                              B=n, S=S, n_heads=cfg.n_heads, head_dim=cfg.head_dim)
            o.gemm_f32_few_rows(dqkv16, sh["core.attn.wqkv"][0], self.dn_f32, M=Ma, N=d, K=3 * d, b_mn=False, ws=self.ws_chain)
            if not fused:
                o.gemm_wgrad(self.n1[t], dqkv16, g["core.attn.wqkv"][0], M=d, N=3 * d, K=Ma, accumulate=acc, ws=self.ws)
            o.rmsnorm_bwd(self.ht[0], p["core.norm1.weight"], self.rstd1[t], self.dn_f32, du if t == 0 else dht, dht, None,
                          g["core.norm1.weight"], pw1, film_gamma=p["core.pass_gamma1"][t],
                          dgamma_out=g["core.pass_gamma1"][t], dbeta_out=g["core.pass_beta1"][t],
                          partial_g=pg1, partial_b=pb1, accumulate_dw=acc)
        # ht = h + alpha * h0 with h = h0: d h (-> dh_first) and alpha * d ht (-> dh0_acc), d alpha from the partial sums
        o.fill_(self.dh0_acc, 0.0)
        o.scaled_residual_bwd(dht, self.h0a, alpha, None, du, None, self.dh0_acc, None, self.part_alpha[0:P], n, S * d)
        self.dh_first = du
        if fused:
            st, K = self._stacked, D * Ma
            o.gemm_wgrad(st["zm"], st["d16_mlp"], g["core.mlp.wd"][0], M=f, N=d, K=K, ws=self.ws)
            o.gemm_wgrad(st["n2"], st["dug16"], g["core.mlp.wug"][0], M=d, N=2 * f, K=K, ws=self.ws)
            o.gemm_wgrad(st["ym"], st["d16_attn"], g["core.attn.wo"][0], M=d, N=d, K=K, ws=self.ws)
            o.gemm_wgrad(st["n1"], st["dqkv16"], g["core.attn.wqkv"][0], M=d, N=3 * d, K=K, ws=self.ws)
        self._defer_param_grads(False)
        self._scalar_grads()
        if eng._param_stream is not None:
            torch.cuda.current_stream(eng.device).wait_stream(eng._param_stream)

    def _scalar_grads(self) -> None:
        """Scalar parameters of the core: per-CTA partial sums -> gradients, in fixed order (slots of part_* beyond the
        CTAs actually launched stay at their initial zero)."""
        eng = self.eng
        o, g, T, P = eng.ops, eng.grads, self.T, self.P
        o.segment_sum(self.part_mlp, g["core.pass_mlp_scale"], T, P)
        o.segment_sum(self.part_attn, g["core.pass_attn_scale"], T, P)
        o.segment_sum(self.part_alpha, g["core.alpha_inj"].view(1), 1, T * P)

    def merge_head(self, hot_w_done):
        """Adds the replay's share of the final-norm / coda gradients to the hot pass's as soon as both exist -- the
        replay's head backward is the first thing its backward does, the hot pass's coda backward the first thing of
        its own -- on a stream of its own, so that these gradients are final (and their bucket can leave) while the
        replay is still inside the core.  Returns the event that marks them final (None: single-stream order)."""
        eng = self.eng
        ms = getattr(eng, "_merge_stream", None)
        if ms is None or self.head_w_done is None:
            return None
        ms.wait_event(self.head_w_done)
        if hot_w_done is not None:
            ms.wait_event(hot_w_done)
        with torch.cuda.stream(ms):
            self.merge_shared()
            ev = torch.cuda.Event()
            ev.record(ms)
        return ev

    def finish_core(self, head_done, hot_w_done=None):
        """What completes the core gradients once the data-gradient chain has left the core: the scalar-parameter sums
        (and, without a merge stream, the add of the replay's share into the hot pass's coda gradients).  Neither feeds
        the chain, so both go to the replay's weight-gradient stream (behind its weight-gradient GEMMs) and the chain
        carries on with the prelude at once.  Returns the event that marks those gradients final."""
        eng = self.eng
        ps = eng._param_stream
        if ps is None:
            self._scalar_grads()
            self.merge_shared()
            return eng._side_event()
        ps.wait_stream(torch.cuda.current_stream(eng.device))
        with torch.cuda.stream(ps):
            self._scalar_grads()
            if head_done is None:
                if hot_w_done is not None:
                    ps.wait_event(hot_w_done)
                self.merge_shared()
            else:
                ps.wait_event(head_done)        # whoever waits for the core's gradients has the head's as well
            ev = torch.cuda.Event()
            ev.record(ps)
        return ev

    def gather_prelude(self) -> None:
        """Copies of what the hot pass's prelude saved for the audited samples (inputs of `backward_prelude`)."""
        eng = self.eng
        o, cfg, n, S = eng.ops, eng.cfg, self.n, self.S
        d, f, H = cfg.d_model, cfg.d_ff, cfg.n_heads
        o.fill_(self.dh0_acc, 0.0)          # accumulator of the core backward (`forward_ce` orders the chain behind this)
        o.gather_rows(eng.tokens, self.idx, self.tokens_a, n, S * 8)
        o.gather_rows(eng.targets, self.idx, self.targets_a, n, S * 8)      # read by `forward_ce`
        for hot, mine, x_in in zip(eng.prelude, self.prelude_a, self.prelude_x_in):
            o.gather_rows(hot.x_in, self.idx, x_in, n, S * d * 4)
            mine.x_in = x_in
            for name, row_bytes in (("n1", S * d * 2), ("n2", S * d * 2), ("y", S * d * 2), ("qkv", S * 3 * d * 2),
                                    ("ug", S * 2 * f * 2), ("z", S * f * 2), ("u", S * d * 4), ("rstd1", S * 4),
                                    ("rstd2", S * 4), ("lse", H * S * 4)):
                o.gather_rows(getattr(hot, name), self.idx, getattr(mine, name), n, row_bytes)
        self._prelude_copied = None
        if eng.device.type == "cuda":
            self._prelude_copied = torch.cuda.Event()
            self._prelude_copied.record(torch.cuda.current_stream(eng.device))

    def merge_shared(self) -> None:
        """Adds the replay's share of the final-norm / coda gradients to the hot pass's (call once both are complete)."""
        eng = self.eng
        lo, hi = self.shared_range
        eng.ops.add_(eng.grad_flat[lo:hi], self.shared_flat)

    def backward_prelude(self) -> None:
        """d h0 of the audited rows (through the alpha*h0 injections and through h[0]) back through the prelude blocks
        and the embedding, into the replay's private mirrors of those gradients."""
        eng = self.eng
        o, n, S, d = eng.ops, self.n, self.S, eng.cfg.d_model
        gs = self.g_shared
        o.add_(self.dh0_acc, self.dh_first)
        o.cast_bf16(self.dh0_acc, self.dpre16[0])
        dcur, dalt = self.dh0_acc, self.dpre
        self._defer_param_grads(True)
        for j, blk in enumerate(reversed(self.prelude_a)):
            eng._block_bwd(blk, dcur, self.dpre16[j], dalt, self.dpre16[j + 1], self.dpre_u, tmp=self.prelude_tmps[j],
                           mark_ready=False, grads=gs, ws=self.ws)
            dcur, dalt = dalt, dcur
        self._defer_param_grads(False)
        o.embed_bwd(self.tokens_a, dcur, self.g_embed, self.embed_accum)
        if eng._param_stream is not None:
            torch.cuda.current_stream(eng.device).wait_stream(eng._param_stream)

    def merge_tail(self, dh0_hot: torch.Tensor | None) -> None:
        """Last join with the hot pass.  With `own_prelude`: adds the replay's prelude and embedding gradients;
        otherwise (`dh0_hot` given, before the hot prelude backward) adds the replay's d h0 rows and the embedding
        share of its logits product."""
        eng = self.eng
        o, n, S, d = eng.ops, self.n, self.S, eng.cfg.d_model
        o.add_(eng.grads["embed.weight"], self.g_embed)
        if self.own_prelude:
            lo, hi = self.prelude_range
            o.add_(eng.grad_flat[lo:hi], self.prelude_flat)
        else:
            o.scatter_add_rows(dh0_hot, self.idx_scatter, self.dh0_acc, n, S * d)
            o.scatter_add_rows(dh0_hot, self.idx_scatter, self.dh_first, n, S * d)

    # ------------------------------------------------------------------ reporting
    def loss_terms(self, hot_per_sample: torch.Tensor, host: dict, chosen: torch.Tensor | None = None) -> dict[str, float]:
        """Host-side assembly of the audited quantities for the reported loss (training.py:1381-1385) from the
        step's fetched results (`terms`, `exact_loss`, `kl_sum` already on the host)."""
        tr, n, Ma, d = self.eng.tr, self.n, self.Ma, self.eng.cfg.d_model
        temp = max(float(tr.distill_temperature), 1e-6)
        if self.padded:
            return self._loss_terms_padded(hot_per_sample, host, temp)
        terms = host["terms"]
        exact = host["exact_loss"].clone()
        hot = hot_per_sample[self.last_chosen if chosen is None else chosen]
        aux = dict(delta_dir=tr.lambda_delta_dir * float(terms[:, 0].mean()),
                   delta_rms=tr.lambda_delta_rms * float(terms[:, 1].mean()),
                   endpoint_normed=tr.lambda_endpoint_normed * float(terms[:, 2].sum()) / (Ma * d),
                   endpoint_raw=tr.lambda_endpoint_raw * float(terms[:, 3].sum()) / (Ma * d),
                   kl=tr.lambda_kl * float(host["kl_sum"]) / n * temp * temp)
        residual = exact - hot
        res = self.residual_metrics(residual)
        if self.clip_reported is not None:
            residual = residual.clamp(-float(self.clip_reported), float(self.clip_reported))
        res["clipped_loss_residual"] = float(residual.mean())
        # the control variate is part of the loss only under gradient correction; its value is reported either way
        corr = float((residual / self.p_inc).sum())
        align = self.alignment_metrics(host["align"], float(hot.mean()) / self.S, float(exact.mean()) / self.S,
                                       kl1=self._kl1_total(host, temp))
        return dict(correction=corr if self.grad else 0.0, correction_metric=corr, exact=exact, aux=aux, alignment=align,
                    residual=res)

    @staticmethod
    def residual_metrics(residual: torch.Tensor) -> dict[str, float]:
        """audit.py:306-310,363: mean / std / variance (population) of exact - hot over the audited samples, before
        any clip."""
        r = residual.double()
        var = float(r.var(unbiased=False)) if r.numel() else 0.0
        return dict(audit_residual_mean=float(r.mean()), audit_residual_std=var ** 0.5, audit_residual_var=var,
                    loss_residual=float(r.mean()))

    def _kl1_total(self, host: dict, temp: float) -> float | None:
        """Sum over the audited rows of KL(exact || hot) at temperature 1 (None with the shortlist head, which keeps no
        full hot logits): the eighth column of the first alignment row, or the distillation's own sum when that already
        runs at temperature 1."""
        if self.eng.shortlist:
            return None
        return float(host["kl_sum"]) if temp == 1.0 else float(host["align"][0, 7])

    def alignment_metrics(self, sums: torch.Tensor, hot_nll: float | None = None, exact_nll: float | None = None,
                          kl1: float | None = None) -> dict:
        """macro_alignment_metrics and compute_residual_metrics (macro.py:499-546, audit.py:207-243) from the
        per-sample sums of `rte_audit_alignment_sums` (`sums`: the audited samples' rows only) and the summed
        temperature-1 KL of the audited rows' logits (`kl1`)."""
        L = float(self.S * self.eng.cfg.d_model)
        s = sums.double()
        ab, aa, bb, dd, pp, ee, pe = (s[:, k] for k in range(7))
        eps = 1e-8
        cos = (ab / (aa.sqrt().clamp_min(eps) * bb.sqrt().clamp_min(eps))).mean()
        dcos = (pe / (pp.sqrt().clamp_min(eps) * ee.sqrt().clamp_min(eps))).mean()
        macro_norm, exact_norm = (aa / L).sqrt().mean(), (bb / L).sqrt().mean()
        pred_rms, exact_rms = (pp / L).sqrt().mean(), (ee / L).sqrt().mean()
        out = dict(hidden_cosine_exact_macro=float(cos), hidden_mse_exact_macro=float(dd.sum() / (L * s.shape[0])),
                   macro_norm=float(macro_norm), exact_norm=float(exact_norm),
                   macro_exact_norm_ratio=float(macro_norm / exact_norm.clamp_min(1e-8)),
                   delta_cosine_exact_macro=float(dcos), delta_rms_exact=float(exact_rms), delta_rms_pred=float(pred_rms),
                   delta_rms_ratio=float(pred_rms / exact_rms.clamp_min(1e-8)))
        out.update(hidden_cosine=out["hidden_cosine_exact_macro"], hidden_residual_l2=out["hidden_mse_exact_macro"] ** 0.5)
        if kl1 is not None:
            out["logit_kl_exact_macro"] = out["logit_kl"] = kl1 / (s.shape[0] * self.S)
        if hot_nll is not None and exact_nll is not None:
            out["hot_exact_nll_gap"] = hot_nll - exact_nll
        return out

    def _loss_terms_padded(self, hot_per_sample: torch.Tensor, host: dict, temp: float) -> dict:
        """`loss_terms` for the Bernoulli sampler and the count schedule: the audited samples, their count and inclusion
        probabilities come back with the step's results; every mean runs over the audited samples (none: all terms 0)."""
        tr, S, d = self.eng.tr, self.S, self.eng.cfg.d_model
        stats = host["audit_stats"]
        a = min(int(round(float(stats[1]))), self.n)
        chosen = host["audit_idx"][:a].long()
        out = dict(chosen=chosen, candidates=int(round(float(stats[0]))), audited=a, p_requested=float(stats[2]),
                   p_inclusion=float(stats[3]))
        zero = dict(delta_dir=0.0, delta_rms=0.0, endpoint_normed=0.0, endpoint_raw=0.0, kl=0.0)
        if a == 0:
            return dict(correction=0.0, correction_metric=0.0, exact=host["exact_loss"][:0].clone(), aux=zero, **out)
        terms, exact, inv_p = host["terms"][:a], host["exact_loss"][:a].clone(), host["audit_inv_p"][:a]
        aux = dict(delta_dir=tr.lambda_delta_dir * float(terms[:, 0].mean()),
                   delta_rms=tr.lambda_delta_rms * float(terms[:, 1].mean()),
                   endpoint_normed=tr.lambda_endpoint_normed * float(terms[:, 2].sum()) / (a * S * d),
                   endpoint_raw=tr.lambda_endpoint_raw * float(terms[:, 3].sum()) / (a * S * d),
                   kl=tr.lambda_kl * float(host["kl_sum"]) / a * temp * temp)
        residual = exact - hot_per_sample[chosen]
        res = self.residual_metrics(residual)
        if self.clip_reported is not None:
            residual = residual.clamp(-float(self.clip_reported), float(self.clip_reported))
        res["clipped_loss_residual"] = float(residual.mean())
        corr = float((residual * inv_p).sum())
        align = self.alignment_metrics(host["align"][:a], float(hot_per_sample[chosen].mean()) / S, float(exact.mean()) / S,
                                       kl1=self._kl1_total(host, temp))
        return dict(correction=corr if self.grad else 0.0, correction_metric=corr, exact=exact, aux=aux, alignment=align,
                    residual=res, **out)
