"""CPU oracle for the ``recursive_macro`` / ``dense_exact`` training step.

TEST INFRASTRUCTURE ONLY.  This file restates, in plain single-process PyTorch
(CPU, fp32, autograd), the algorithm of the reference "Recursive Training
Engine" for the one path this repository accelerates.  Nothing in the product
package imports it; only the test-suite, the smoke entry and the benchmark's
CPU-baseline leg do, and there only as the checker / the timed baseline.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference
package in the build container, runs it on seeded inputs and stores its
outputs, losses, gradients and a 20-step loss curve; ``tests/test_oracle_golden.py``
checks this restatement against those fixtures.

Every function cites the reference file:line it follows (paths relative to the
reference project's ``src/recursive_training_engine``).

Parameters travel as a flat ``dict[str, Tensor]`` using the reference's own
``state_dict`` names (``embed.weight``, ``prelude.0.attn.wqkv.weight``,
``core.attn.wqkv`` ...), so a checkpoint of either side loads into the other.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn.functional as F

# --------------------------------------------------------------------------
# configuration (field names = reference config.py:11-81 / 85-336 subset)
# --------------------------------------------------------------------------


@dataclass
class ModelCfg:
    vocab_size: int = 2048
    d_model: int = 128
    n_heads: int = 4
    d_ff: int = 512
    n_dense_layers: int = 4
    n_prelude: int = 1
    n_coda: int = 1
    t_max: int = 4
    depth_choices: tuple = (1, 2, 4)
    attn_banks: int = 1
    ffn_banks: int = 1
    head_groups: int = 4
    ffn_groups: int = 8
    active_head_groups: int = 2
    active_ffn_groups: int = 2
    recipe_count: int = 5
    macro_rank: int = 32
    macro_update_scale: float = 0.05
    # variants of the macro operator (macro.py:42-124): only their parameter inventory is restated -- modes that
    # evaluate the operator are restated for the plain bounded-residual form alone
    macro_type: str = "bounded_residual"
    macro_hidden_mult: int = 1
    macro_use_gated_update: bool = False
    macro_update_scale_init: float = 1.0
    macro_include_delta_to_h0: bool = False
    macro_use_delta_to_h0: bool = False
    macro_use_depth_embedding: bool = False
    macro_use_recipe_embedding: bool = False
    router_hidden: int | None = None
    topology: str = "recursive"
    shortlist_clusters: int = 64       # OutputConfig.num_clusters (sizes shortlist_head.cluster_router)

    @property
    def router_hidden_dim(self) -> int:  # routing.py:50
        return self.router_hidden or max(32, self.d_model)


@dataclass
class OutputCfg:
    """config.py:340-346."""
    mode: str = "full"
    num_clusters: int = 64
    shortlist_top_clusters: int = 2
    shortlist_max_tokens: int = 128
    hard_negatives: int = 32
    random_negatives: int = 32


@dataclass
class TrainCfg:
    mode: str = "recursive_macro"
    lr: float = 1e-3
    weight_decay: float = 0.1
    batch_size: int = 8
    seq_len: int = 64
    seed: int = 0
    fixed_recipe: int | None = None
    fixed_recipe_schedule: tuple | None = None      # recursive_exact: pass t runs recipe schedule[t] for every sample
    fixed_depth: int | None = 4
    audit_fixed_count_per_batch: int | None = None  # None + p=0 -> no audit
    audit_mode: str = "gradient_corrected"
    audit_residual_clip: float | None = None
    audit_sampler: str = "fixed_count"              # or "bernoulli": adaptive probability, optional cap (audit.py:79-132)
    audit_p_min: float = 0.0
    audit_p_max: float = 0.0
    audit_alpha: float = 0.08
    audit_beta: float = 0.08
    audit_gamma: float = 0.08
    audit_cap: int | None = None
    audit_schedule_enabled: bool = False            # the fixed count halves / doubles from step to step (audit.py:137-185)
    audit_schedule_min_count: int | None = None
    audit_schedule_nll_gap_threshold: float = 0.05
    audit_schedule_hidden_cosine_threshold: float = 0.98
    audit_schedule_residual_var_threshold: float = 1.0
    audit_schedule_delta_rms_ratio_min: float = 0.9
    audit_schedule_delta_rms_ratio_max: float = 1.1
    audit_schedule_hidden_mse_threshold: float = 1.0
    audit_schedule_macro_norm_threshold: float | None = None
    audit_schedule_macro_norm_threshold_mult: float = 2.0
    audit_schedule_require_negative_mse_slope: bool = True
    audit_schedule_require_negative_norm_slope: bool = True
    lambda_depth: float = 1e-4
    lambda_load: float = 1e-2
    lambda_cover: float = 1e-2
    lambda_kl: float = 1e-2
    lambda_delta_dir: float = 2.0
    lambda_delta_rms: float = 2.0
    lambda_endpoint_normed: float = 1.0
    lambda_endpoint_raw: float = 0.05
    lambda_cons: float = 0.0                        # (the reference's default is 1e-3; the BASELINE workloads use 0)
    distill_temperature: float = 2.0
    coverage_min: float = 0.01
    coverage_beta: float = 0.98
    disable_router_aux: bool = False
    grad_clip_norm: float | None = None
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8


# --------------------------------------------------------------------------
# recipes (recipes.py:65-107)
# --------------------------------------------------------------------------


@dataclass(frozen=True)
class Recipe:
    recipe_id: int
    attention_banks: tuple
    ffn_banks: tuple
    head_groups: tuple
    ffn_groups: tuple


def build_recipes(cfg: ModelCfg) -> list[Recipe]:
    """recipes.py:65-100: recipe 0 is the dense fallback, the rest rotate
    through head/ffn slots and banks."""
    out = [
        Recipe(0, tuple(range(cfg.attn_banks)), tuple(range(cfg.ffn_banks)),
               tuple(range(cfg.head_groups)), tuple(range(cfg.ffn_groups)))
    ]
    head_slots = max(1, cfg.head_groups // cfg.active_head_groups)
    ffn_slots = max(1, cfg.ffn_groups // cfg.active_ffn_groups)
    for idx in range(cfg.recipe_count - 1):
        head_slot, ffn_slot = idx % head_slots, idx % ffn_slots
        attn_bank = (idx // head_slots) % cfg.attn_banks
        ffn_bank = (idx // ffn_slots) % cfg.ffn_banks
        hs, fs = head_slot * cfg.active_head_groups, ffn_slot * cfg.active_ffn_groups
        out.append(Recipe(
            idx + 1, (attn_bank,), (ffn_bank,),
            tuple((hs + j) % cfg.head_groups for j in range(cfg.active_head_groups)),
            tuple((fs + j) % cfg.ffn_groups for j in range(cfg.active_ffn_groups)),
        ))
    return out


def recipe_head_cols(cfg: ModelCfg, r: Recipe) -> list[int]:
    """layers.py:673-682: columns of the active heads, head-major."""
    hpg, hd = cfg.n_heads // cfg.head_groups, cfg.d_model // cfg.n_heads
    cols: list[int] = []
    for g in r.head_groups:
        for head in range(g * hpg, (g + 1) * hpg):
            cols.extend(range(head * hd, (head + 1) * hd))
    return cols


def recipe_ffn_cols(cfg: ModelCfg, r: Recipe) -> list[int]:
    """layers.py:744-749: hidden units of the active FFN slabs."""
    slab = cfg.d_ff // cfg.ffn_groups
    cols: list[int] = []
    for g in r.ffn_groups:
        cols.extend(range(g * slab, (g + 1) * slab))
    return cols


def active_touch_table(cfg: ModelCfg) -> torch.Tensor:
    """recipes.py:102-107,139-145."""
    d = cfg.d_model
    vals = []
    for r in build_recipes(cfg):
        attn = len(r.attention_banks) * 4 * d * d * len(r.head_groups) / cfg.head_groups
        ffn = len(r.ffn_banks) * 3 * d * cfg.d_ff * len(r.ffn_groups) / cfg.ffn_groups
        vals.append(float(attn + ffn))
    return torch.tensor(vals, dtype=torch.float32)


# --------------------------------------------------------------------------
# parameter inventory and the benchmark's seeded initialisation
# --------------------------------------------------------------------------


def _block_shapes(prefix: str, cfg: ModelCfg) -> list[tuple[str, tuple]]:
    d, f = cfg.d_model, cfg.d_ff
    return [
        (f"{prefix}.norm1.weight", (d,)),
        (f"{prefix}.attn.wqkv.weight", (3 * d, d)),
        (f"{prefix}.attn.wo.weight", (d, d)),
        (f"{prefix}.norm2.weight", (d,)),
        (f"{prefix}.mlp.wug.weight", (2 * f, d)),
        (f"{prefix}.mlp.wd.weight", (d, f)),
    ]


def macro_param_shapes(cfg) -> list[tuple[str, tuple]]:
    """Parameters of ``MacroOperators`` in registration order for every variant the reference builds (macro.py:42-124):
    the bounded-residual operator with its optional hidden layer, gate, delta-to-h0 / depth-embedding inputs and
    trainable update scale, and the v2 delta-radius operator.  Only the plain bounded-residual form is evaluated by this file (`macro_phi`); the others
    are carried by `recursive_exact`, which never calls the operator."""
    r, k, d, m = cfg.recipe_count, len(cfg.depth_choices), cfg.d_model, cfg.macro_rank
    g = lambda name, default: getattr(cfg, name, default)      # noqa: E731
    delta = g("macro_include_delta_to_h0", False)
    depth_emb, hidden = g("macro_use_depth_embedding", False), max(m, m * g("macro_hidden_mult", 1))
    out: list[tuple[str, tuple]] = []
    if g("macro_type", "bounded_residual") == "v2_delta_radius":
        n_in = 3 * d + (d if (delta or g("macro_use_delta_to_h0", False)) else 0) + (d if depth_emb else 0)
        if depth_emb:
            out.append(("macro.depth_embed", (k, d)))
        if g("macro_use_recipe_embedding", False):
            n_in += d
            out.append(("macro.recipe_embed", (r, d)))
        return out + [("macro.v", (r, k, n_in, hidden)), ("macro.v2", (r, k, hidden, m)), ("macro.u", (r, k, m, d)),
                      ("macro.bias", (r, k, d)), ("macro.rho_base_raw", (r, k)), ("macro.rho_head", (r, k, d, 1))]
    n_in = 3 * d + (d if delta else 0) + (d if depth_emb else 0)
    gated = g("macro_use_gated_update", False)
    legacy = (g("macro_hidden_mult", 1) == 1 and not gated and not delta and not depth_emb
              and g("macro_update_scale_init", 1.0) == 1.0)          # then `update_scale` is a buffer, not a parameter
    if depth_emb:
        out.append(("macro.depth_embed", (k, d)))
    out += [("macro.d_gain", (r, k, d)), ("macro.v", (r, k, n_in, hidden))]
    if hidden != m:
        out.append(("macro.v2", (r, k, hidden, m)))
    out.append(("macro.u", (r, k, m, d)))
    if not legacy:
        out.append(("macro.update_scale", (r, k, d)))
    out.append(("macro.bias", (r, k, d)))
    if gated:
        out += [("macro.gate_v", (r, k, n_in, m)), ("macro.gate_u", (r, k, m, d)), ("macro.gate_bias", (r, k, d))]
    return out


def param_shapes(cfg: ModelCfg) -> list[tuple[str, tuple]]:
    """Names/shapes in the reference's ``named_parameters()`` order
    (models.py:125-151; dense: models.py:78-93)."""
    d, f, v = cfg.d_model, cfg.d_ff, cfg.vocab_size
    if cfg.topology == "dense":
        out = [("embed.weight", (v, d))]
        for i in range(cfg.n_dense_layers):
            out += _block_shapes(f"blocks.{i}", cfg)
        return out + [("final_norm.weight", (d,))]
    hid, r, k, t, m = cfg.router_hidden_dim, cfg.recipe_count, len(cfg.depth_choices), cfg.t_max, cfg.macro_rank
    head_slots = max(1, cfg.head_groups // cfg.active_head_groups)
    ffn_slots = max(1, cfg.ffn_groups // cfg.active_ffn_groups)
    out = [("embed.weight", (v, d))]
    for i in range(cfg.n_prelude):
        out += _block_shapes(f"prelude.{i}", cfg)
    out += [("router.pass_recipe_bias", (t, r)), ("router.pass_factor_bias", (t, hid))]
    for name, o in (("recipe_mlp", r),):
        out += [(f"router.{name}.0.weight", (hid, d)), (f"router.{name}.0.bias", (hid,)),
                (f"router.{name}.2.weight", (o, hid)), (f"router.{name}.2.bias", (o,))]
    out += [("router.factor_mlp.0.weight", (hid, d)), ("router.factor_mlp.0.bias", (hid,)),
            ("router.factor_mlp.2.weight", (hid, hid)), ("router.factor_mlp.2.bias", (hid,))]
    for name, o in (("attn_bank_head", cfg.attn_banks), ("ffn_bank_head", cfg.ffn_banks),
                    ("head_slot_head", head_slots), ("ffn_slot_head", ffn_slots)):
        out += [(f"router.{name}.weight", (o, hid)), (f"router.{name}.bias", (o,))]
    out += [("router.depth_mlp.0.weight", (hid, d)), ("router.depth_mlp.0.bias", (hid,)),
            ("router.depth_mlp.2.weight", (k, hid)), ("router.depth_mlp.2.bias", (k,))]
    out += [("core.pass_gamma1", (t, d)), ("core.pass_beta1", (t, d)),
            ("core.pass_gamma2", (t, d)), ("core.pass_beta2", (t, d)),
            ("core.pass_attn_scale", (t,)), ("core.pass_mlp_scale", (t,)), ("core.alpha_inj", ()),
            ("core.norm1.weight", (d,)), ("core.attn.wqkv", (cfg.attn_banks, d, 3 * d)),
            ("core.attn.wo", (cfg.attn_banks, d, d)), ("core.norm2.weight", (d,)),
            ("core.mlp.wug", (cfg.ffn_banks, d, 2 * f)), ("core.mlp.wd", (cfg.ffn_banks, f, d))]
    out += macro_param_shapes(cfg)
    for i in range(cfg.n_coda):
        out += _block_shapes(f"coda.{i}", cfg)
    out += [("final_norm.weight", (d,)), ("shortlist_head.cluster_router.weight", (cfg.shortlist_clusters, d))]
    return out


def init_params(cfg: ModelCfg, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
    """The benchmark's weight rule: every tensor with ndim >= 2 ~ N(0, std) drawn
    from one seeded CPU generator in ``named_parameters()`` order; norm gains and
    per-pass scales 1, ``alpha_inj`` 0.1 (layers.py:826-827), biases 0."""
    gen = torch.Generator().manual_seed(seed)
    params: dict[str, torch.Tensor] = {}
    for name, shape in param_shapes(cfg):
        if len(shape) >= 2:
            params[name] = torch.randn(shape, generator=gen, dtype=torch.float32) * std
        elif name.endswith("norm1.weight") or name.endswith("norm2.weight") or name.endswith("final_norm.weight") \
                or name.endswith("pass_attn_scale") or name.endswith("pass_mlp_scale"):
            params[name] = torch.ones(shape, dtype=torch.float32)
        elif name == "core.alpha_inj":
            params[name] = torch.tensor(0.1, dtype=torch.float32)
        else:
            params[name] = torch.zeros(shape, dtype=torch.float32)
    return params


def macro_update_scale_buffer(cfg: ModelCfg) -> torch.Tensor:
    """macro.py:99-108: in the legacy shape ``update_scale`` is a buffer of ones."""
    return torch.ones(cfg.recipe_count, len(cfg.depth_choices), cfg.d_model)


# --------------------------------------------------------------------------
# synthetic Zipf token stream (stands in for the reference's TinyStories stream)
# --------------------------------------------------------------------------


def zipf_tokens(n: int, vocab: int, seed: int = 0, s: float = 1.1) -> torch.Tensor:
    ranks = torch.arange(1, vocab + 1, dtype=torch.float64)
    probs = ranks.pow(-s)
    probs = (probs / probs.sum()).float()
    gen = torch.Generator().manual_seed(seed)
    return torch.multinomial(probs, n, replacement=True, generator=gen)


def batches(tokens: torch.Tensor, batch_size: int, seq_len: int):
    """utils.py:84-99: windows of seq_len+1 with stride seq_len, wrap to 0."""
    max_start = tokens.numel() - seq_len - 1
    cursor = 0
    while True:
        xs, ys = [], []
        for _ in range(batch_size):
            if cursor > max_start:
                cursor = 0
            chunk = tokens[cursor: cursor + seq_len + 1]
            xs.append(chunk[:-1])
            ys.append(chunk[1:])
            cursor += seq_len
        yield torch.stack(xs), torch.stack(ys)


# --------------------------------------------------------------------------
# per-op restatements
# --------------------------------------------------------------------------


def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None = None, eps: float = 1e-5) -> torch.Tensor:
    """kernels/reference.py:9-17 (weight given) and macro.py:16-18 (no weight)."""
    n = x * torch.rsqrt(x.float().pow(2).mean(dim=-1, keepdim=True) + eps).to(x.dtype)
    return n if weight is None else n * weight


def rope_tables(seq: int, head_dim: int, base: float = 10000.0) -> tuple[torch.Tensor, torch.Tensor]:
    """layers.py:36-44: adjacent-pair layout, cos/sin repeated per pair."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2).float() / head_dim))
    fr = torch.outer(torch.arange(seq, dtype=torch.float32), inv)
    emb = torch.repeat_interleave(fr, 2, dim=-1)
    return emb.cos(), emb.sin()


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """kernels/reference.py:20-28 for one tensor [..., S, hd]."""
    x1, x2 = x[..., ::2], x[..., 1::2]
    rot = torch.stack((-x2, x1), dim=-1).flatten(-2)
    return x * cos + rot * sin


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """kernels/reference.py:40-41: softmax(q k^T / sqrt(hd) + causal) v on [B,H,S,hd]."""
    s = q.shape[-2]
    scores = (q @ k.transpose(-1, -2)) / math.sqrt(q.shape[-1])
    mask = torch.ones(s, s, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    return torch.softmax(scores, dim=-1) @ v


def dense_attention(x: torch.Tensor, wqkv: torch.Tensor, wo: torch.Tensor, n_heads: int) -> torch.Tensor:
    """layers.py:64-75: fused QKV (q|k|v, head-major), RoPE, causal attention, wo."""
    b, s, d = x.shape
    hd = d // n_heads
    qkv = (x @ wqkv.t()).view(b, s, 3, n_heads, hd)
    q, k, v = (t.transpose(1, 2) for t in qkv.unbind(dim=2))
    cos, sin = rope_tables(s, hd)
    y = causal_attention(rope_apply(q, cos, sin), rope_apply(k, cos, sin), v)
    return y.transpose(1, 2).reshape(b, s, d) @ wo.t()


def dense_swiglu(x: torch.Tensor, wug: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """layers.py:85-87: rows [0,F) of wug are *up*, rows [F,2F) are *gate*."""
    up, gate = (x @ wug.t()).chunk(2, dim=-1)
    return (up * F.silu(gate)) @ wd.t()


def dense_block(p: dict, prefix: str, x: torch.Tensor, n_heads: int) -> torch.Tensor:
    """layers.py:646-656 (pre-norm block)."""
    u = x + dense_attention(rmsnorm(x, p[f"{prefix}.norm1.weight"]), p[f"{prefix}.attn.wqkv.weight"],
                            p[f"{prefix}.attn.wo.weight"], n_heads)
    return u + dense_swiglu(rmsnorm(u, p[f"{prefix}.norm2.weight"]), p[f"{prefix}.mlp.wug.weight"],
                            p[f"{prefix}.mlp.wd.weight"])


def lm_loss_per_sample(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """models.py:73-75: per-token CE summed over the sequence."""
    tok = F.cross_entropy(logits.flatten(0, -2), targets.flatten(), reduction="none")
    return tok.view_as(targets).sum(dim=-1)


def argmax_lowest(x: torch.Tensor) -> torch.Tensor:
    """Index of the maximum along the last axis; ties go to the LOWEST index
    (the rule this build fixes; torch CPU argmax also returns the first max)."""
    mx = x.max(dim=-1, keepdim=True).values
    idx = torch.arange(x.shape[-1]).expand_as(x)
    return torch.where(x == mx, idx, torch.full_like(idx, x.shape[-1])).min(dim=-1).values


def topk_lowest(x: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-k along the last axis, descending value, ties to the LOWEST index
    (stable descending sort).  torch.topk's tie order is unspecified."""
    order = torch.sort(-x.double(), dim=-1, stable=True).indices[..., :k]
    return torch.gather(x, -1, order), order


def router_forward(p: dict, cfg: ModelCfg, h0: torch.Tensor, fixed_recipe: int | None,
                   fixed_depth: int | None) -> dict[str, torch.Tensor]:
    """routing.py:88-188 (temperature 1).  Only the fields the macro step and
    the audit replay consume are produced."""
    pooled = h0.mean(dim=1)

    def mlp(name: str) -> torch.Tensor:
        hid = F.silu(pooled @ p[f"router.{name}.0.weight"].t() + p[f"router.{name}.0.bias"])
        return hid @ p[f"router.{name}.2.weight"].t() + p[f"router.{name}.2.bias"]

    recipe_logits = mlp("recipe_mlp")
    depth_logits = mlp("depth_mlp")
    logits_by_pass = recipe_logits.unsqueeze(1) + p["router.pass_recipe_bias"].unsqueeze(0)
    recipe_probs = F.softmax(recipe_logits, dim=-1)
    probs_by_pass = F.softmax(logits_by_pass, dim=-1)
    depth_probs = F.softmax(depth_logits, dim=-1)
    b = h0.shape[0]
    if fixed_recipe is None:
        recipe_id = argmax_lowest(recipe_probs)
        recipe_id_by_pass = argmax_lowest(probs_by_pass)
    else:
        recipe_id = torch.full((b,), fixed_recipe, dtype=torch.long)
        recipe_id_by_pass = torch.full((b, cfg.t_max), fixed_recipe, dtype=torch.long)
    depth_values = torch.tensor(cfg.depth_choices, dtype=torch.long)
    if fixed_depth is None:
        depth_id = argmax_lowest(depth_probs)
    else:
        depth_id = torch.full((b,), list(cfg.depth_choices).index(fixed_depth), dtype=torch.long)
    recipe_entropy = -(recipe_probs.clamp_min(1e-9).log() * recipe_probs).sum(-1)
    depth_entropy = -(depth_probs.clamp_min(1e-9).log() * depth_probs).sum(-1)
    return dict(
        recipe_logits=recipe_logits, recipe_probs=recipe_probs, recipe_id=recipe_id,
        recipe_id_by_pass=recipe_id_by_pass, depth_logits=depth_logits, depth_probs=depth_probs,
        depth_id=depth_id, depth=depth_values[depth_id],
        expected_depth=(depth_probs * depth_values.float()).sum(-1),
        router_entropy=recipe_entropy + depth_entropy,
    )


def macro_phi(p: dict, cfg: ModelCfg, h: torch.Tensor, h0: torch.Tensor, recipe_ids: torch.Tensor,
              stride_ids: torch.Tensor) -> torch.Tensor:
    """macro.py:201-236, legacy shape (hidden == rank, no gate, no extra inputs):
    h + s_cfg * scale * tanh(gain*h + silu([rmsnorm(h), mean_S rmsnorm(h), h0] @ v) @ u + bias)."""
    gain = p["macro.d_gain"][recipe_ids, stride_ids]
    v = p["macro.v"][recipe_ids, stride_ids]
    u = p["macro.u"][recipe_ids, stride_ids]
    bias = p["macro.bias"][recipe_ids, stride_ids]
    scale = p.get("macro.update_scale", macro_update_scale_buffer(cfg))[recipe_ids, stride_ids]
    normed = rmsnorm(h)
    pooled = normed.mean(dim=1, keepdim=True).expand_as(normed)
    z = torch.cat([normed, pooled, h0], dim=-1)
    low = torch.bmm(F.silu(torch.bmm(z, v)), u)
    update = gain.unsqueeze(1) * h + low + bias.unsqueeze(1)
    return h + cfg.macro_update_scale * scale.unsqueeze(1) * torch.tanh(update)


def macro_consistency_loss(p: dict, cfg: ModelCfg, h0: torch.Tensor, recipe_ids: torch.Tensor) -> torch.Tensor:
    """macro.py:342-359 as audit.py:370-379 calls it (h = h0): for every stride k of the depth choices whose double 2k
    is a depth choice too, mse( Phi_2k(h0, h0),  Phi_k(Phi_k(h0, h0), h0) ) over the pairs stacked along the batch."""
    strides = list(cfg.depth_choices)
    pairs = [(i, strides.index(s * 2)) for i, s in enumerate(strides) if s * 2 in strides]       # macro.py:126
    if not pairs:
        return h0.new_zeros(())
    b = h0.shape[0]
    h_rep = h0.unsqueeze(0).expand(len(pairs), *h0.shape).reshape(len(pairs) * b, *h0.shape[1:])
    rid = recipe_ids.unsqueeze(0).expand(len(pairs), b).reshape(-1)
    src = torch.tensor([a for a, _ in pairs]).unsqueeze(1).expand(len(pairs), b).reshape(-1)
    dst = torch.tensor([c for _, c in pairs]).unsqueeze(1).expand(len(pairs), b).reshape(-1)
    direct = macro_phi(p, cfg, h_rep, h_rep, rid, dst)
    twice = macro_phi(p, cfg, macro_phi(p, cfg, h_rep, h_rep, rid, src), h_rep, rid, src)
    return F.mse_loss(direct, twice)


def stride_ids_for_depths(cfg: ModelCfg, depths: torch.Tensor) -> torch.Tensor:
    """macro.py:144-146."""
    dv = torch.tensor(cfg.depth_choices, dtype=torch.long)
    return (depths.unsqueeze(-1) == dv.unsqueeze(0)).float().argmax(dim=-1)


def banked_attention(p: dict, cfg: ModelCfg, x: torch.Tensor, r: Recipe) -> torch.Tensor:
    """layers.py:702-728: per bank, x @ wqkv[bank][:, cols|cols+d|cols+2d] ([in,out]
    layout), RoPE, causal attention over the active heads, y @ wo[bank][cols, :];
    mean over banks."""
    b, s, d = x.shape
    hd = d // cfg.n_heads
    cols = torch.tensor(recipe_head_cols(cfg, r), dtype=torch.long)
    qkv_cols = torch.cat([cols, cols + d, cols + 2 * d])
    ad = cols.numel()
    cos, sin = rope_tables(s, hd)
    out = x.new_zeros(b, s, d)
    for bank in r.attention_banks:
        qkv = x @ p["core.attn.wqkv"][bank][:, qkv_cols]
        q, k, v = (t.view(b, s, ad // hd, hd).transpose(1, 2) for t in qkv.split(ad, dim=-1))
        y = causal_attention(rope_apply(q, cos, sin), rope_apply(k, cos, sin), v)
        out = out + y.transpose(1, 2).reshape(b, s, ad) @ p["core.attn.wo"][bank][cols, :]
    return out / max(len(r.attention_banks), 1)


def banked_swiglu(p: dict, cfg: ModelCfg, x: torch.Tensor, r: Recipe) -> torch.Tensor:
    """layers.py:765-779."""
    slabs = torch.tensor(recipe_ffn_cols(cfg, r), dtype=torch.long)
    gate_cols = torch.cat([slabs, slabs + cfg.d_ff])
    out = x.new_zeros(*x.shape)
    for bank in r.ffn_banks:
        up, gate = (x @ p["core.mlp.wug"][bank][:, gate_cols]).split(slabs.numel(), dim=-1)
        out = out + (up * F.silu(gate)) @ p["core.mlp.wd"][bank][slabs, :]
    return out / max(len(r.ffn_banks), 1)


def core_step_group(p: dict, cfg: ModelCfg, h: torch.Tensor, h0: torch.Tensor, r: Recipe, t: int) -> torch.Tensor:
    """layers.py:831-852 (no global corrector): the residual base is h + alpha*h0."""
    ht = h + p["core.alpha_inj"] * h0
    n1 = rmsnorm(ht, p["core.norm1.weight"]) * (1.0 + p["core.pass_gamma1"][t]) + p["core.pass_beta1"][t]
    u = ht + p["core.pass_attn_scale"][t] * banked_attention(p, cfg, n1, r)
    n2 = rmsnorm(u, p["core.norm2.weight"]) * (1.0 + p["core.pass_gamma2"][t]) + p["core.pass_beta2"][t]
    return u + p["core.pass_mlp_scale"][t] * banked_swiglu(p, cfg, n2, r)


def core_forward_step(p: dict, cfg: ModelCfg, h: torch.Tensor, h0: torch.Tensor, recipe_ids: torch.Tensor,
                      active: torch.Tensor, t: int) -> torch.Tensor:
    """layers.py:854-870: samples grouped by recipe, inactive ones pass through."""
    recipes = build_recipes(cfg)
    pieces = []
    for i in range(h.shape[0]):
        if bool(active[i]):
            pieces.append(core_step_group(p, cfg, h[i:i + 1], h0[i:i + 1], recipes[int(recipe_ids[i])], t))
        else:
            pieces.append(h[i:i + 1])
    return torch.cat(pieces, dim=0)


def coda_logits(p: dict, cfg: ModelCfg, h: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """models.py:185-192: coda blocks, final norm, tied-embedding logits."""
    for i in range(cfg.n_coda):
        h = dense_block(p, f"coda.{i}", h, cfg.n_heads)
    hidden = rmsnorm(h, p["final_norm.weight"])
    return hidden, hidden @ p["embed.weight"].t()


def exact_from_h0(p: dict, cfg: ModelCfg, h0: torch.Tensor, targets: torch.Tensor, route: dict,
                  schedule: tuple | None = None) -> dict:
    """models.py:416-512 with reused router decisions: t_max banked passes using the
    per-pass recipe ids, samples with depth <= t frozen.  `schedule` (models.py:230-247, 449-451): pass t runs recipe
    schedule[t] for every sample instead."""
    if schedule is not None:
        if len(schedule) < cfg.t_max:
            raise ValueError(f"fixed_recipe_schedule length {len(schedule)} is shorter than t_max={cfg.t_max}")
        if any(not 0 <= int(r) < cfg.recipe_count for r in schedule):
            raise ValueError("fixed_recipe_schedule recipe outside the recipe bank")
    h = h0
    for t in range(cfg.t_max):
        rid = route["recipe_id_by_pass"][:, t] if schedule is None else torch.full_like(route["recipe_id"], int(schedule[t]))
        h = core_forward_step(p, cfg, h, h0, rid, route["depth"] > t, t)
    hidden, logits = coda_logits(p, cfg, h)
    return dict(recurrent_hidden=h, hidden=hidden, logits=logits,
                loss_per_sample=lm_loss_per_sample(logits, targets))


def forward_macro(p: dict, cfg: ModelCfg, tokens: torch.Tensor, targets: torch.Tensor,
                  fixed_recipe: int | None = None, fixed_depth: int | None = None, oc: OutputCfg | None = None,
                  seed: int = 0, top_clusters: torch.Tensor | None = None) -> dict:
    """models.py:681-723 (full-vocabulary branch, or the shortlist branch when `oc` is given)."""
    h0 = p["embed.weight"][tokens]
    for i in range(cfg.n_prelude):
        h0 = dense_block(p, f"prelude.{i}", h0, cfg.n_heads)
    route = router_forward(p, cfg, h0, fixed_recipe, fixed_depth)
    if [n for n, _ in macro_param_shapes(cfg)] != ["macro.d_gain", "macro.v", "macro.u", "macro.bias"]:
        raise NotImplementedError("the macro operator is restated in its plain bounded-residual form only")
    h = macro_phi(p, cfg, h0, h0, route["recipe_id"], stride_ids_for_depths(cfg, route["depth"]))
    if oc is not None:
        x = h
        for i in range(cfg.n_coda):
            x = dense_block(p, f"coda.{i}", x, cfg.n_heads)
        hidden = rmsnorm(x, p["final_norm.weight"])
        sl = shortlist_loss(p, cfg, oc, hidden, targets, seed, top_clusters)
        return dict(h0=h0, route=route, recurrent_hidden=h, hidden=hidden, logits=sl["logits"], shortlist=sl,
                    loss_per_sample=sl["loss_per_sample"])
    hidden, logits = coda_logits(p, cfg, h)
    return dict(h0=h0, route=route, recurrent_hidden=h, hidden=hidden, logits=logits,
                loss_per_sample=lm_loss_per_sample(logits, targets))


def shortlist_candidates(targets: torch.Tensor, top_clusters: torch.Tensor, random_negs: torch.Tensor, vocab: int,
                         oc: OutputCfg) -> torch.Tensor:
    """output.py:81-108: [target | members of the top clusters | hard | random | filler | target + 0..2K-1]."""
    c, k = oc.num_clusters, oc.shortlist_max_tokens
    mpc = (vocab + c - 1) // c
    members = top_clusters.unsqueeze(-1) + torch.arange(mpc).view(1, 1, 1, -1) * c      # cluster c = ids c, c+C, ...
    members = torch.where(members < vocab, members, torch.zeros_like(members)).flatten(start_dim=-2)
    b, s = targets.shape
    hard = (torch.arange(oc.hard_negatives) % vocab).view(1, 1, -1).expand(b, s, -1)
    filler = (torch.arange(k) % vocab).view(1, 1, -1).expand(b, s, -1)
    tfill = (targets.unsqueeze(-1) + torch.arange(2 * k).view(1, 1, -1)) % vocab
    return torch.cat([targets.unsqueeze(-1), members, hard, random_negs, filler, tfill], dim=-1)


def dedupe_preserve_first(cands: torch.Tensor, k: int) -> torch.Tensor:
    """output.py:46-70: the k distinct ids with the smallest first position, in that order."""
    flat = cands.reshape(-1, cands.shape[-1])
    out = torch.empty(flat.shape[0], k, dtype=torch.long)
    for r in range(flat.shape[0]):
        seen: dict[int, None] = {}
        for v in flat[r].tolist():
            if v not in seen:
                seen[v] = None
                if len(seen) == k:
                    break
        out[r] = torch.tensor(list(seen), dtype=torch.long)
    return out.view(*cands.shape[:-1], k)


def shortlist_loss(p: dict, cfg: ModelCfg, oc: OutputCfg, hidden: torch.Tensor, targets: torch.Tensor, seed: int,
                   top_clusters: torch.Tensor | None = None) -> dict:
    """output.py:72-136: cluster router -> top clusters -> shortlist -> gathered-row logits -> CE vs slot 0.
    `top_clusters` may be injected (tests that compare at identical routing)."""
    b, s, _ = hidden.shape
    cluster_logits = hidden @ p["shortlist_head.cluster_router.weight"].t()
    if top_clusters is None:
        top_clusters = topk_lowest(cluster_logits, min(oc.shortlist_top_clusters, oc.num_clusters))[1]
    gen = torch.Generator().manual_seed(seed)
    random_negs = torch.randint(0, cfg.vocab_size, (b, s, oc.random_negatives), generator=gen)
    cands = shortlist_candidates(targets, top_clusters, random_negs, cfg.vocab_size, oc)
    shortlist = dedupe_preserve_first(cands, oc.shortlist_max_tokens)
    rows = p["embed.weight"][shortlist]
    logits = (hidden.unsqueeze(-2) * rows).sum(dim=-1)
    tok = F.cross_entropy(logits.flatten(0, -2), torch.zeros(b * s, dtype=torch.long), reduction="none").view(b, s)
    return dict(loss_per_sample=tok.sum(-1), logits=logits, shortlist=shortlist, cluster_logits=cluster_logits,
                top_clusters=top_clusters, random_negs=random_negs)


def forward_dense(p: dict, cfg: ModelCfg, tokens: torch.Tensor, targets: torch.Tensor) -> dict:
    """models.py:98-122."""
    x = p["embed.weight"][tokens]
    for i in range(cfg.n_dense_layers):
        x = dense_block(p, f"blocks.{i}", x, cfg.n_heads)
    hidden = rmsnorm(x, p["final_norm.weight"])
    logits = hidden @ p["embed.weight"].t()
    return dict(hidden=hidden, logits=logits, loss_per_sample=lm_loss_per_sample(logits, targets))


def router_aux_losses(tr: TrainCfg, recipe_probs: torch.Tensor, expected_depth: torch.Tensor,
                      usage_ema: torch.Tensor) -> dict[str, torch.Tensor]:
    """metrics.py:97-112."""
    if tr.disable_router_aux:  # training.py:510-512
        z = recipe_probs.new_zeros(())
        return dict(load=z, cover=z, depth=z)
    r = recipe_probs.shape[-1]
    load = r * recipe_probs.mean(dim=0).square().sum() - 1.0
    cover = F.relu(tr.coverage_min - usage_ema).square().sum()
    return dict(load=tr.lambda_load * load, cover=tr.lambda_cover * cover,
                depth=tr.lambda_depth * expected_depth.float().mean())


def _rms(x: torch.Tensor, dim) -> torch.Tensor:
    return x.float().pow(2).mean(dim=dim).sqrt()


def macro_distill_loss(tr: TrainCfg, hot_hidden, exact_hidden, hot_logits, exact_logits, h0) -> dict:
    """macro.py:394-469, delta objective (h0 given); rms-trust term off."""
    exact_hidden, exact_logits, h0 = exact_hidden.detach(), exact_logits.detach(), h0.detach()
    dp, de = hot_hidden - h0, exact_hidden - h0
    delta_dir = 1.0 - F.cosine_similarity(dp.flatten(1), de.flatten(1), dim=-1, eps=1e-8).mean()
    delta_rms = (torch.log(_rms(dp, (1, 2)).clamp_min(1e-8)) - torch.log(_rms(de, (1, 2)).clamp_min(1e-8))).square().mean()
    endpoint_normed = F.smooth_l1_loss(rmsnorm(hot_hidden), rmsnorm(exact_hidden))
    endpoint_raw = F.smooth_l1_loss(hot_hidden, exact_hidden)
    temp = max(float(tr.distill_temperature), 1e-6)
    if hot_logits.shape == exact_logits.shape:
        exact_logp = F.log_softmax(exact_logits / temp, dim=-1)
        hot_logp = F.log_softmax(hot_logits / temp, dim=-1)
        kl = F.kl_div(hot_logp, exact_logp.exp(), reduction="batchmean") * temp ** 2
    else:       # shortlist logits [.., K] against exact full-vocabulary logits [.., V]: no KL term (macro.py:452)
        kl = hot_hidden.new_zeros(())
    return dict(kl=tr.lambda_kl * kl, delta_dir=tr.lambda_delta_dir * delta_dir,
                delta_rms=tr.lambda_delta_rms * delta_rms,
                endpoint_normed=tr.lambda_endpoint_normed * endpoint_normed,
                endpoint_raw=tr.lambda_endpoint_raw * endpoint_raw)


def macro_alignment_metrics(hot_hidden: torch.Tensor, exact_hidden: torch.Tensor, h0: torch.Tensor,
                            hot_logits: torch.Tensor | None = None, exact_logits: torch.Tensor | None = None) -> dict:
    """macro.py:499-546 with audit.py:207-243: cosine / mse / norms of the macro and the exact endpoint and of their
    deltas against h0, each per-sample quantity averaged over the audited samples, and the KL(exact || hot) of the
    audited rows' logits at temperature 1 (metrics.py:119-124), averaged over rows."""
    hot_hidden, exact_hidden, h0 = hot_hidden.detach(), exact_hidden.detach(), h0.detach()
    out = dict(hidden_cosine_exact_macro=F.cosine_similarity(hot_hidden.flatten(1), exact_hidden.flatten(1), dim=-1, eps=1e-8).mean(),
               hidden_mse_exact_macro=(hot_hidden - exact_hidden).square().mean())
    macro_norm, exact_norm = _rms(hot_hidden, (1, 2)).mean(), _rms(exact_hidden, (1, 2)).mean()
    dp, de = hot_hidden - h0, exact_hidden - h0
    pred_rms, exact_rms = _rms(dp, (1, 2)).mean(), _rms(de, (1, 2)).mean()
    out.update(macro_norm=macro_norm, exact_norm=exact_norm, macro_exact_norm_ratio=macro_norm / exact_norm.clamp_min(1e-8),
               delta_cosine_exact_macro=F.cosine_similarity(dp.flatten(1), de.flatten(1), dim=-1, eps=1e-8).mean(),
               delta_rms_exact=exact_rms, delta_rms_pred=pred_rms, delta_rms_ratio=pred_rms / exact_rms.clamp_min(1e-8))
    out.update(hidden_cosine=out["hidden_cosine_exact_macro"], hidden_residual_l2=out["hidden_mse_exact_macro"].sqrt())
    if hot_logits is not None and exact_logits is not None and hot_logits.shape == exact_logits.shape:
        le, lh = F.log_softmax(exact_logits.detach(), dim=-1), F.log_softmax(hot_logits.detach(), dim=-1)
        out["logit_kl_exact_macro"] = out["logit_kl"] = (le.exp() * (le - lh)).sum(dim=-1).mean()
    return {k: float(v) for k, v in out.items()}


def audit_schedule_next_count(tr: TrainCfg, current: int, metrics: dict, batch_size: int, state: dict) -> int:
    """audit.py:137-185: after a step that audited somebody, the fixed count halves (not below the minimum) when the
    macro endpoint tracked the exact one -- small loss residual, cosine, delta-RMS ratio, mse, norm, residual variance
    within their thresholds, mse and norm not rising since the last audited step -- and doubles (up to the batch)
    otherwise.  `state` keeps the last mse and norm.  A missing metric counts as failing its test."""
    if not tr.audit_schedule_enabled or current <= 0:
        return current
    inf = float("inf")
    min_count = tr.audit_schedule_min_count if tr.audit_schedule_min_count is not None else max(1, batch_size // 128)
    hidden_cos = float(metrics.get("hidden_cosine_exact_macro", 0.0))
    residual_var = float(metrics.get("audit_residual_var", inf))
    loss_gap = abs(float(metrics.get("hot_exact_nll_gap", metrics.get("loss_residual", inf))))
    ratio = float(metrics.get("delta_rms_ratio", inf))
    mse, macro_norm = float(metrics.get("hidden_mse_exact_macro", inf)), float(metrics.get("macro_norm", inf))
    norm_limit = tr.audit_schedule_macro_norm_threshold
    if norm_limit is None:
        norm_limit = tr.audit_schedule_macro_norm_threshold_mult * float(metrics.get("exact_norm", 0.0))
    mse_slope = 0.0 if state.get("last_hidden_mse") is None else mse - state["last_hidden_mse"]
    norm_slope = 0.0 if state.get("last_macro_norm") is None else macro_norm - state["last_macro_norm"]
    good = (loss_gap <= tr.audit_schedule_nll_gap_threshold
            and hidden_cos >= tr.audit_schedule_hidden_cosine_threshold
            and tr.audit_schedule_delta_rms_ratio_min <= ratio <= tr.audit_schedule_delta_rms_ratio_max
            and mse <= tr.audit_schedule_hidden_mse_threshold
            and macro_norm <= norm_limit
            and (not tr.audit_schedule_require_negative_mse_slope or mse_slope <= 0)
            and (not tr.audit_schedule_require_negative_norm_slope or norm_slope <= 0)
            and residual_var <= tr.audit_schedule_residual_var_threshold)
    state["last_hidden_mse"], state["last_macro_norm"] = mse, macro_norm
    return max(min_count, current // 2) if good else min(batch_size, max(current, current * 2))


def audit_choice(n: int, k: int, seed: int) -> torch.Tensor:
    """audit.py:99-116 fixed-count sampler: the first k entries of a seeded
    permutation (CPU generator), inclusion probability k/n for every sample."""
    gen = torch.Generator().manual_seed(seed)
    return torch.randperm(n, generator=gen)[:k]


def audit_probability(tr: TrainCfg, route: dict, recent_residual: float, audit_ema: torch.Tensor) -> torch.Tensor:
    """audit.py:79-97: requested audit probability per sample from the router's entropy, the residual seen at the last
    audit and how far the sample's recipe is below its audit-coverage floor."""
    r_plus_k = route["recipe_logits"].shape[-1] + route["depth_logits"].shape[-1]
    uncertainty = route["router_entropy"].detach() / r_plus_k
    deficit = (tr.coverage_min - audit_ema[route["recipe_id"]]).clamp_min(0.0) / max(tr.coverage_min, 1e-12)
    prob = tr.audit_p_min + tr.audit_alpha * uncertainty + tr.audit_beta * recent_residual + tr.audit_gamma * deficit
    return prob.clamp(tr.audit_p_min, tr.audit_p_max)


def audit_sample_bernoulli(prob: torch.Tensor, seed: int, cap: int | None) -> tuple[torch.Tensor, torch.Tensor]:
    """audit.py:117-132: Bernoulli draws from a seeded CPU generator; more than `cap` hits are thinned to `cap` by a
    seeded permutation of the hit list, and the inclusion probability becomes p * cap / hits."""
    gen = torch.Generator().manual_seed(seed)
    mask = torch.bernoulli(prob, generator=gen).bool()
    inclusion = prob.clone()
    if cap is not None and int(mask.sum()) > cap:
        selected = mask.nonzero(as_tuple=False).flatten()
        perm = torch.randperm(selected.numel(), generator=gen)
        capped = torch.zeros_like(mask)
        capped[selected[perm[:cap]]] = True
        inclusion = prob * (float(cap) / float(selected.numel()))
        mask = capped
    return mask, inclusion


def macro_step_loss(p: dict, cfg: ModelCfg, tr: TrainCfg, tokens: torch.Tensor, targets: torch.Tensor,
                    step: int, usage_ema: torch.Tensor, oc: OutputCfg | None = None,
                    top_clusters: torch.Tensor | None = None, audit_state: dict | None = None) -> tuple[torch.Tensor, dict]:
    """training.py:1336-1392 + audit.py:245-387 (fixed-count sampler,
    the three audit modes, residual clip, consistency term)."""
    shortlist = tr.mode == "recursive_macro_shortlist"
    hot = forward_macro(p, cfg, tokens, targets, tr.fixed_recipe, tr.fixed_depth, oc if shortlist else None,
                        seed=tr.seed + step, top_clusters=top_clusters)      # training.py:1364
    corrected = hot["loss_per_sample"].clone()
    aux: dict[str, torch.Tensor] = {}
    info: dict[str, Any] = dict(hot=hot)
    k = tr.audit_fixed_count_per_batch or 0
    if tr.audit_schedule_enabled and audit_state is not None:
        k = int(audit_state.get("fixed_count", k))           # audit.py:182-183: the schedule rewrites the count
    b = tokens.shape[0]
    mask = p_inc = None
    if tr.audit_sampler == "bernoulli" and tr.audit_p_max > 0:
        state = audit_state if audit_state is not None else {}
        ema = state.setdefault("audit_ema", torch.zeros(cfg.recipe_count))
        prob = audit_probability(tr, hot["route"], float(state.get("recent_residual", 0.0)), ema)
        mask, p_inc = audit_sample_bernoulli(prob.detach().float(), tr.seed + 10_000 + step, tr.audit_cap)
        info.update(audit_prob=prob)
    elif k > 0:
        chosen = audit_choice(b, min(k, b), tr.seed + 10_000 + step)
        mask = torch.zeros(b, dtype=torch.bool)
        mask[chosen] = True
        p_inc = torch.full((b,), float(min(k, b)) / float(b))
    if mask is not None and bool(mask.any()):
        route = {key: val[mask] for key, val in hot["route"].items()}
        exact = exact_from_h0(p, cfg, hot["h0"][mask], targets[mask], route)
        hot_subset = hot["loss_per_sample"][mask]
        residual = exact["loss_per_sample"] - hot_subset
        raw = residual.detach().float()                   # audit.py:306-310,363: reported before the clip
        info["residual"] = dict(audit_residual_mean=float(raw.mean()), audit_residual_std=float(raw.std(unbiased=False)),
                                audit_residual_var=float(raw.var(unbiased=False)), loss_residual=float(raw.mean()))
        if tr.audit_residual_clip is not None:
            residual = residual.clamp(-tr.audit_residual_clip, tr.audit_residual_clip)
        info["residual"]["clipped_loss_residual"] = float(residual.detach().mean())
        if tr.audit_mode == "gradient_corrected":
            corrected[mask] = hot_subset + residual / p_inc[mask].clamp_min(1e-12)
        aux = macro_distill_loss(tr, hot["recurrent_hidden"][mask], exact["recurrent_hidden"],
                                 hot["logits"][mask], exact["logits"], hot["h0"][mask])
        info.update(exact=exact, alignment=macro_alignment_metrics(hot["recurrent_hidden"][mask], exact["recurrent_hidden"],
                                                                   hot["h0"][mask], hot["logits"][mask], exact["logits"]))
        info["audit_count"] = int(mask.sum())
        if tr.audit_schedule_enabled and tr.audit_sampler != "bernoulli" and audit_state is not None:      # audit.py:365
            audit_state["fixed_count"] = audit_schedule_next_count(tr, k, dict(info["alignment"], **info["residual"]), b,
                                                                    audit_state)
            info["audit_schedule_next_count"] = audit_state["fixed_count"]
        if audit_state is not None:          # audit.py:213-218: the residual the next step's probabilities see
            cos = F.cosine_similarity(hot["recurrent_hidden"][mask].detach().flatten(1),
                                      exact["recurrent_hidden"].detach().flatten(1), dim=-1, eps=1e-8).mean()
            audit_state["recent_residual"] = float((1.0 - cos).clamp_min(0))
    if mask is not None:
        info.update(mask=mask, p_inc=p_inc)
        if audit_state is not None and "audit_ema" in audit_state:        # audit.py:70-77
            counts = torch.bincount(hot["route"]["recipe_id"][mask].long(), minlength=cfg.recipe_count).float()
            audit_state["audit_ema"].mul_(tr.coverage_beta).add_(counts / counts.sum().clamp_min(1.0), alpha=1.0 - tr.coverage_beta)
    if tr.lambda_cons != 0.0:       # audit.py:370-379: on every step of the macro modes, audited or not
        aux = dict(aux, cons=tr.lambda_cons * macro_consistency_loss(p, cfg, hot["h0"], hot["route"]["recipe_id"]))
    aux_router = router_aux_losses(tr, hot["route"]["recipe_probs"], hot["route"]["expected_depth"], usage_ema)
    loss = corrected.mean() / float(targets.shape[1]) + sum(aux.values()) + sum(aux_router.values())
    info.update(corrected=corrected, aux=aux, aux_router=aux_router)
    return loss, info


def exact_step_loss(p: dict, cfg: ModelCfg, tr: TrainCfg, tokens: torch.Tensor, targets: torch.Tensor,
                    usage_ema: torch.Tensor) -> tuple[torch.Tensor, dict]:
    """training.py:771-797 (`recursive_exact`): prelude -> router -> t_max banked passes for every sample -> coda ->
    cross entropy, plus the router's auxiliary losses (models.py:202-228, 416-512)."""
    h0 = p["embed.weight"][tokens]
    for i in range(cfg.n_prelude):
        h0 = dense_block(p, f"prelude.{i}", h0, cfg.n_heads)
    route = router_forward(p, cfg, h0, tr.fixed_recipe, tr.fixed_depth)
    out = exact_from_h0(p, cfg, h0, targets, route, tr.fixed_recipe_schedule)
    aux_router = router_aux_losses(tr, route["recipe_probs"], route["expected_depth"], usage_ema)
    loss = out["loss_per_sample"].mean() / float(targets.shape[1]) + sum(aux_router.values())
    out.update(route=route, h0=h0)
    if tr.fixed_recipe_schedule is not None:      # models.py:480-497: what the usage average then counts
        out["usage_ids"] = torch.tensor([int(r) for r in tr.fixed_recipe_schedule[:cfg.t_max]]).expand(h0.shape[0], -1)
    return loss, dict(hot=out, aux_router=aux_router)


def deferred_schedule(cfg: ModelCfg, tr: TrainCfg) -> list[int]:
    """models.py:551-566: one recipe per micro-pass of the grouped block -- `fixed_recipe` (default 1) repeated
    `fixed_depth` (default t_max) times, or the first entries of `fixed_recipe_schedule`, its last one repeated."""
    depth = max(1, min(int(tr.fixed_depth or cfg.t_max), cfg.t_max))
    if tr.fixed_recipe_schedule is None:
        schedule = [int(tr.fixed_recipe if tr.fixed_recipe is not None else 1)] * depth
    else:
        schedule = [int(r) for r in tr.fixed_recipe_schedule[:depth]] or [int(tr.fixed_recipe if tr.fixed_recipe is not None else 1)]
        schedule += [schedule[-1]] * (depth - len(schedule))
    for r in schedule:
        if not 0 <= r < cfg.recipe_count:
            raise ValueError(f"deferred grouped recipe {r} is outside [0, {cfg.recipe_count})")
    return schedule


def deferred_grouped_block(p: dict, cfg: ModelCfg, h: torch.Tensor, h0: torch.Tensor, schedule: list[int],
                           active: torch.Tensor) -> torch.Tensor:
    """layers.py:872-912 (no global corrector): ONE block whose attention and MLP halves each sum the branches of all
    scheduled recipes, every branch reading the same normed input under its own pass's FiLM and scale."""
    recipes = build_recipes(cfg)
    ht = h + p["core.alpha_inj"] * h0
    n1 = rmsnorm(ht, p["core.norm1.weight"])
    u = ht
    for t, rid in enumerate(schedule):
        i = min(t, cfg.t_max - 1)
        u = u + p["core.pass_attn_scale"][i] * banked_attention(p, cfg, n1 * (1.0 + p["core.pass_gamma1"][i]) + p["core.pass_beta1"][i],
                                                                recipes[rid])
    n2 = rmsnorm(u, p["core.norm2.weight"])
    out = u
    for t, rid in enumerate(schedule):
        i = min(t, cfg.t_max - 1)
        out = out + p["core.pass_mlp_scale"][i] * banked_swiglu(p, cfg, n2 * (1.0 + p["core.pass_gamma2"][i]) + p["core.pass_beta2"][i],
                                                                recipes[rid])
    return torch.where(active.view(-1, 1, 1), out, h)


def deferred_step_loss(p: dict, cfg: ModelCfg, tr: TrainCfg, tokens: torch.Tensor, targets: torch.Tensor,
                       usage_ema: torch.Tensor) -> tuple[torch.Tensor, dict]:
    """training.py:823-877 (`recursive_deferred_grouped_exact`), models.py:538-603."""
    h0 = p["embed.weight"][tokens]
    for i in range(cfg.n_prelude):
        h0 = dense_block(p, f"prelude.{i}", h0, cfg.n_heads)
    route = router_forward(p, cfg, h0, tr.fixed_recipe, tr.fixed_depth)
    schedule = deferred_schedule(cfg, tr)
    h = deferred_grouped_block(p, cfg, h0, h0, schedule, route["depth"] > 0)
    hidden, logits = coda_logits(p, cfg, h)
    out = dict(recurrent_hidden=h, hidden=hidden, logits=logits, loss_per_sample=lm_loss_per_sample(logits, targets),
               route=route, h0=h0, usage_ids=torch.tensor(schedule).expand(h0.shape[0], -1))
    aux_router = router_aux_losses(tr, route["recipe_probs"], route["expected_depth"], usage_ema)
    loss = out["loss_per_sample"].mean() / float(targets.shape[1]) + sum(aux_router.values())
    return loss, dict(hot=out, aux_router=aux_router)


def dense_step_loss(p: dict, cfg: ModelCfg, tokens: torch.Tensor, targets: torch.Tensor) -> tuple[torch.Tensor, dict]:
    """training.py:742-769."""
    out = forward_dense(p, cfg, tokens, targets)
    return out["loss_per_sample"].mean() / float(targets.shape[1]), dict(hot=out)


def update_usage(usage_ema: torch.Tensor, recipe_ids: torch.Tensor, beta: float) -> torch.Tensor:
    """recipes.py:119-123."""
    counts = torch.bincount(recipe_ids.long().flatten(), minlength=usage_ema.numel()).float()
    return usage_ema * beta + (counts / counts.sum().clamp_min(1.0)) * (1.0 - beta)


def adamw_update(param: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor, step: int,
                 lr: float, wd: float, betas=(0.9, 0.999), eps: float = 1e-8) -> None:
    """torch.optim.AdamW single-tensor rule (training.py:341-354 builds it with
    default betas/eps): decoupled decay, bias-corrected moments, in place."""
    b1, b2 = betas
    param.mul_(1.0 - lr * wd)
    m.mul_(b1).add_(grad, alpha=1.0 - b1)
    v.mul_(b2).addcmul_(grad, grad, value=1.0 - b2)
    bc1, bc2 = 1.0 - b1 ** step, 1.0 - b2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    param.addcdiv_(m, denom, value=-lr / bc1)


@dataclass
class OracleTrainer:
    """training.py:1336-1476 + 445-468 as a loop over ``step``.  Parameters that
    received no gradient are skipped by the optimiser exactly as
    ``torch.optim.AdamW`` skips ``grad is None`` (no decay, no step count)."""
    cfg: ModelCfg
    tr: TrainCfg
    params: dict
    global_step: int = 0
    usage_ema: torch.Tensor | None = None
    opt_state: dict = field(default_factory=dict)
    oc: OutputCfg | None = None
    top_clusters: torch.Tensor | None = None      # test hook: shortlist routing injected for the next step
    audit_state: dict = field(default_factory=dict)       # Bernoulli sampler: recent residual, audit-coverage average

    def __post_init__(self) -> None:
        if self.usage_ema is None:
            self.usage_ema = torch.zeros(self.cfg.recipe_count)

    def loss_and_grads(self, tokens: torch.Tensor, targets: torch.Tensor, commit: bool = False):
        """`commit`: let the step advance the Bernoulli sampler's state (what `train_step` does); a bare call leaves it."""
        import copy
        state = self.audit_state if commit else copy.deepcopy(self.audit_state)
        leaves = {k: v.detach().clone().requires_grad_(True) for k, v in self.params.items()}
        if self.cfg.topology == "dense":
            loss, info = dense_step_loss(leaves, self.cfg, tokens, targets)
        elif self.tr.mode == "recursive_exact":
            loss, info = exact_step_loss(leaves, self.cfg, self.tr, tokens, targets, self.usage_ema)
        elif self.tr.mode == "recursive_deferred_grouped_exact":
            loss, info = deferred_step_loss(leaves, self.cfg, self.tr, tokens, targets, self.usage_ema)
        else:
            loss, info = macro_step_loss(leaves, self.cfg, self.tr, tokens, targets, self.global_step, self.usage_ema,
                                         self.oc, self.top_clusters, audit_state=state)
        loss.backward()
        grads = {k: v.grad for k, v in leaves.items() if v.grad is not None}
        if self.tr.grad_clip_norm is not None:  # training.py:456-462, before the optimiser reads them
            total = torch.sqrt(sum(g.float().pow(2).sum() for g in grads.values()))
            coef = min(1.0, float(self.tr.grad_clip_norm / (total + 1e-6)))
            grads = {k: g * coef for k, g in grads.items()}
        return loss.detach(), grads, info

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> float:
        loss, grads, info = self.loss_and_grads(tokens, targets, commit=True)
        self.last_info = info            # what the step decided (routing, audited subset), for the parity tests
        for name, g in grads.items():
            st = self.opt_state.setdefault(name, dict(step=0, m=torch.zeros_like(g), v=torch.zeros_like(g)))
            st["step"] += 1
            adamw_update(self.params[name], g, st["m"], st["v"], st["step"], self.tr.lr,
                         self.tr.weight_decay, self.tr.betas, self.tr.eps)
        if self.cfg.topology != "dense":
            ids = info["hot"].get("usage_ids", info["hot"]["route"]["recipe_id"])
            self.usage_ema = update_usage(self.usage_ema, ids, self.tr.coverage_beta)
        self.global_step += 1
        return float(loss)


# ----------------------------------------------------------------------------- static cluster-pool sparse FFN
def cluster_route(x: torch.Tensor, up_a: torch.Tensor, gate_a: torch.Tensor, centers: torch.Tensor) -> torch.Tensor:
    """kernels/cluster_pool_ffn.py:127-139: arg-max over centres of the L2-normalised selector features
    (lowest index on ties, the rule this build fixes)."""
    feats = F.normalize(torch.cat([x @ up_a, x @ gate_a], dim=-1).float(), dim=-1)
    return argmax_lowest(feats @ centers.float().t())


def cluster_pack_indices(assignments: torch.Tensor, cluster_count: int):
    """kernels/cluster_pool_ffn.py:162-188: per cluster the member tokens in ascending order, padded with token 0
    to the largest cluster; flat_gather[token] = cluster * max_count + rank."""
    counts = torch.bincount(assignments, minlength=cluster_count)
    max_count = int(counts.max()) if counts.numel() else 0
    pack_index = torch.zeros(cluster_count, max_count, dtype=torch.long)
    flat_gather = torch.empty(assignments.shape[0], dtype=torch.long)
    for c in range(cluster_count):
        idx = torch.nonzero(assignments == c).flatten()
        pack_index[c, : idx.numel()] = idx
        flat_gather[idx] = c * max_count + torch.arange(idx.numel())
    return pack_index, flat_gather, counts, max_count


def cluster_pool_ffn(x: torch.Tensor, assignments: torch.Tensor, w_up: torch.Tensor, w_gate: torch.Tensor,
                     w_down_rows: torch.Tensor, candidate_ids: torch.Tensor) -> torch.Tensor:
    """kernels/cluster_pool_ffn.py:90-124,142-159: every token runs SwiGLU over its cluster's candidate neurons.
    w_up / w_gate / w_down_rows are [d_ff, d_model] (row f = neuron f); differentiable."""
    out = torch.zeros_like(x)
    for c in range(candidate_ids.shape[0]):
        idx = torch.nonzero(assignments == c).flatten()
        if idx.numel() == 0:
            continue
        ids = candidate_ids[c]
        xc = x[idx]
        z = (xc @ w_up[ids].t()) * F.silu(xc @ w_gate[ids].t())
        out = out.index_add(0, idx, z @ w_down_rows[ids])
    return out


def static_cluster_pool_swiglu(x: torch.Tensor, wug: torch.Tensor, wd: torch.Tensor, up_a: torch.Tensor,
                               gate_a: torch.Tensor, centers: torch.Tensor, candidate_ids: torch.Tensor,
                               assignments: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """layers.py:188-220: route, then the pooled FFN with wug [2F, d] = (up rows | gate rows), wd [d, F]."""
    flat = x.reshape(-1, x.shape[-1])
    if assignments is None:
        assignments = cluster_route(flat, up_a, gate_a, centers)
    f = wd.shape[1]
    out = cluster_pool_ffn(flat, assignments, wug[:f], wug[f:], wd.t(), candidate_ids)
    return out.view(x.shape), assignments


# ----------------------------------------------------------------------------- SVD-factor sparse FFN (mask mode)
def topk_membership(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Boolean mask of the k largest entries per row, lowest index first among equals."""
    mask = torch.zeros_like(scores, dtype=torch.bool)
    if k > 0:
        mask.scatter_(-1, topk_lowest(scores, min(k, scores.shape[-1]))[1], True)
    return mask


def svd_ffn_hats(x, up_a, up_b, gate_a, gate_b):
    """layers.py:585-588: low-rank estimates of the up and gate pre-activations."""
    return (x @ up_a) @ up_b, (x @ gate_a) @ gate_b


def svd_ffn_candidates(up_hat, gate_hat, wd_norm, up_m: int, gate_m: int, product_m: int) -> torch.Tensor:
    """layers.py:589-592,473-489: union of the top-m neurons under the three selector scores."""
    gact = F.silu(gate_hat)
    cand = topk_membership(up_hat.abs() * wd_norm, up_m)
    cand |= topk_membership(gact.abs() * wd_norm, gate_m)
    cand |= topk_membership((up_hat * gact).abs() * wd_norm, product_m)
    return cand


def svd_ffn_select(z, cand, wd_norm, top_k: int) -> torch.Tensor:
    """layers.py:617-621: the top_k candidates by |z| * ||w_down row||."""
    return topk_membership((z.abs() * wd_norm).masked_fill(~cand, float("-inf")), top_k)


def svd_sparse_ffn(x, w_up, w_gate, w_down, up_a, up_b, gate_a, gate_b, *, top_k: int, up_m: int, gate_m: int,
                   product_m: int, selected: torch.Tensor | None = None):
    """SVDFactorSparseFFN.forward in mask mode (layers.py:531-637): exact SwiGLU over the selected neurons only.
    Differentiable in x and the three weight matrices; the selection carries no gradient.  Requires
    max(up_m, gate_m, product_m) >= top_k (otherwise the reference's result depends on an unspecified order)."""
    flat = x.reshape(-1, x.shape[-1])
    wd_norm = w_down.detach().float().norm(dim=-1)
    z = (flat @ w_up.t()) * F.silu(flat @ w_gate.t())
    if selected is None:
        up_hat, gate_hat = svd_ffn_hats(flat.detach(), up_a, up_b, gate_a, gate_b)
        cand = svd_ffn_candidates(up_hat, gate_hat, wd_norm, up_m, gate_m, product_m)
        selected = svd_ffn_select(z.detach(), cand, wd_norm, top_k)
    out = (z * selected) @ w_down
    return out.view(x.shape), selected


# ----------------------------------------------------------------------------- offline cluster-pool codebook build
def svd_factor_cache(wug: torch.Tensor, max_rank: int) -> dict[str, torch.Tensor]:
    """cli.py:3244-3261: truncated SVD factors of the up and gate halves of a fused W_ug [2F, d] (transposed to
    [d, F]): `*_a` = U[:, :r] * S[:r] ([d, r]), `*_b` = Vh[:r, :] ([r, F])."""
    up_w, gate_w = wug.detach().float().chunk(2, dim=0)
    out: dict[str, torch.Tensor] = {}
    for name, mat in (("up", up_w.t().contiguous()), ("gate", gate_w.t().contiguous())):
        u, s, vh = torch.linalg.svd(mat, full_matrices=False)
        r = min(max_rank, s.numel())
        out[f"{name}_a"], out[f"{name}_b"] = u[:, :r] * s[:r], vh[:r, :]
    return out


def cluster_features_and_scores(normed: torch.Tensor, factors: dict, wd_norm: torch.Tensor, rank: int,
                                score_mode: str) -> tuple[torch.Tensor, torch.Tensor]:
    """cli.py:3357-3389: selector features [q_up | q_gate] and per-neuron pool scores of every token."""
    flat = normed.reshape(-1, normed.shape[-1])
    rank = min(max(1, int(rank)), factors["up_a"].shape[1], factors["gate_a"].shape[1])
    q_up, q_gate = flat @ factors["up_a"][:, :rank], flat @ factors["gate_a"][:, :rank]
    up_hat, gate_hat = q_up @ factors["up_b"][:rank, :], q_gate @ factors["gate_b"][:rank, :]
    gact = F.silu(gate_hat)
    up_s, gate_s, prod_s = up_hat.abs() * wd_norm, gact.abs() * wd_norm, (up_hat * gact).abs() * wd_norm
    scores = {"sum": up_s + gate_s + prod_s, "upgate": up_s + gate_s, "product": prod_s}[score_mode]
    return torch.cat([q_up, q_gate], dim=-1), scores


def fit_cluster_centers(features: torch.Tensor, cluster_count: int, iters: int) -> tuple[torch.Tensor, torch.Tensor]:
    """cli.py:3297-3323: cosine k-means -- rows L2-normalised, centres initialised from rows at evenly spaced
    indices, `iters` rounds of (arg-max assignment, mean of members re-normalised; an empty cluster keeps its
    centre).  Assignment ties go to the lowest centre index."""
    n = features.shape[0]
    cluster_count = min(max(1, int(cluster_count)), max(1, n))
    x = F.normalize(features.float(), dim=-1)
    if cluster_count == 1 or n == 1:
        return torch.zeros(n, dtype=torch.long), F.normalize(x.mean(dim=0, keepdim=True), dim=-1)
    init_idx = torch.linspace(0, n - 1, steps=cluster_count).round().long()
    centers = x.index_select(0, init_idx).contiguous()
    assignments = torch.zeros(n, dtype=torch.long)
    for _ in range(max(1, int(iters))):
        assignments = argmax_lowest(x @ centers.t())
        new_centers = torch.zeros_like(centers)
        counts = torch.bincount(assignments, minlength=cluster_count).to(new_centers.dtype)
        new_centers.index_add_(0, assignments, x)
        nonempty = counts > 0
        new_centers[nonempty] = new_centers[nonempty] / counts[nonempty].unsqueeze(-1).clamp_min(1.0)
        new_centers[~nonempty] = centers[~nonempty]
        centers = F.normalize(new_centers, dim=-1)
    return assignments, centers


def aggregate_cluster_scores(scores: torch.Tensor, assignments: torch.Tensor, cluster_count: int, aggregation: str) -> torch.Tensor:
    """cli.py:3326-3351: per-cluster mean or max of the members' scores (zeros for an empty cluster)."""
    out = scores.new_zeros(cluster_count, scores.shape[-1])
    for c in range(cluster_count):
        mask = assignments == c
        if bool(mask.any()):
            out[c] = scores[mask].mean(dim=0) if aggregation == "mean" else scores[mask].amax(dim=0)
    return out


def build_cluster_pool_codebook(features: torch.Tensor, scores: torch.Tensor, cluster_count: int, candidate_m: int,
                                aggregation: str, iters: int) -> dict[str, torch.Tensor]:
    """cli.py:4741-4771 for one layer: centres from the calibration features, candidate ids = the `candidate_m` best
    neurons of every cluster by aggregated score (ties to the lowest index)."""
    assignments, centers = fit_cluster_centers(features, cluster_count, iters)
    agg = aggregate_cluster_scores(scores.float(), assignments, centers.shape[0], aggregation)
    ids = topk_lowest(agg, min(candidate_m, agg.shape[-1]))[1]
    return dict(centers=centers, candidate_ids=ids, assignments=assignments, aggregate=agg)


def active_union_ids(candidate_ids: torch.Tensor, hidden: int, cap: int | None = None) -> torch.Tensor:
    """cli.py:4914-4941: sorted union of all clusters' candidates; above `cap`, the `cap` best by a
    frequency-plus-rank score (rank weights 1 .. 1/M), ties to the lowest index."""
    ids = candidate_ids.long()
    full = torch.unique(ids.reshape(-1), sorted=True)
    if cap is None or int(cap) <= 0 or full.numel() <= int(cap):
        return full
    cap = min(int(cap), hidden)
    c, m = ids.shape
    weight = torch.linspace(1.0, 1.0 / max(m, 1), steps=m).unsqueeze(0).expand(c, m).reshape(-1)
    score = torch.zeros(hidden).index_add_(0, ids.reshape(-1), weight)
    return torch.sort(topk_lowest(score.unsqueeze(0), cap)[1][0]).values
