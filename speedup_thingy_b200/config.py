"""Configuration of the accelerated training step.

The dataclasses carry the reference's complete ``model:`` / ``training:`` / ``output:`` / ``data:`` schema
(src/recursive_training_engine/config.py:11-81, 85-336, 340-379, 406-449) with the same field names, defaults
and structural validation, so every reference YAML parses unchanged.  Keys that cannot change the step's
arithmetic (compile flags, optimizer implementation flags, TF32, logging, data source) are kept and ignored.
Values the sm_100a path does not implement are NOT rejected while parsing: ``unsupported(config)`` lists them,
and ``TrainEngine`` (or ``load_config(..., check=True)``) raises ``NotImplementedError`` naming each one.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any

SUPPORTED_MODES = ("recursive_macro", "recursive_macro_shortlist", "recursive_exact", "recursive_deferred_grouped_exact",
                   "dense_exact")
EXACT_MODES = ("recursive_exact", "recursive_deferred_grouped_exact")        # modes that never evaluate the macro operator
REFERENCE_MODES = ("dense_exact", "recursive_exact", "recursive_deferred_grouped_exact", "recursive_exact_route_em",
                   "recursive_exact_factorized_soft", "recursive_exact_dense_hidden_distill", "recursive_sandwich_supernet",
                   "recursive_macro", "recursive_macro_shortlist", "recursive_macro_distill_only",
                   "recursive_macro_lm_aligned", "recursive_macro_shadow_coda")


@dataclass
class ModelConfig:
    topology: str = "recursive"
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
    tie_embeddings: bool = True
    use_rope: bool = True
    use_recursive_input_skip: bool = True
    use_global_lowrank_corrector: bool = False
    global_corrector_rank: int = 16
    fairness_tolerance: float = 0.01
    macro_type: str = "bounded_residual"
    macro_rank: int = 32
    macro_update_scale: float = 0.05
    macro_hidden_mult: int = 1
    macro_use_gated_update: bool = False
    macro_update_scale_init: float = 1.0
    macro_include_delta_to_h0: bool = False
    macro_use_delta_to_h0: bool = False
    macro_use_depth_embedding: bool = False
    macro_use_recipe_embedding: bool = False
    macro_radius_init_from_teacher: bool = False
    macro_radius_clamp_mult_min: float = 0.25
    macro_radius_clamp_mult_max: float = 4.0
    macro_decomposition: str = "direct"
    router_hidden: int | None = None

    def __post_init__(self) -> None:
        self.depth_choices = tuple(self.depth_choices)
        if self.topology not in ("recursive", "dense"):
            raise ValueError("topology must be 'recursive' or 'dense'")
        if self.d_model % self.n_heads:
            raise ValueError("d_model must be divisible by n_heads")
        if self.n_heads % self.head_groups:
            raise ValueError("n_heads must be divisible by head_groups")
        if self.d_ff % self.ffn_groups:
            raise ValueError("d_ff must be divisible by ffn_groups")
        if not 1 <= self.active_head_groups <= self.head_groups:
            raise ValueError("active_head_groups must be in [1, head_groups]")
        if not 1 <= self.active_ffn_groups <= self.ffn_groups:
            raise ValueError("active_ffn_groups must be in [1, ffn_groups]")
        if self.t_max not in self.depth_choices:
            raise ValueError("t_max must be present in depth_choices")
        if sorted(self.depth_choices) != list(self.depth_choices):
            raise ValueError("depth_choices must be sorted ascending")
        if self.recipe_count < 2:
            raise ValueError("recipe_count must include sparse recipes plus dense fallback")
        if self.macro_rank < 1:
            raise ValueError("macro_rank must be positive")
        if self.macro_hidden_mult < 1:
            raise ValueError("macro_hidden_mult must be positive")

    @property
    def router_hidden_dim(self) -> int:
        return self.router_hidden or max(32, self.d_model)

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads


@dataclass
class TrainingConfig:
    mode: str = "recursive_macro"
    loss_normalization: str = "token_mean"
    optimizer: str = "adamw"
    lr: float = 3e-4
    lr_base: float | None = None
    lr_macro: float | None = None
    lr_coda: float | None = None
    lr_output: float | None = None
    lr_router: float | None = None
    lr_schedule: str = "constant"
    lr_decay_start_tokens: int | None = None
    lr_decay_end_tokens: int | None = None
    lr_final_scale: float = 1.0
    weight_decay: float = 0.1
    batch_size: int = 4
    seq_len: int = 32
    grad_accum_steps: int = 1
    grad_clip_norm: float | None = None
    seed: int = 1337
    # the reference's default is "fp32" (autocast off); this path computes in bf16 with fp32 master weights and says
    # so through `unsupported` when a configuration asks for fp32
    precision: str = "bf16"
    audit_p_min: float = 0.0
    audit_p_max: float = 0.0
    audit_alpha: float = 0.08
    audit_beta: float = 0.08
    audit_gamma: float = 0.08
    audit_sampler: str = "bernoulli"
    audit_fixed_count: int | None = None
    audit_cap: int | None = None
    audit_fixed_count_per_batch: int | None = None
    audit_mode: str = "gradient_corrected"
    audit_residual_clip: float | None = None
    audit_gradient_correction: bool = True
    audit_schedule_enabled: bool = False
    audit_schedule_min_count: int | None = None
    audit_schedule_gap_threshold: float = 0.05
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
    target_speedup_vs_dense: float | None = None
    max_active_param_equiv_per_token: float | None = None
    max_hotpath_flops_per_token: float | None = None
    lambda_depth: float = 1e-4
    lambda_load: float = 1e-2
    lambda_cover: float = 1e-2
    lambda_router: float = 1.0
    lambda_hid: float = 1e-2
    lambda_cos: float = 1e-2
    lambda_kl: float = 1e-2
    lambda_hidden_mse: float | None = None
    lambda_hidden_cosine: float | None = None
    lambda_logit_kl: float | None = None
    lambda_dense_hidden: float = 1.0
    lambda_dense_delta: float = 0.5
    lambda_dense_kl: float = 0.25
    lambda_norm: float = 0.05
    lambda_delta_dir: float = 2.0
    lambda_delta_rms: float = 2.0
    lambda_endpoint_normed: float = 1.0
    lambda_endpoint_raw: float = 0.05
    macro_rms_trust_region: bool = False
    macro_rms_clamp_early: bool = False
    macro_rms_clamp_min: float = 0.5
    macro_rms_clamp_max: float = 2.0
    lambda_macro_rms_trust: float = 2.0
    distill_temperature: float = 2.0
    dense_distill_temperature: float = 2.0
    dense_hidden_layer_map: list | None = None
    # the reference's default is 1e-3; the consistency term (macro.py:342-359) is not on this path, so the default
    # here is 0 and a non-zero value is reported by `unsupported`
    lambda_cons: float = 0.0
    coverage_min: float = 0.01
    coverage_beta: float = 0.98
    fixed_recipe: int | None = None
    fixed_recipe_schedule: list | None = None
    fixed_depth: int | None = None
    route_em_candidates: int = 4
    route_em_allow_dense_fallback: bool = False
    route_em_proposal: str = "router"
    factorized_route_top_k: int = 4
    factorized_route_temperature: float = 1.0
    sandwich_random_paths: int = 2
    sandwich_temperature: float = 2.0
    lambda_sandwich_rand_ce: float = 0.5
    lambda_sandwich_kd: float = 1.0
    lambda_sandwich_rand_kd: float = 0.5
    lambda_sandwich_hidden: float = 0.1
    disable_router_aux: bool = False
    debug_force_full_output: bool = False
    coda_warmup_steps: int = 0
    aligned_lm_teacher_checkpoint: str | None = None
    aligned_lm_freeze_teacher: bool = True
    aligned_lm_phase_a_train: list = field(default_factory=lambda: ["macro"])
    aligned_lm_phase_b_train: list = field(default_factory=lambda: ["macro", "coda"])
    aligned_lm_phase_c_train: list = field(default_factory=lambda: ["macro", "coda", "output"])
    unfreeze_prelude_core_after_gate: bool = True
    log_every: int = 1
    compile_model: bool = False
    compile_mode: str = "reduce-overhead"
    fused_optimizer: bool = True
    foreach_optimizer: bool = True
    allow_tf32: bool = True
    strict_cuda: bool = True
    require_triton: bool = False
    require_flash_attention: bool = True

    def __post_init__(self) -> None:
        if self.mode not in REFERENCE_MODES:
            raise ValueError(f"unknown training mode {self.mode!r}")
        if self.audit_fixed_count is not None:          # config.py:216-221
            self.audit_fixed_count_per_batch = self.audit_fixed_count
        if self.audit_sampler == "fixed_count" and self.audit_fixed_count_per_batch is None:
            raise ValueError("audit_sampler='fixed_count' requires audit_fixed_count")
        if self.audit_fixed_count_per_batch is not None:
            self.audit_sampler = "fixed_count"
        if self.grad_accum_steps < 1:
            raise ValueError("grad_accum_steps must be >= 1")
        if self.lr_final_scale <= 0:
            raise ValueError("lr_final_scale must be positive")
        if self.lr_schedule not in ("constant", "linear_decay_after"):
            raise ValueError(f"unknown lr_schedule {self.lr_schedule!r}")
        if self.lr_schedule == "linear_decay_after":
            if self.lr_decay_start_tokens is None or self.lr_decay_end_tokens is None:
                raise ValueError("linear_decay_after requires lr_decay_start_tokens and lr_decay_end_tokens")
            if self.lr_decay_end_tokens <= self.lr_decay_start_tokens:
                raise ValueError("lr_decay_end_tokens must be greater than lr_decay_start_tokens")
        if self.audit_cap is not None and self.audit_cap < 0:
            raise ValueError("audit_cap must be non-negative when provided")
        if self.audit_fixed_count_per_batch is not None:
            if self.audit_fixed_count_per_batch < 0:
                raise ValueError("audit_fixed_count_per_batch must be non-negative when provided")
            if self.audit_fixed_count_per_batch > self.batch_size:
                raise ValueError("audit_fixed_count_per_batch must be <= batch_size")
        if self.distill_temperature <= 0:
            raise ValueError("distill_temperature must be positive")
        if self.audit_mode == "gradient_corrected" and not self.audit_gradient_correction and self.audit_p_max > 0:
            raise ValueError("audit_mode='gradient_corrected' requires audit_gradient_correction=true "
                             "when audits are enabled")             # config.py:255-263
        for name in ("target_speedup_vs_dense", "max_active_param_equiv_per_token", "max_hotpath_flops_per_token"):
            if getattr(self, name) is not None and getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")

    def lr_for(self, group: str) -> float:
        """Per-group learning rates (reference training.py:302-339)."""
        override = {"embedding": self.lr_base, "prelude": self.lr_base, "core": self.lr_base, "dense": self.lr_base,
                    "macro": self.lr_macro, "coda": self.lr_coda, "output": self.lr_output, "router": self.lr_router}[group]
        return self.lr if override is None else override

    def lr_scale(self, tokens_seen: int) -> float:
        """training.py:470-483: the factor every group's base learning rate is multiplied with at `tokens_seen`."""
        if self.lr_schedule == "constant":
            return 1.0
        if tokens_seen <= self.lr_decay_start_tokens:
            return 1.0
        if tokens_seen >= self.lr_decay_end_tokens:
            return self.lr_final_scale
        progress = (tokens_seen - self.lr_decay_start_tokens) / (self.lr_decay_end_tokens - self.lr_decay_start_tokens)
        return 1.0 + progress * (self.lr_final_scale - 1.0)

    @property
    def audits_enabled(self) -> bool:
        """Whether any sample can be audited: a fixed count > 0, or a Bernoulli sampler with a non-zero ceiling and a
        non-zero cap (audit.py:79-132)."""
        if self.audit_fixed_count_per_batch is not None:
            return self.audit_fixed_count_per_batch > 0
        return self.audit_p_max > 0 and self.audit_cap != 0


@dataclass
class OutputConfig:
    """Vocabulary-shortlist head settings (reference config.py:340-346)."""
    mode: str = "full"
    num_clusters: int = 64
    shortlist_top_clusters: int = 2
    shortlist_max_tokens: int = 128
    hard_negatives: int = 32
    random_negatives: int = 32

    def __post_init__(self) -> None:
        if self.mode not in ("full", "shortlist"):
            raise ValueError("output.mode must be 'full' or 'shortlist'")


@dataclass
class DataConfig:
    """Data source settings (reference config.py:349-372).  Parsed for completeness; the step takes token batches."""
    dataset: str = "synthetic"
    tokenizer: str = "gpt2_bpe"
    vocab_projection: str = "filter"
    projection_lane: str | None = None
    cache_dir: str = ".cache/rte"
    local_text_path: str | None = None
    train_split: str = "train"
    eval_split: str = "validation"
    seed: int | None = None
    train_tokens: int | None = None
    max_tokens: int = 200_000
    eval_tokens: int = 20_000
    synthetic_tokens: int = 20_000

    def __post_init__(self) -> None:
        if self.projection_lane is None:
            self.projection_lane = self.vocab_projection
        elif self.projection_lane != self.vocab_projection:
            raise ValueError("data.projection_lane and data.vocab_projection must match")
        if self.train_tokens is not None:
            self.max_tokens = self.train_tokens


@dataclass
class ExperimentConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    output: OutputConfig = field(default_factory=OutputConfig)
    data: DataConfig = field(default_factory=DataConfig)
    run_name: str = "rte-run"
    output_dir: str = "runs"
    allow_unknown_config_keys: bool = False


def unsupported(config: ExperimentConfig) -> list[str]:
    """Every configured VALUE the sm_100a path does not implement, as 'section.key=value: why' strings (empty when
    the configuration can run).  Keys without influence on the arithmetic are never listed."""
    m, t = config.model, config.training
    out: list[str] = []

    def no(section: str, key: str, why: str) -> None:
        out.append(f"{section}.{key}={getattr(getattr(config, section), key)!r}: {why}")

    if t.mode not in SUPPORTED_MODES:
        no("training", "mode", "implemented modes are " + ", ".join(SUPPORTED_MODES))
    # kernel size limits (what TrainEngine would otherwise refuse at construction)
    head_dim = m.d_model // max(m.n_heads, 1)
    if m.d_model % 8:
        no("model", "d_model", "kernel limit: a multiple of 8")
    if head_dim not in (8, 16, 32, 64, 128):
        no("model", "n_heads", f"kernel limit: head_dim = d_model / n_heads in {{8, 16, 32, 64, 128}}, not {head_dim}")
    if m.d_ff % 64:
        no("model", "d_ff", "kernel limit: a multiple of 64")
    if m.vocab_size % 8:
        no("model", "vocab_size", "kernel limit: a multiple of 8")
    if t.seq_len > 256:
        no("training", "seq_len", "kernel limit: at most 256")
    if m.topology == "recursive":
        if m.recipe_count > 32:
            no("model", "recipe_count", "kernel limit: at most 32")
        if len(m.depth_choices) > 8:
            no("model", "depth_choices", "kernel limit: at most 8 depth choices")
        if m.t_max > 128:
            no("model", "t_max", "kernel limit: at most 128 passes")
        if m.macro_rank > 64:
            no("model", "macro_rank", "kernel limit: at most 64")
    if t.precision != "bf16":
        no("training", "precision", "the kernels compute in bf16 with fp32 master weights and accumulation; "
                                    "pass precision='bf16' to load_config to run this configuration that way")
    if t.loss_normalization != "token_mean":
        no("training", "loss_normalization", "only token_mean")
    for key, want in (("tie_embeddings", True), ("use_rope", True), ("use_recursive_input_skip", True),
                      ("use_global_lowrank_corrector", False), ("macro_type", "bounded_residual"),
                      ("macro_hidden_mult", 1), ("macro_use_gated_update", False), ("macro_include_delta_to_h0", False),
                      ("macro_use_delta_to_h0", False), ("macro_use_depth_embedding", False),
                      ("macro_use_recipe_embedding", False), ("macro_decomposition", "direct")):
        # (mode recursive_exact never evaluates the macro operator: its variants then only add parameters the step
        #  carries untouched -- no influence on the arithmetic)
        inert = key.startswith("macro_") and t.mode in EXACT_MODES
        if m.topology == "recursive" and getattr(m, key) != want and not inert:
            no("model", key, f"only {want!r} (the 3d -> rank -> d bounded-residual macro operator, macro.py:201-236)")
    if m.topology == "dense" and not m.tie_embeddings:
        no("model", "tie_embeddings", "only tied input / output embeddings")
    recursive = t.mode in ("recursive_macro", "recursive_macro_shortlist")
    if recursive and t.audits_enabled:
        if t.audit_mode not in ("gradient_corrected", "metric_only", "distill_only"):
            no("training", "audit_mode", "one of gradient_corrected, metric_only, distill_only")
        if t.macro_rms_trust_region or t.macro_rms_clamp_early:
            no("training", "macro_rms_trust_region", "the RMS trust region is not implemented")
    if t.fixed_recipe_schedule is not None and t.mode not in EXACT_MODES:
        no("training", "fixed_recipe_schedule", "per-pass fixed recipes are implemented for the exact modes only")
    if t.mode == "recursive_deferred_grouped_exact" and (m.attn_banks != 1 or m.ffn_banks != 1):
        no("model", "attn_banks" if m.attn_banks != 1 else "ffn_banks", "the grouped block is implemented for one bank each")
    # (coda_warmup_steps only gates the phases of mode recursive_macro_lm_aligned, training.py:262-277: no influence here)
    if t.debug_force_full_output and t.mode == "recursive_macro_shortlist":
        no("training", "debug_force_full_output", "not implemented for the shortlist mode")
    if (t.mode == "recursive_macro_shortlist") != (config.output.mode == "shortlist") and t.mode in SUPPORTED_MODES:
        if t.mode == "recursive_macro_shortlist":
            no("output", "mode", "recursive_macro_shortlist needs output.mode='shortlist'")
    return out


def check_supported(config: ExperimentConfig) -> None:
    problems = unsupported(config)
    if problems:
        raise NotImplementedError("rte_b200 does not implement: " + "; ".join(problems))


def _build(cls, data: dict[str, Any], path: str, allow_unknown: bool):
    valid = {f.name for f in fields(cls)}
    unknown = sorted(set(data) - valid)
    if unknown and not allow_unknown:
        raise ValueError("unknown config key(s): " + ", ".join(f"{path}.{k}" for k in unknown))
    return cls(**{k: v for k, v in data.items() if k in valid})


def load_config(path: str | Path, *, check: bool = False, precision: str | None = None) -> ExperimentConfig:
    """Reads a reference-style YAML (config.py:406-449): same sections, same keys, same defaults except where a
    docstring above says otherwise (`precision`, `lambda_cons`, `audit_p_min/max`).  Sections present in the file fall
    back to the REFERENCE's defaults for keys they omit, so a file means here what it means there.
    `precision='bf16'` overrides the file's precision (the reference's presets say fp32; this path computes in bf16).
    `check=True` raises NotImplementedError for values the path does not implement (see `unsupported`)."""
    import yaml

    raw = yaml.safe_load(Path(path).read_text()) or {}
    allow_unknown = bool(raw.get("allow_unknown_config_keys", False))
    root_valid = {"model", "training", "output", "data", "run_name", "output_dir", "allow_unknown_config_keys"}
    root_unknown = sorted(set(raw) - root_valid)
    if root_unknown and not allow_unknown:
        raise ValueError("unknown config key(s): " + ", ".join(root_unknown))
    training = dict(raw.get("training", {}))
    # the reference's defaults where this module's differ (a YAML that omits the key means the reference's value)
    for key, ref_default in (("precision", "fp32"), ("lambda_cons", 1e-3), ("audit_p_min", 0.05), ("audit_p_max", 0.25),
                             ("strict_cuda", False)):
        training.setdefault(key, ref_default)
    if precision is not None:
        training["precision"] = precision
    cfg = ExperimentConfig(model=_build(ModelConfig, raw.get("model", {}), "model", allow_unknown),
                           training=_build(TrainingConfig, training, "training", allow_unknown),
                           output=_build(OutputConfig, raw.get("output", {}), "output", allow_unknown),
                           data=_build(DataConfig, raw.get("data", {}), "data", allow_unknown),
                           run_name=raw.get("run_name", "rte-run"), output_dir=raw.get("output_dir", "runs"),
                           allow_unknown_config_keys=allow_unknown)
    if check:
        check_supported(cfg)
    return cfg
