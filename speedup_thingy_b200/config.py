"""Configuration of the accelerated training step.

Field names and meanings follow the reference's ``ModelConfig`` / ``TrainingConfig``
(src/recursive_training_engine/config.py:11-81, 85-336) for the subset the `recursive_macro` and
`dense_exact` steps read, so a reference YAML's ``model:`` / ``training:`` blocks load unchanged;
keys the accelerated path does not implement are rejected rather than ignored.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any


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
    macro_type: str = "bounded_residual"
    macro_rank: int = 32
    macro_update_scale: float = 0.05
    macro_decomposition: str = "direct"
    router_hidden: int | None = None
    fairness_tolerance: float = 0.01

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
        if self.t_max not in self.depth_choices:
            raise ValueError("t_max must be present in depth_choices")
        if sorted(self.depth_choices) != list(self.depth_choices):
            raise ValueError("depth_choices must be sorted ascending")
        if self.recipe_count < 2:
            raise ValueError("recipe_count must include sparse recipes plus dense fallback")
        for flag, want in (("tie_embeddings", True), ("use_rope", True), ("use_recursive_input_skip", True),
                           ("macro_type", "bounded_residual"), ("macro_decomposition", "direct")):
            if getattr(self, flag) != want:
                raise NotImplementedError(f"rte_b200 implements {flag}={want!r} only")

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
    lr: float = 3e-4
    lr_base: float | None = None
    lr_macro: float | None = None
    lr_coda: float | None = None
    lr_output: float | None = None
    lr_router: float | None = None
    weight_decay: float = 0.1
    batch_size: int = 4
    seq_len: int = 32
    grad_clip_norm: float | None = None
    seed: int = 1337
    precision: str = "bf16"
    audit_fixed_count_per_batch: int | None = None
    audit_mode: str = "gradient_corrected"
    audit_residual_clip: float | None = None
    lambda_depth: float = 1e-4
    lambda_load: float = 1e-2
    lambda_cover: float = 1e-2
    lambda_kl: float = 1e-2
    lambda_delta_dir: float = 2.0
    lambda_delta_rms: float = 2.0
    lambda_endpoint_normed: float = 1.0
    lambda_endpoint_raw: float = 0.05
    distill_temperature: float = 2.0
    coverage_min: float = 0.01
    coverage_beta: float = 0.98
    fixed_recipe: int | None = None
    fixed_depth: int | None = None
    disable_router_aux: bool = False
    strict_cuda: bool = True
    target_speedup_vs_dense: float | None = None
    max_active_param_equiv_per_token: float | None = None
    max_hotpath_flops_per_token: float | None = None

    def __post_init__(self) -> None:
        if self.mode not in ("recursive_macro", "recursive_macro_shortlist", "recursive_exact", "dense_exact"):
            raise NotImplementedError("rte_b200 implements modes recursive_macro, recursive_macro_shortlist, "
                                      f"recursive_exact and dense_exact, not {self.mode!r}")
        if self.loss_normalization != "token_mean":
            raise NotImplementedError("only loss_normalization='token_mean'")
        if self.precision != "bf16":
            raise NotImplementedError("the sm_100a path computes in bf16 with fp32 master weights (precision='bf16')")
        if self.audit_fixed_count_per_batch is not None and self.audit_fixed_count_per_batch > self.batch_size:
            raise ValueError("audit_fixed_count_per_batch must be <= batch_size")
        for name in ("target_speedup_vs_dense", "max_active_param_equiv_per_token", "max_hotpath_flops_per_token"):
            if getattr(self, name) is not None and getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")

    def lr_for(self, group: str) -> float:
        """Per-group learning rates (reference training.py:302-339)."""
        override = {"embedding": self.lr_base, "prelude": self.lr_base, "core": self.lr_base, "dense": self.lr_base,
                    "macro": self.lr_macro, "coda": self.lr_coda, "output": self.lr_output, "router": self.lr_router}[group]
        return self.lr if override is None else override


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
class ExperimentConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    output: OutputConfig = field(default_factory=OutputConfig)


def _build(cls, data: dict[str, Any], path: str):
    valid = {f.name for f in fields(cls)}
    unknown = sorted(set(data) - valid)
    if unknown:
        raise ValueError("unknown or unsupported config key(s): " + ", ".join(f"{path}.{k}" for k in unknown))
    return cls(**data)


def load_config(path: str | Path) -> ExperimentConfig:
    """Reads the ``model`` and ``training`` blocks of a reference-style YAML (config.py:406-449)."""
    import yaml

    raw = yaml.safe_load(Path(path).read_text()) or {}
    return ExperimentConfig(model=_build(ModelConfig, raw.get("model", {}), "model"),
                            training=_build(TrainingConfig, raw.get("training", {}), "training"),
                            output=_build(OutputConfig, raw.get("output", {}), "output"))
