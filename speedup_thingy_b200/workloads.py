"""The benchmark configurations of the `recursive_macro` training step, expressed in the reference's
config schema (src/recursive_training_engine/config.py:11-81, 85-346).

Each entry is the nearest configuration the reference can express for one named workload; fields the
workload description leaves open (bank counts, head groups, macro rank, recipe count) are fixed here and
used identically by the benchmark, the parity tests and the CPU baseline.

    c1  CPU-runnable recursive_macro: d128, 4 heads, F512 (8 slabs of 64, 2 active), depth 4, batch 8 x 64, no audit
    c2  dense_exact: 4 layers, d512, 8 heads, F2048, batch 128 x 64
    c3  recursive_macro: d512, 8 heads, F2048 (16 slabs of 128, 4 active), depth 4, batch 128 x 64,
        one audited sample per batch (p = 1/128), gradient-corrected control variate
    c4  recursive_macro_shortlist: d512, F2048, depth 8, batch 128 x 128, two audited samples (p = 1/64),
        vocabulary shortlist head
    c5  data-parallel scale-up, per rank: d1024, 16 heads, F4096 (32 slabs of 128, 8 active), depth 16,
        vocabulary 32768, batch 32 x 256, no audit
"""
from __future__ import annotations

from .config import ExperimentConfig, ModelConfig, OutputConfig, TrainingConfig

WORKLOADS: dict[str, dict] = {
    "c1": dict(
        title="BASELINE configs[0]: recursive_macro depth 4, d128 H4 F512 (8x64 slabs, 2 active) V2048, batch 8x64, no audit",
        model=dict(vocab_size=2048, d_model=128, n_heads=4, d_ff=512, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
                   attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=8, active_head_groups=2, active_ffn_groups=2,
                   recipe_count=5, macro_rank=32, n_dense_layers=4),
        train=dict(mode="recursive_macro", lr=1e-3, weight_decay=0.1, batch_size=8, seq_len=64, seed=0, fixed_depth=4)),
    "c2": dict(
        title="BASELINE configs[1]: dense_exact 4 layers, d512 H8 F2048 V2048, batch 128x64",
        model=dict(topology="dense", vocab_size=2048, d_model=512, n_heads=8, d_ff=2048, n_dense_layers=4),
        train=dict(mode="dense_exact", lr=1e-3, weight_decay=0.1, batch_size=128, seq_len=64, seed=0)),
    "c3": dict(
        title="BASELINE configs[2]: recursive_macro depth 4, d512 H8 F2048 (16x128 slabs, 4 active) V2048, batch 128x64, audit 1/128",
        model=dict(vocab_size=2048, d_model=512, n_heads=8, d_ff=2048, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
                   attn_banks=1, ffn_banks=1, head_groups=8, ffn_groups=16, active_head_groups=2, active_ffn_groups=4,
                   recipe_count=5, macro_rank=32),
        train=dict(mode="recursive_macro", lr=1e-3, weight_decay=0.1, batch_size=128, seq_len=64, seed=0, fixed_depth=4,
                   audit_fixed_count_per_batch=1)),
    "c4": dict(
        title="BASELINE configs[3]: recursive_macro_shortlist depth 8, d512 H8 F2048 V2048, batch 128x128, audit 2/128, "
              "shortlist head (64 clusters, top 2, 128 tokens)",
        model=dict(vocab_size=2048, d_model=512, n_heads=8, d_ff=2048, n_prelude=1, n_coda=1, t_max=8, depth_choices=(1, 2, 4, 8),
                   attn_banks=1, ffn_banks=1, head_groups=8, ffn_groups=16, active_head_groups=2, active_ffn_groups=4,
                   recipe_count=5, macro_rank=32),
        train=dict(mode="recursive_macro_shortlist", lr=1e-3, weight_decay=0.1, batch_size=128, seq_len=128, seed=0,
                   fixed_depth=8, audit_fixed_count_per_batch=2),
        output=dict(mode="shortlist", num_clusters=64, shortlist_top_clusters=2, shortlist_max_tokens=128, hard_negatives=32,
                    random_negatives=32)),
    "c5": dict(
        title="BASELINE configs[4] per rank: recursive_macro depth 16, d1024 H16 F4096 (32x128 slabs, 8 active) V32768, "
              "batch 32x256, no audit",
        model=dict(vocab_size=32768, d_model=1024, n_heads=16, d_ff=4096, n_prelude=1, n_coda=1, t_max=16,
                   depth_choices=(1, 2, 4, 8, 16), attn_banks=1, ffn_banks=1, head_groups=16, ffn_groups=32,
                   active_head_groups=4, active_ffn_groups=8, recipe_count=5, macro_rank=32),
        train=dict(mode="recursive_macro", lr=1e-3, weight_decay=0.1, batch_size=32, seq_len=256, seed=0, fixed_depth=16)),
}


def workload(name: str, **train_overrides) -> tuple[ExperimentConfig, dict]:
    """(ExperimentConfig, raw dicts) of a named workload; keyword arguments override training fields
    (a smaller batch for a parity test, another seed for another rank)."""
    w = WORKLOADS[name]
    train = {**w["train"], **train_overrides}
    cfg = ExperimentConfig(ModelConfig(**w["model"]), TrainingConfig(**train), OutputConfig(**w.get("output", {})))
    return cfg, dict(title=w["title"], model=dict(w["model"]), train=train, output=dict(w.get("output", {})))


def train_flops_per_token(cfg: ExperimentConfig) -> float:
    """Algorithmic training FLOPs per token of the hot step: 3 x forward, forward = blocks * (8 d^2 + 6 d F + 4 S d)
    + 8 d m (macro operator, recursive topology) + 2 d V (logits; the shortlist head scores K rows instead of V)."""
    m, tr = cfg.model, cfg.training
    d, f, s = m.d_model, m.d_ff, tr.seq_len
    block = 8 * d * d + 6 * d * f + 4 * s * d
    if m.topology == "dense":
        return 3.0 * (m.n_dense_layers * block + 2 * d * m.vocab_size)
    out_rows = cfg.output.shortlist_max_tokens + cfg.output.num_clusters if tr.mode == "recursive_macro_shortlist" else m.vocab_size
    return 3.0 * ((m.n_prelude + m.n_coda) * block + 8 * d * m.macro_rank + 2 * d * out_rows)
