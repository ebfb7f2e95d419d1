"""The golden cases: model/training settings whose reference outputs are stored beside this file.
Kept free of any import of the reference so that the fixtures can be consumed where it is absent."""
from oracle import rte_oracle as O

GOLDEN_CASES = {
    # BASELINE config 1 (the reference's CPU-runnable case), audit probability 0.
    "c1_macro": dict(
        model=dict(vocab_size=2048, d_model=128, n_heads=4, d_ff=512, n_dense_layers=4, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=8,
                   active_head_groups=2, active_ffn_groups=2, recipe_count=5, macro_rank=32),
        train=dict(mode="recursive_macro", lr=1e-3, weight_decay=0.1, batch_size=8, seq_len=64, seed=0,
                   fixed_depth=4, audit_fixed_count_per_batch=None),
        steps=20,
    ),
    # small model with one audited sample per batch, gradient-corrected control variate + distillation terms
    "small_audit": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=2, ffn_banks=2, head_groups=4, ffn_groups=4,
                   active_head_groups=2, active_ffn_groups=1, recipe_count=6, macro_rank=8),
        train=dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=3,
                   fixed_depth=None, audit_fixed_count_per_batch=1, grad_clip_norm=1.0),
        steps=6,
    ),
    # router decides depth and recipe (no fixed depth), no audit, aux losses on
    "small_routed": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=2, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4,
                   active_head_groups=1, active_ffn_groups=2, recipe_count=4, macro_rank=8),
        train=dict(mode="recursive_macro", lr=2e-3, weight_decay=0.05, batch_size=6, seq_len=12, seed=5,
                   fixed_depth=None, audit_fixed_count_per_batch=None),
        steps=6,
    ),
    # vocabulary-shortlist head (recursive_macro_shortlist) with one audited sample per batch
    "small_shortlist": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4,
                   active_head_groups=1, active_ffn_groups=2, recipe_count=4, macro_rank=8, shortlist_clusters=8),
        train=dict(mode="recursive_macro_shortlist", lr=2e-3, weight_decay=0.05, batch_size=4, seq_len=12, seed=9,
                   fixed_depth=None, audit_fixed_count_per_batch=1),
        output=dict(mode="shortlist", num_clusters=8, shortlist_top_clusters=2, shortlist_max_tokens=16,
                    hard_negatives=4, random_negatives=4),
        steps=6,
    ),
    # macro consistency term (lambda_cons) + residual clip of the control variate, two audited samples
    "small_cons_clip": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4,
                   active_head_groups=2, active_ffn_groups=2, recipe_count=5, macro_rank=8),
        train=dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=6, seq_len=16, seed=23,
                   fixed_depth=None, audit_fixed_count_per_batch=3, audit_residual_clip=0.1, lambda_cons=0.05,
                   grad_clip_norm=1.0),
        steps=6,
    ),
    # audit without gradient correction: the exact subset only feeds metrics and the distillation terms
    "small_metric_only": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4,
                   active_head_groups=2, active_ffn_groups=2, recipe_count=5, macro_rank=8),
        train=dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=29,
                   fixed_depth=None, audit_fixed_count_per_batch=1, audit_mode="metric_only"),
        steps=6,
    ),
    # Bernoulli audit sampler: adaptive probability (entropy, last residual, coverage deficit), capped at 3 per batch
    "small_bernoulli": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4,
                   active_head_groups=2, active_ffn_groups=2, recipe_count=5, macro_rank=8),
        train=dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=8, seq_len=16, seed=31,
                   fixed_depth=None, audit_fixed_count_per_batch=None, audit_sampler="bernoulli", audit_p_min=0.2,
                   audit_p_max=0.7, audit_alpha=0.5, audit_beta=2.0, audit_gamma=0.3, audit_cap=3, grad_clip_norm=1.0),
        steps=5,        # (at step 6 a near-tied router decision of one sample flips between two fp32 implementations)
    ),
    # fixed-count sampler with the count schedule: the count halves after a step whose macro endpoint tracked the exact
    # one and doubles otherwise (thresholds chosen so that both happen within the case)
    "small_schedule": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4,
                   active_head_groups=2, active_ffn_groups=2, recipe_count=5, macro_rank=8),
        train=dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=8, seq_len=16, seed=37,
                   fixed_depth=None, audit_fixed_count_per_batch=2, grad_clip_norm=1.0, audit_schedule_enabled=True,
                   audit_schedule_min_count=1, audit_schedule_nll_gap_threshold=0.335,
                   audit_schedule_hidden_cosine_threshold=0.9, audit_schedule_residual_var_threshold=1.0,
                   audit_schedule_delta_rms_ratio_min=0.0, audit_schedule_delta_rms_ratio_max=10.0,
                   audit_schedule_require_negative_mse_slope=False, audit_schedule_require_negative_norm_slope=False),
        steps=8,
    ),
    # recursive_exact: every sample runs the banked recurrent core (two banks, router-chosen depth)
    "small_exact": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=2, ffn_banks=2, head_groups=4, ffn_groups=4,
                   active_head_groups=2, active_ffn_groups=1, recipe_count=6, macro_rank=8),
        train=dict(mode="recursive_exact", lr=2e-3, weight_decay=0.05, batch_size=4, seq_len=12, seed=13,
                   fixed_depth=None, audit_fixed_count_per_batch=None),
        steps=6,
    ),
    # recursive_exact with a fixed per-pass recipe schedule (every sample runs recipe schedule[t] in pass t)
    "small_exact_schedule": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4,
                   active_head_groups=2, active_ffn_groups=2, recipe_count=5, macro_rank=8),
        train=dict(mode="recursive_exact", lr=2e-3, weight_decay=0.05, batch_size=4, seq_len=12, seed=43,
                   fixed_depth=None, audit_fixed_count_per_batch=None, fixed_recipe_schedule=(1, 3, 0, 2)),
        steps=6,
    ),
    # recursive_exact on a model whose macro operator is a variant (hidden layer, gate, delta-to-h0 and depth-embedding
    # inputs, trainable update scale): the step never evaluates it, its parameters ride along untouched
    "small_exact_variant": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4,
                   active_head_groups=2, active_ffn_groups=2, recipe_count=5, macro_rank=8, macro_hidden_mult=2,
                   macro_use_gated_update=True, macro_include_delta_to_h0=True, macro_use_depth_embedding=True,
                   macro_update_scale_init=0.1),
        train=dict(mode="recursive_exact", lr=2e-3, weight_decay=0.05, batch_size=4, seq_len=12, seed=47,
                   fixed_depth=None, audit_fixed_count_per_batch=None),
        steps=4,
    ),
    # recursive_deferred_grouped_exact: ONE grouped block (three scheduled recipes summed per half) instead of passes
    "small_deferred": dict(
        model=dict(vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=3, n_prelude=1, n_coda=1,
                   t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4,
                   active_head_groups=2, active_ffn_groups=2, recipe_count=5, macro_rank=8),
        train=dict(mode="recursive_deferred_grouped_exact", lr=2e-3, weight_decay=0.05, batch_size=4, seq_len=12, seed=53,
                   fixed_depth=None, audit_fixed_count_per_batch=None, fixed_recipe_schedule=(1, 3, 2)),
        steps=6,
    ),
    "small_dense": dict(
        model=dict(topology="dense", vocab_size=96, d_model=32, n_heads=4, d_ff=64, n_dense_layers=2, n_prelude=1,
                   n_coda=1, t_max=4, depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=4,
                   ffn_groups=4, active_head_groups=1, active_ffn_groups=1, recipe_count=4, macro_rank=8),
        train=dict(mode="dense_exact", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=7),
        steps=6,
    ),
}



def oracle_cfgs(case: dict) -> tuple[O.ModelCfg, O.TrainCfg]:
    return O.ModelCfg(**case["model"]), O.TrainCfg(**case["train"])


def oracle_output_cfg(case: dict) -> "O.OutputCfg | None":
    return O.OutputCfg(**case["output"]) if "output" in case else None


def cluster_pool_inputs(seed: int = 21, tokens=(5, 40), d=64, f=128, rank=8, clusters=4, pool=64):
    """Seeded inputs of the static cluster-pool FFN golden case (shared by the generator and the tests)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*tokens, d, generator=g)
    wug = torch.randn(2 * f, d, generator=g) * 0.1
    wd = torch.randn(d, f, generator=g) * 0.1
    up_a = torch.randn(d, rank, generator=g) * 0.3
    gate_a = torch.randn(d, rank, generator=g) * 0.3
    centers = torch.nn.functional.normalize(torch.randn(clusters, 2 * rank, generator=g), dim=-1)
    candidate_ids = torch.stack([torch.randperm(f, generator=g)[:pool] for _ in range(clusters)])
    probe = torch.randn(*tokens, d, generator=g)
    return dict(x=x, wug=wug, wd=wd, up_a=up_a, gate_a=gate_a, centers=centers, candidate_ids=candidate_ids, probe=probe)


SVD_FFN = dict(d=32, f=64, rank=8, top_k=8, up_m=8, gate_m=8, product_m=8)


def svd_ffn_inputs(seed: int = 31, tokens=(3, 11)):
    """Seeded inputs of the SVD-factor sparse FFN golden case (factors drawn directly, no SVD refresh)."""
    import torch
    c = SVD_FFN
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, scale: torch.randn(*s, generator=g) * scale  # noqa: E731
    return dict(x=r(*tokens, c["d"], scale=1.0), w_up=r(c["f"], c["d"], scale=0.2), w_gate=r(c["f"], c["d"], scale=0.2),
                w_down=r(c["f"], c["d"], scale=0.2), up_a=r(c["d"], c["rank"], scale=0.3), up_b=r(c["rank"], c["f"], scale=0.3),
                gate_a=r(c["d"], c["rank"], scale=0.3), gate_b=r(c["rank"], c["f"], scale=0.3), probe=r(*tokens, c["d"], scale=1.0))


# macro consistency term (reference macro.py:342-359) with weights large enough for the term to matter
MACRO_CONS = dict(d=32, rank=8, recipes=4, depth_choices=(1, 2, 4, 8), batch=5, seq=12, update_scale=0.05)


def macro_cons_inputs() -> dict:
    import torch
    c = MACRO_CONS
    g = torch.Generator().manual_seed(91)
    R, K, d, m = c["recipes"], len(c["depth_choices"]), c["d"], c["rank"]
    params = {"macro.d_gain": torch.randn(R, K, d, generator=g) * 0.3, "macro.v": torch.randn(R, K, 3 * d, m, generator=g) * 0.2,
              "macro.u": torch.randn(R, K, m, d, generator=g) * 0.5, "macro.bias": torch.randn(R, K, d, generator=g) * 0.2}
    return dict(params=params, h0=torch.randn(c["batch"], c["seq"], d, generator=g),
                recipe_ids=torch.randint(0, R, (c["batch"],), generator=g))


# offline cluster-pool codebook build (reference cli.py:3244-3389, 4741-4771): seeded inputs of one layer
CODEBOOK = dict(d=64, f=256, rank=16, tokens=320, clusters=6, candidate_m=64, iters=5)


def codebook_inputs() -> dict:
    """Well-separated synthetic calibration data: tokens drawn around `clusters` prototype directions, so that the
    k-means assignments do not hinge on near-ties."""
    import torch
    c = CODEBOOK
    g = torch.Generator().manual_seed(77)
    wug = torch.randn(2 * c["f"], c["d"], generator=g) * 0.3
    wd = torch.randn(c["d"], c["f"], generator=g) * 0.3
    protos = torch.randn(c["clusters"], c["d"], generator=g) * 2.0
    which = torch.randint(0, c["clusters"], (c["tokens"],), generator=g)
    normed = protos[which] + 0.25 * torch.randn(c["tokens"], c["d"], generator=g)
    return dict(wug=wug, wd=wd, normed=normed)
