"""Host-side logic of the engine (hand-written backward sequencing, buffer reuse, optimiser plan)
checked against the CPU oracle with the test-only operator emulation (tests/emul_ops.py)."""
import numpy as np
import pytest
import torch

from oracle import rte_oracle as O
from speedup_thingy_b200.config import ExperimentConfig, ModelConfig, OutputConfig, TrainingConfig
from speedup_thingy_b200.engine import TrainEngine, init_parameters, parameter_shapes
from tests.emul_ops import EmulOps

CASES = {
    "macro_fixed_depth": (
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8),
        dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=3, fixed_depth=4)),
    "macro_routed_clip": (
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=2, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=1, active_ffn_groups=2,
             recipe_count=4, macro_rank=8),
        dict(mode="recursive_macro", lr=2e-3, weight_decay=0.05, batch_size=6, seq_len=12, seed=5, fixed_depth=None,
             grad_clip_norm=0.5)),
    "macro_audit_two_banks": (
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=2, ffn_banks=2, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=1,
             recipe_count=6, macro_rank=8),
        dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=3, fixed_depth=None,
             audit_fixed_count_per_batch=2, grad_clip_norm=1.0)),
    "macro_audit_residual_clip": (        # clip chosen so that some audited residuals fall inside and some outside
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8),
        dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=6, seq_len=16, seed=13, fixed_depth=None,
             audit_fixed_count_per_batch=4, audit_residual_clip=0.15, grad_clip_norm=1.0)),
    "macro_audit_metric_only": (
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8),
        dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=17, fixed_depth=None,
             audit_fixed_count_per_batch=2, audit_mode="metric_only", audit_gradient_correction=False)),
    "macro_consistency": (                 # lambda_cons with four depth choices: stride pairs (1,2), (2,4), (4,8)
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=8, depth_choices=(1, 2, 4, 8),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8),
        dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=19, fixed_depth=None,
             audit_fixed_count_per_batch=1, lambda_cons=2000.0, grad_clip_norm=1.0)),
    "macro_bernoulli_cap": (               # Bernoulli sampler, adaptive probability, cap 3 of batch 8
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8),
        dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=8, seq_len=16, seed=31, fixed_depth=None,
             audit_fixed_count_per_batch=None, audit_sampler="bernoulli", audit_p_min=0.2, audit_p_max=0.7, audit_alpha=0.5,
             audit_beta=2.0, audit_gamma=0.3, audit_cap=3, grad_clip_norm=1.0)),
    "macro_bernoulli_nocap_clip": (        # no cap (capacity from p_max), residual clip on per-sample probabilities
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8),
        dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=8, seq_len=16, seed=37, fixed_depth=None,
             audit_fixed_count_per_batch=None, audit_sampler="bernoulli", audit_p_min=0.3, audit_p_max=0.6, audit_alpha=0.5,
             audit_beta=1.0, audit_gamma=0.3, audit_residual_clip=0.2,
             # (the log-ratio term of a near-zero macro delta turns Adam's first +-lr steps on noise-level gradients into
             #  per-cent loss differences between a bf16 and an fp32 run; the other cases carry these terms)
             lambda_delta_rms=0.0, lambda_delta_dir=0.0)),
    "macro_scheduled": (                   # fixed count 2 of 8 under the count schedule (capacity: the batch)
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8),
        dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=8, seq_len=16, seed=41, fixed_depth=None,
             audit_fixed_count_per_batch=2, grad_clip_norm=1.0, audit_schedule_enabled=True, audit_schedule_min_count=1,
             audit_schedule_nll_gap_threshold=0.3, audit_schedule_hidden_cosine_threshold=0.9,
             audit_schedule_delta_rms_ratio_min=0.0, audit_schedule_delta_rms_ratio_max=10.0,
             audit_schedule_require_negative_mse_slope=False, audit_schedule_require_negative_norm_slope=False)),
    "preset_small": (                      # the dimensions and settings of the reference's configs/small.yaml
        dict(vocab_size=512, d_model=32, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=64,
             depth_choices=(1, 2, 4, 8, 16, 32, 64), attn_banks=2, ffn_banks=1, head_groups=4, ffn_groups=16,
             active_head_groups=2, active_ffn_groups=2, recipe_count=8, macro_rank=8),
        dict(mode="recursive_macro_shortlist", lr=3e-4, weight_decay=0.05, batch_size=4, seq_len=32, seed=1337,
             fixed_depth=None, audit_fixed_count_per_batch=None, audit_sampler="bernoulli", audit_p_min=0.05,
             audit_p_max=0.25, lambda_cons=1e-3),
        dict(mode="shortlist", num_clusters=32, shortlist_top_clusters=2, shortlist_max_tokens=64, hard_negatives=16,
             random_negatives=16)),
    "macro_shortlist": (
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8),
        dict(mode="recursive_macro_shortlist", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=9,
             fixed_depth=None, audit_fixed_count_per_batch=1),
        dict(mode="shortlist", num_clusters=8, shortlist_top_clusters=2, shortlist_max_tokens=40, hard_negatives=6,
             random_negatives=5)),
    "exact_two_banks": (
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=2, ffn_banks=2, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=1,
             recipe_count=6, macro_rank=8),
        dict(mode="recursive_exact", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=21, fixed_depth=None)),
    "exact_one_bank": (                    # one bank each: the passes' weight-gradient products run as one
        dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8),
        dict(mode="recursive_exact", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=27, fixed_depth=None)),
    "dense": (
        dict(topology="dense", vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_dense_layers=2),
        dict(mode="dense_exact", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=7)),
}


def _pair(name):
    m, t, *rest = CASES[name]
    out = rest[0] if rest else {}
    cfg = ExperimentConfig(ModelConfig(**m), TrainingConfig(**t), OutputConfig(**out))
    ocfg = O.ModelCfg(**m, shortlist_clusters=cfg.output.num_clusters)
    otr = O.TrainCfg(**{k: v for k, v in t.items() if k in O.TrainCfg.__dataclass_fields__})
    return cfg, ocfg, otr


def _oracle(cfg, ocfg, otr, params):
    oc = O.OutputCfg(**cfg.output.__dict__) if cfg.training.mode == "recursive_macro_shortlist" else None
    return O.OracleTrainer(ocfg, otr, {k: v.clone() for k, v in params.items()}, oc=oc)


def _drop_absent_core(eng, grads):
    """Bernoulli sampler, nobody audited: the core's gradients are exact zeros, which the optimiser treats as absent
    (the reference's are `None`)."""
    if eng.audit is None or not eng.audit.bernoulli or eng.last_audit["audited"] > 0:
        return grads
    from speedup_thingy_b200.audit import CORE_PARAMS
    assert all(not bool(grads[n].any()) for n in CORE_PARAMS)
    return {n: g for n, g in grads.items() if n not in CORE_PARAMS}


def _check_alignment(eng, info):
    """macro_alignment_metrics of the audited samples (macro.py:499-546) against the oracle's."""
    if eng.audit is None or "alignment" not in info:
        return
    got = dict(eng.last_audit["alignment"], **eng.last_audit["residual"])
    for key, ref in dict(info["alignment"], **info["residual"]).items():
        if key.startswith("logit_kl"):
            # the engine's logits are bf16: their rounding noise is a sizeable share of a KL of 1e-3 between two
            # nearly equal distributions (the kernel itself is checked to 1e-3 on given logits)
            assert abs(got[key] - ref) <= 0.25 * abs(ref) + 1e-4, (key, got[key], ref)
        elif key.startswith("audit_residual_") or key.endswith("loss_residual"):
            assert abs(got[key] - ref) <= 2e-2 * max(abs(ref), 1.0), (key, got[key], ref)   # differences of summed losses
        else:
            assert abs(got[key] - ref) <= 2e-2 * max(abs(ref), 5e-2), (key, got[key], ref)  # (cosines near 0: absolute 1e-3)


def _share_top_clusters(eng, *oracles):
    """The cluster ranking is a discrete decision on near-tied bf16 scores: the oracle replays the engine's."""
    if eng.shortlist:
        for o in oracles:
            o.top_clusters = eng.top_clusters.view(eng.B, eng.S, -1).cpu().long()


def test_parameter_inventory_and_init_match_oracle():
    for name in CASES:
        cfg, ocfg, otr = _pair(name)
        assert parameter_shapes(cfg.model, cfg.output.num_clusters) == O.param_shapes(ocfg)
        a, b = init_parameters(cfg.model, seed=11, num_clusters=cfg.output.num_clusters), O.init_params(ocfg, seed=11)
        for k in a:
            assert torch.equal(a[k], b[k]), k


@pytest.mark.parametrize("name", list(CASES))
def test_engine_sequence_matches_oracle(name):
    cfg, ocfg, otr = _pair(name)
    tr = cfg.training
    params = init_parameters(cfg.model, seed=tr.seed, num_clusters=cfg.output.num_clusters)
    # the dense case also exercises the un-fused SwiGLU path (what large batches take)
    eng = TrainEngine(cfg, params, device="cpu", ops=EmulOps(), use_cuda_graph=False,
                      swiglu_fuse_max_rows=0 if name == "dense" else 1024)
    oracle = _oracle(cfg, ocfg, otr, params)
    stream = O.zipf_tokens(tr.batch_size * tr.seq_len * 6 + 1, cfg.model.vocab_size, seed=tr.seed)
    it = O.batches(stream, tr.batch_size, tr.seq_len)
    batch = next(it)
    otr_noclip = O.TrainCfg(**{**otr.__dict__, "grad_clip_norm": None})
    oracle_nc = _oracle(cfg, ocfg, otr_noclip, params)
    loss, grads = eng.loss_and_grads(batch)
    _share_top_clusters(eng, oracle_nc)
    ref_loss, ref_grads, ref_info = oracle_nc.loss_and_grads(*batch)
    assert abs(loss - float(ref_loss)) < 2e-2
    grads = _drop_absent_core(eng, grads)
    _check_alignment(eng, ref_info)
    assert sorted(grads) == sorted(ref_grads)
    for n, g in grads.items():
        err = (g - ref_grads[n]).abs().max().item()
        scale = ref_grads[n].abs().max().item()
        assert err <= 2e-2 * max(scale, 1e-3) + 2e-4, (n, err, scale)
    # three optimiser steps: losses and weights track the fp32 oracle
    it = O.batches(stream, tr.batch_size, tr.seq_len)
    # (residual clip under per-sample probabilities: one step -- a residual that crosses the clip between a bf16 and an
    #  fp32 run switches a whole sample's exact-path gradient on or off, which Adam turns into +-lr everywhere)
    n_steps = 1 if name == "macro_bernoulli_nocap_clip" else 3
    for _ in range(n_steps):
        b = next(it)
        r = eng.train_step(b)
        _share_top_clusters(eng, oracle)
        ol = oracle.train_step(*b)
        assert abs(r.loss - ol) < max(3e-2, 2e-3 * abs(ol)), (r.loss, ol)       # bf16 products under Adam: 0.2 %
    # Adam normalises the step, so a bf16-level gradient perturbation on a near-zero gradient can flip a
    # whole +-lr step: bound the worst case by the optimiser's own step bound and the typical case tightly
    for n in eng.trainable:
        diff = (eng.params[n] - oracle.params[n]).abs()
        assert diff.max().item() <= 2.1 * tr.lr * n_steps, n
        assert diff.mean().item() <= 0.25 * tr.lr * n_steps, n
    untouched = [n for n, _ in parameter_shapes(cfg.model, cfg.output.num_clusters) if n not in eng.trainable]
    for n in untouched:
        assert torch.equal(eng.params[n], params[n]), n


@pytest.mark.parametrize("name", ["macro_audit_two_banks", "macro_shortlist"])
def test_pipelined_train_steps_equal_synchronous_steps(name):
    """`train_steps` keeps two steps queued; losses, metrics and weights must be those of one `train_step` per batch
    (per-step seeds, the audited subset of each step and the usage average all advance in submission order)."""
    cfg, _, _ = _pair(name)
    tr = cfg.training
    params = init_parameters(cfg.model, seed=tr.seed, num_clusters=cfg.output.num_clusters)
    stream = O.zipf_tokens(tr.batch_size * tr.seq_len * 5 + 1, cfg.model.vocab_size, seed=tr.seed)
    batches = [b for _, b in zip(range(5), O.batches(stream, tr.batch_size, tr.seq_len))]
    a = TrainEngine(cfg, {k: v.clone() for k, v in params.items()}, device="cpu", ops=EmulOps(), use_cuda_graph=False)
    b = TrainEngine(cfg, {k: v.clone() for k, v in params.items()}, device="cpu", ops=EmulOps(), use_cuda_graph=False)
    ra = [a.train_step(x) for x in batches]
    rb = list(b.train_steps(iter(batches)))
    assert [r.loss for r in ra] == [r.loss for r in rb]
    assert ra[-1].metrics == rb[-1].metrics and a.global_step == b.global_step == 5
    for n in a.params:
        assert torch.equal(a.params[n], b.params[n]), n
    b.submit(batches[0]); b.submit(batches[1])
    with pytest.raises(RuntimeError, match="in flight"):
        b.submit(batches[2])
    with pytest.raises(RuntimeError, match="in flight"):
        b.train_step(batches[2])
    b.collect(); b.collect()
    with pytest.raises(RuntimeError, match="no step in flight"):
        b.collect()


def test_hot_budget_matches_reference_estimators_and_enforces_limits():
    """training.py:707-740 / metrics.py:69-94, pinned to values the reference computed for BASELINE config 1."""
    from pathlib import Path

    from speedup_thingy_b200.engine import dense_aligned_param_count, hot_budget
    from tests.golden.cases import GOLDEN_CASES
    gold = np.load(Path(__file__).resolve().parent / "golden" / "per_op.npz")["budget"]
    case = GOLDEN_CASES["c1_macro"]
    model = ModelConfig(**{k: v for k, v in case["model"].items() if k != "shortlist_clusters"})
    tr = TrainingConfig(**{**case["train"], "audit_fixed_count_per_batch": None})
    assert hot_budget(model, tr, None)["active_param_equiv_per_token"] == gold[0]
    assert hot_budget(model, tr, 128)["active_param_equiv_per_token"] == gold[1]
    assert hot_budget(model, tr, None)["hotpath_flops_per_token_est"] == 2.0 * gold[0]
    assert float(dense_aligned_param_count(model)) == gold[2]
    with pytest.raises(RuntimeError, match="active parameter budget"):
        hot_budget(model, TrainingConfig(**{**tr.__dict__, "max_active_param_equiv_per_token": gold[0] - 1}), None)
    with pytest.raises(RuntimeError, match="FLOPs/token budget"):
        hot_budget(model, TrainingConfig(**{**tr.__dict__, "max_hotpath_flops_per_token": gold[0]}), None)
    with pytest.raises(RuntimeError, match="active parameter budget"):
        hot_budget(model, TrainingConfig(**{**tr.__dict__, "target_speedup_vs_dense": 1e6}), None)
    ok = hot_budget(model, TrainingConfig(**{**tr.__dict__, "target_speedup_vs_dense": 1.01}), None)
    assert ok["active_param_budget"] == gold[2] / 1.01


@pytest.mark.parametrize("name", ["macro_fixed_depth", "exact_two_banks", "dense", "macro_audit_two_banks"])
def test_evaluate_is_forward_only_and_matches_the_oracle_forward(name):
    """`TrainEngine.evaluate` (the counterpart of `rte evaluate`, cli.py:193-319): the mode's forward loss per sample,
    nothing else touched."""
    cfg, ocfg, otr = _pair(name)
    tr = cfg.training
    params = init_parameters(cfg.model, seed=tr.seed, num_clusters=cfg.output.num_clusters)
    eng = TrainEngine(cfg, {k: v.clone() for k, v in params.items()}, device="cpu", ops=EmulOps(), use_cuda_graph=False)
    stream = O.zipf_tokens(tr.batch_size * tr.seq_len * 3 + 1, cfg.model.vocab_size, seed=tr.seed)
    batches = [b for _, b in zip(range(2), O.batches(stream, tr.batch_size, tr.seq_len))]
    out = eng.evaluate(batches)
    want = []
    for tokens, targets in batches:
        if cfg.model.topology == "dense":
            want.append(O.forward_dense(params, ocfg, tokens, targets)["loss_per_sample"])
        elif tr.mode == "recursive_exact":
            _, info = O.exact_step_loss(params, ocfg, otr, tokens, targets, torch.zeros(ocfg.recipe_count))
            want.append(info["hot"]["loss_per_sample"])
        else:
            want.append(O.forward_macro(params, ocfg, tokens, targets, tr.fixed_recipe, tr.fixed_depth)["loss_per_sample"])
    ref = float(torch.cat(want).mean())
    assert abs(out["eval_loss_per_sample"] - ref) <= 5e-3 * abs(ref), (out, ref)
    assert out["eval_nll_per_token"] == pytest.approx(out["eval_loss_per_sample"] / tr.seq_len)
    assert out["samples"] == 2 * tr.batch_size
    for n in eng.params:                                   # weights, moments and counters untouched
        assert torch.equal(eng.params[n], params[n]), n
    assert eng.global_step == 0 and int(eng.plan.step_count.max()) == 0
    assert (eng.audit is not None) == bool(tr.audit_fixed_count_per_batch)


def _macro_scaled(params):
    """Macro-operator weights far from their near-zero initialisation, so that the consistency term and its gradients
    are of the same order as the rest of the loss."""
    g = torch.Generator().manual_seed(123)
    out = {k: v.clone() for k, v in params.items()}
    out["macro.u"] = torch.randn(out["macro.u"].shape, generator=g) * 0.5
    out["macro.v"] = torch.randn(out["macro.v"].shape, generator=g) * 0.2
    out["macro.d_gain"] = torch.randn(out["macro.d_gain"].shape, generator=g) * 0.3
    out["macro.bias"] = torch.randn(out["macro.bias"].shape, generator=g) * 0.2
    return out


def test_consistency_term_is_material_and_matches_the_oracle():
    """lambda_cons * mse(Phi_2k(h0,h0), Phi_k(Phi_k(h0,h0),h0)) (macro.py:342-359): loss and every gradient against the
    oracle with macro weights for which the term dominates the macro operator's gradients."""
    cfg, ocfg, otr = _pair("macro_consistency")
    tr = cfg.training
    params = _macro_scaled(init_parameters(cfg.model, seed=tr.seed, num_clusters=cfg.output.num_clusters))
    eng = TrainEngine(cfg, params, device="cpu", ops=EmulOps(), use_cuda_graph=False)
    nc = {**otr.__dict__, "grad_clip_norm": None}
    with_cons, without = _oracle(cfg, ocfg, O.TrainCfg(**nc), params), _oracle(cfg, ocfg, O.TrainCfg(**{**nc, "lambda_cons": 0.0}), params)
    stream = O.zipf_tokens(tr.batch_size * tr.seq_len * 3 + 1, cfg.model.vocab_size, seed=tr.seed)
    batch = next(O.batches(stream, tr.batch_size, tr.seq_len))
    loss, grads = eng.loss_and_grads(batch)
    ref_loss, ref_grads, info = with_cons.loss_and_grads(*batch)
    base_loss, base_grads, _ = without.loss_and_grads(*batch)
    assert float(info["aux"]["cons"]) > 0.01 * abs(float(base_loss))                 # the term matters
    assert (ref_grads["macro.u"] - base_grads["macro.u"]).abs().max() > 0.5 * base_grads["macro.u"].abs().max()
    assert (ref_grads["embed.weight"] - base_grads["embed.weight"]).abs().max() > 0.05 * base_grads["embed.weight"].abs().max()
    assert abs(loss - float(ref_loss)) < 2e-2 * max(1.0, abs(float(ref_loss)))
    assert abs(eng.last_consistency - float(info["aux"]["cons"])) <= 2e-2 * float(info["aux"]["cons"])
    for n, g in grads.items():
        err = (g - ref_grads[n]).abs().max().item()
        scale = ref_grads[n].abs().max().item()
        assert err <= 2e-2 * max(scale, 1e-3) + 2e-4, (n, err, scale)


def test_count_schedule_follows_the_reference_trajectory():
    """audit.py:137-185 through the engine: on the golden case the reference ran (count 2 -> 4 -> 2 -> 1 -> 2 -> 4 -> 8
    -> 8 of a batch of 8) every step audits the reference's subset, decides the reference's next count and reports its
    loss; two steps can never be in flight, since a step's count depends on the metrics of the step before."""
    from pathlib import Path

    from tests.golden.cases import GOLDEN_CASES
    case = GOLDEN_CASES["small_schedule"]
    gold = np.load(Path(__file__).resolve().parent / "golden" / "small_schedule.npz")
    cfg = ExperimentConfig(ModelConfig(**case["model"]), TrainingConfig(**case["train"]), OutputConfig())
    tr = cfg.training
    params = init_parameters(cfg.model, seed=tr.seed)
    eng = TrainEngine(cfg, params, device="cpu", ops=EmulOps(), use_cuda_graph=False)
    assert eng.audit.n == tr.batch_size and eng.audit.scheduled
    stream = O.zipf_tokens(tr.batch_size * tr.seq_len * (case["steps"] + 2) + 1, cfg.model.vocab_size, seed=tr.seed)
    it = O.batches(stream, tr.batch_size, tr.seq_len)
    counts = []
    for step, r in enumerate(eng.train_steps(next(it) for _ in range(case["steps"]))):
        mask = torch.zeros(tr.batch_size, dtype=torch.bool)
        mask[eng.last_audit["chosen"]] = True
        assert np.array_equal(mask.numpy(), gold[f"audit_mask_step{step}"]), step
        assert r.metrics["audit_schedule_next_count"] == float(gold[f"audit_next_count_step{step}"]), step
        assert r.metrics["audit_count"] == r.metrics["audit_fixed_count"] == float(gold[f"audit_mask_step{step}"].sum())
        assert abs(r.loss - float(gold["losses"][step])) <= 2e-2 * abs(float(gold["losses"][step])), step
        for key in ("hidden_cosine_exact_macro", "loss_residual", "audit_residual_var", "macro_norm", "exact_norm"):
            ref = float(gold[f"audit_metric_step{step}/{key}"])
            assert abs(r.metrics[key] - ref) <= 5e-2 * max(abs(ref), 0.05), (step, key, r.metrics[key], ref)
        counts.append(int(r.metrics["audit_count"]))
    assert counts == [2, 4, 2, 1, 2, 4, 8, 8]
    eng.submit(next(it))
    with pytest.raises(RuntimeError, match="in flight"):
        eng.submit(next(it))
    eng.collect()
    small = TrainEngine(cfg, params, device="cpu", ops=EmulOps(), use_cuda_graph=False, audit_capacity=2)
    small.train_step(next(it))                   # 2 of capacity 2; the schedule then asks for 4
    with pytest.raises(RuntimeError, match="audit_capacity"):
        small.train_step(next(it))


def test_recursive_exact_with_a_fixed_recipe_schedule_follows_the_reference():
    """`fixed_recipe_schedule` in mode recursive_exact (models.py:230-247, 449-451): every sample runs recipe
    schedule[t] in pass t.  First-step gradients against the oracle, the loss curve against the golden the reference
    produced, the usage average counts the schedule; a schedule shorter than t_max or outside the bank is refused."""
    from pathlib import Path

    from tests.golden.cases import GOLDEN_CASES
    case = GOLDEN_CASES["small_exact_schedule"]
    gold = np.load(Path(__file__).resolve().parent / "golden" / "small_exact_schedule.npz")
    cfg = ExperimentConfig(ModelConfig(**case["model"]), TrainingConfig(**case["train"]), OutputConfig())
    tr = cfg.training
    params = init_parameters(cfg.model, seed=tr.seed)
    eng = TrainEngine(cfg, params, device="cpu", ops=EmulOps(), use_cuda_graph=False)
    oracle = O.OracleTrainer(O.ModelCfg(**case["model"]), O.TrainCfg(**case["train"]), {k: v.clone() for k, v in params.items()})
    stream = O.zipf_tokens(tr.batch_size * tr.seq_len * (case["steps"] + 2) + 1, cfg.model.vocab_size, seed=tr.seed)
    batches = [b for _, b in zip(range(case["steps"]), O.batches(stream, tr.batch_size, tr.seq_len))]
    loss, grads = eng.loss_and_grads(batches[0])
    ref_loss, ref_grads, _ = oracle.loss_and_grads(*batches[0])
    assert abs(loss - float(ref_loss)) < 2e-2 and sorted(grads) == sorted(ref_grads)
    for n, g in grads.items():
        err, scale = (g - ref_grads[n]).abs().max().item(), ref_grads[n].abs().max().item()
        assert err <= 2e-2 * max(scale, 1e-3) + 2e-4, (n, err, scale)
    # the routed recipes would have given other gradients: the schedule is what ran
    free = O.OracleTrainer(O.ModelCfg(**case["model"]), O.TrainCfg(**{**case["train"], "fixed_recipe_schedule": None}),
                           {k: v.clone() for k, v in params.items()})
    _, free_grads, _ = free.loss_and_grads(*batches[0])
    name = "core.mlp.wug"
    assert (free_grads[name] - ref_grads[name]).abs().max() > 0.2 * ref_grads[name].abs().max()
    losses = [eng.train_step(b).loss for b in batches]
    for b in batches:
        oracle.train_step(*b)
    rel = np.abs(np.array(losses) - gold["losses"]) / np.abs(gold["losses"])
    assert rel.max() <= 1e-2, (rel.max(), losses, gold["losses"])
    assert torch.allclose(eng.usage_ema, oracle.usage_ema, atol=1e-6)
    assert float(eng.usage_ema[4]) == 0.0 and float(eng.usage_ema[[0, 1, 2, 3]].min()) > 0.0      # recipe 4 never ran
    for bad in ((1, 2, 3), (1, 2, 3, 9)):
        with pytest.raises(ValueError, match="fixed_recipe_schedule"):
            TrainEngine(ExperimentConfig(ModelConfig(**case["model"]), TrainingConfig(**{**case["train"], "fixed_recipe_schedule": bad}),
                                         OutputConfig()), params, device="cpu", ops=EmulOps(), use_cuda_graph=False)
    with pytest.raises(NotImplementedError, match="fixed_recipe_schedule"):
        TrainEngine(ExperimentConfig(ModelConfig(**case["model"]),
                                     TrainingConfig(**{**case["train"], "mode": "recursive_macro"}), OutputConfig()),
                    params, device="cpu", ops=EmulOps(), use_cuda_graph=False)


def test_recursive_exact_carries_a_variant_macro_operator_untouched():
    """Mode recursive_exact never evaluates the macro operator, so a model whose operator is one of the reference's
    variants (hidden layer, gate, extra inputs, trainable update scale: macro.py:42-124) trains like any other: the
    reference's parameter names and shapes, its loss curve, and every macro parameter exactly as initialised."""
    from pathlib import Path

    from speedup_thingy_b200.config import unsupported
    from tests.golden.cases import GOLDEN_CASES
    case = GOLDEN_CASES["small_exact_variant"]
    gold = np.load(Path(__file__).resolve().parent / "golden" / "small_exact_variant.npz")
    cfg = ExperimentConfig(ModelConfig(**case["model"]), TrainingConfig(**case["train"]), OutputConfig())
    assert not [m for m in unsupported(cfg) if "precision" not in m]
    macro_mode = ExperimentConfig(ModelConfig(**case["model"]), TrainingConfig(**{**case["train"], "mode": "recursive_macro"}),
                                  OutputConfig())
    assert any("macro_hidden_mult" in m for m in unsupported(macro_mode))          # still refused where it would be evaluated
    tr = cfg.training
    assert parameter_shapes(cfg.model, cfg.output.num_clusters) == O.param_shapes(O.ModelCfg(**case["model"]))
    names = [n for n, _ in parameter_shapes(cfg.model)]
    for extra in ("macro.depth_embed", "macro.v2", "macro.update_scale", "macro.gate_v", "macro.gate_u", "macro.gate_bias"):
        assert extra in names
    params = init_parameters(cfg.model, seed=tr.seed)
    eng = TrainEngine(cfg, {k: v.clone() for k, v in params.items()}, device="cpu", ops=EmulOps(), use_cuda_graph=False)
    assert not any(n.startswith("macro.") for n in eng.trainable)
    stream = O.zipf_tokens(tr.batch_size * tr.seq_len * (case["steps"] + 2) + 1, cfg.model.vocab_size, seed=tr.seed)
    losses = [eng.train_step(b).loss for _, b in zip(range(case["steps"]), O.batches(stream, tr.batch_size, tr.seq_len))]
    rel = np.abs(np.array(losses) - gold["losses"]) / np.abs(gold["losses"])
    assert rel.max() <= 1e-2, (rel.max(), losses, gold["losses"])
    for n in names:
        if n.startswith("macro."):
            assert torch.equal(eng.params[n], params[n]), n


@pytest.mark.parametrize("fused", ["1", "0"])
def test_deferred_grouped_exact_mode_follows_the_reference(fused, monkeypatch):
    """`recursive_deferred_grouped_exact` (training.py:823-877, layers.py:872-912): one grouped block that sums the
    scheduled recipes' branches.  First-step loss and every gradient against the oracle, the loss curve against the
    golden the reference produced, the usage average counts the schedule; with the branches' weight gradients as one
    product over all branches and as one product per branch."""
    from pathlib import Path

    from tests.golden.cases import GOLDEN_CASES
    monkeypatch.setenv("RTE_REPLAY_FUSED_WGRAD", fused)
    case = GOLDEN_CASES["small_deferred"]
    gold = np.load(Path(__file__).resolve().parent / "golden" / "small_deferred.npz")
    cfg = ExperimentConfig(ModelConfig(**case["model"]), TrainingConfig(**case["train"]), OutputConfig())
    tr = cfg.training
    params = init_parameters(cfg.model, seed=tr.seed)
    eng = TrainEngine(cfg, {k: v.clone() for k, v in params.items()}, device="cpu", ops=EmulOps(), use_cuda_graph=False)
    assert eng.exact_schedule == [1, 3, 2, 2] and eng.exact_core.fused_wgrad == (fused == "1")
    oracle = O.OracleTrainer(O.ModelCfg(**case["model"]), O.TrainCfg(**case["train"]), {k: v.clone() for k, v in params.items()})
    stream = O.zipf_tokens(tr.batch_size * tr.seq_len * (case["steps"] + 2) + 1, cfg.model.vocab_size, seed=tr.seed)
    batches = [b for _, b in zip(range(case["steps"]), O.batches(stream, tr.batch_size, tr.seq_len))]
    loss, grads = eng.loss_and_grads(batches[0])
    ref_loss, ref_grads, _ = oracle.loss_and_grads(*batches[0])
    assert abs(loss - float(ref_loss)) < 2e-2 and sorted(grads) == sorted(ref_grads)
    for n, g in grads.items():
        err, scale = (g - ref_grads[n]).abs().max().item(), ref_grads[n].abs().max().item()
        assert err <= 2e-2 * max(scale, 1e-3) + 2e-4, (n, err, scale)
    losses = [eng.train_step(b).loss for b in batches]
    for b in batches:
        oracle.train_step(*b)
    rel = np.abs(np.array(losses) - gold["losses"]) / np.abs(gold["losses"])
    assert rel.max() <= 1e-2, (rel.max(), losses, gold["losses"])
    assert torch.allclose(eng.usage_ema, oracle.usage_ema, atol=1e-6)
    for n in eng.trainable:
        assert (eng.params[n] - oracle.params[n]).abs().max().item() <= 2.1 * tr.lr * len(batches), n
    two_banks = ExperimentConfig(ModelConfig(**{**case["model"], "ffn_banks": 2}), TrainingConfig(**case["train"]), OutputConfig())
    with pytest.raises(NotImplementedError, match="ffn_banks"):
        TrainEngine(two_banks, params, device="cpu", ops=EmulOps(), use_cuda_graph=False)
