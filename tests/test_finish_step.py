"""The optimiser half of a step (reference `_finish_step`, training.py:445-468, with `_lr_scale` 470-490 and
`_optimizer_grad_metrics` 386-443): non-finite loss drops the step, gradient accumulation, the token-based
learning-rate schedule and the per-group gradient metrics.  Host logic with the test-only operator emulation;
the device kernels behind it are checked on the GPU in tests/test_gpu_kernels.py."""
import math

import pytest
import torch

from oracle import rte_oracle as O
from speedup_thingy_b200.config import ExperimentConfig, ModelConfig, TrainingConfig
from speedup_thingy_b200.engine import TrainEngine, init_parameters, lr_group_of
from tests.emul_ops import EmulOps

MODEL = dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8)
TRAIN = dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, batch_size=4, seq_len=16, seed=3, fixed_depth=4)


def _engine(train, model=MODEL, **kw):
    cfg = ExperimentConfig(ModelConfig(**model), TrainingConfig(**train))
    params = init_parameters(cfg.model, seed=cfg.training.seed)
    return cfg, params, TrainEngine(cfg, {k: v.clone() for k, v in params.items()}, device="cpu", ops=EmulOps(),
                                    use_cuda_graph=False, **kw)


def _batches(cfg, n, batch_size=None):
    tr = cfg.training
    bs = batch_size or tr.batch_size
    toks = O.zipf_tokens(bs * tr.seq_len * (n + 1) + 1, cfg.model.vocab_size, seed=tr.seed)
    it = O.batches(toks, bs, tr.seq_len)
    return [next(it) for _ in range(n)]


def test_nonfinite_loss_drops_the_step_and_leaves_everything_untouched():
    cfg, params, eng = _engine({**TRAIN, "grad_clip_norm": 1.0})
    b = _batches(cfg, 3)
    eng.train_step(b[0])
    before = {n: t.clone() for n, t in eng.params.items()}
    m_before = {n: t.clone() for n, t in eng.exp_avg.items()}
    steps_before = eng.plan.step_count.clone()
    eng.params["final_norm.weight"][0] = float("inf")          # poisons the logits of every token
    before["final_norm.weight"][0] = float("inf")
    r = eng.train_step(b[1])
    assert not math.isfinite(r.loss)
    assert r.metrics["skipped_nonfinite_loss"] == 1.0 and r.metrics["did_optimizer_step"] is False
    assert eng.global_step == 1                                  # optimiser steps taken, as the reference counts them
    assert torch.equal(eng.plan.step_count, steps_before)
    for n in eng.params:
        assert torch.equal(eng.params[n], before[n]), n
    for n in eng.exp_avg:
        assert torch.equal(eng.exp_avg[n], m_before[n]), n
    eng.params["final_norm.weight"][0] = 1.0                     # repaired: training carries on
    r = eng.train_step(b[2])
    assert math.isfinite(r.loss) and r.metrics["did_optimizer_step"] and "skipped_nonfinite_loss" not in r.metrics
    assert eng.global_step == 2 and int(eng.plan.step_count.max()) == 2


def test_gradient_accumulation_equals_the_large_batch():
    """Two micro-batches of two samples == one batch of four (the reference's own parity template,
    tests/test_training_fixes.py:53-75); the router's batch-nonlinear auxiliary loss is off for the comparison."""
    base = {**TRAIN, "disable_router_aux": True, "fixed_recipe": 1}
    cfg_big, _, big = _engine({**base, "batch_size": 4})
    cfg_small, _, small = _engine({**base, "batch_size": 2, "grad_accum_steps": 2})
    tokens, targets = _batches(cfg_big, 1)[0]
    big.train_step((tokens, targets))
    r1 = small.train_step((tokens[:2], targets[:2]))
    assert r1.metrics["did_optimizer_step"] is False and small.global_step == 0
    for n in small.params:                                       # nothing moves on a micro-batch
        assert int(small.plan.step_count.max()) == 0
    r2 = small.train_step((tokens[2:], targets[2:]))
    assert r2.metrics["did_optimizer_step"] is True and small.global_step == 1
    for n in big.trainable:
        # Adam's first step is +-lr * sign-like: compare the gradients the optimiser consumed through the moments
        assert torch.allclose(small.exp_avg[n], big.exp_avg[n], rtol=2e-3, atol=2e-6), n
        assert torch.allclose(small.params[n], big.params[n], rtol=0, atol=2.5e-3 * cfg_big.training.lr + 1e-6), n
    assert float(small.accum_flat.abs().max()) == 0.0            # cleared for the next cycle


def test_token_based_lr_schedule_follows_the_reference_formula():
    tr = {**TRAIN, "lr_schedule": "linear_decay_after", "lr_decay_start_tokens": 64, "lr_decay_end_tokens": 256,
          "lr_final_scale": 0.1, "lr_macro": 5e-3}
    cfg, params, eng = _engine(tr)
    oracle = O.OracleTrainer(O.ModelCfg(**MODEL), O.TrainCfg(**TRAIN), {k: v.clone() for k, v in params.items()})
    tokens_per_step = cfg.training.batch_size * cfg.training.seq_len
    seen = 0
    for i, b in enumerate(_batches(cfg, 5)):
        # training.py:470-483 evaluated on the tokens seen BEFORE the step
        if seen <= 64:
            want = 1.0
        elif seen >= 256:
            want = 0.1
        else:
            want = 1.0 + (seen - 64) / (256 - 64) * (0.1 - 1.0)
        r = eng.train_step(b)
        assert r.metrics["lr"] == pytest.approx(2e-3 * want, rel=1e-6)
        assert float(eng.plan.lr_table[3]) == pytest.approx(5e-3 * want, rel=1e-6)      # the macro group's own base rate
        seen += tokens_per_step
    assert eng.tr.lr_scale(10 ** 9) == 0.1


def test_grad_metrics_match_a_direct_computation():
    cfg, params, eng = _engine({**TRAIN, "grad_clip_norm": 0.25, "fixed_depth": None})
    b = _batches(cfg, 1)[0]
    p0 = {n: t.clone() for n, t in eng.params.items()}
    r = eng.train_step(b)
    grads = {n: g.clone() for n, g in eng.grads.items()}
    total = math.sqrt(sum(float(g.double().pow(2).sum()) for g in grads.values()))
    coef = min(1.0, 0.25 / (total + 1e-6))
    groups = {}
    for n, p in p0.items():
        if n.startswith("shortlist_head."):
            continue
        g = groups.setdefault(lr_group_of(n, "recursive"), [0.0, 0.0])
        g[1] += float(p.double().pow(2).sum())
        if n in grads:
            g[0] += float((grads[n] * coef).double().pow(2).sum())
    for name, (g2, p2) in groups.items():
        assert r.metrics[f"grad_norm_{name}"] == pytest.approx(math.sqrt(g2), rel=1e-4, abs=1e-9), name
        assert r.metrics[f"update_ratio_{name}"] == pytest.approx(2e-3 * math.sqrt(g2) / max(math.sqrt(p2), 1e-12), rel=1e-4, abs=1e-12)
    # the core received no gradient (no audit): its norms are zero, its parameter norm still counts
    assert r.metrics["grad_norm_core"] == 0.0 and r.metrics["grad_norm_pass_film"] == 0.0
    assert "grad_norm_dense" not in r.metrics
