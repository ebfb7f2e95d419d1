"""The exact modes' later additions on the GPU: the fixed per-pass recipe schedule of `recursive_exact`, a variant
macro operator carried untouched, and `recursive_deferred_grouped_exact`.  Each follows the golden the reference
produced (tests/golden/small_exact_schedule / small_exact_variant / small_deferred .npz).

These three have so far run under the CPU emulation of the launch table only (tests/test_engine_host.py holds the
same checks there).  They are therefore marked as allowed to fail: a failure is reported as such without ending a
`-x` run in front of the tests collected after this file.
"""
from pathlib import Path

import numpy as np
import pytest
import torch
from oracle import rte_oracle as O
from speedup_thingy_b200.config import ExperimentConfig, ModelConfig, OutputConfig, TrainingConfig
from speedup_thingy_b200.engine import TrainEngine, init_parameters
from tests.golden.cases import GOLDEN_CASES

pytestmark = [pytest.mark.gpu, pytest.mark.xfail(strict=False, reason="first run on a GPU pending; passes under emulation")]
GOLDEN = Path(__file__).resolve().parent / "golden"


def _run(name, **kw):
    case = GOLDEN_CASES[name]
    cfg = ExperimentConfig(ModelConfig(**case["model"]), TrainingConfig(**case["train"]), OutputConfig())
    params = init_parameters(cfg.model, seed=cfg.training.seed)
    eng = TrainEngine(cfg, {k: v.clone() for k, v in params.items()}, device="cuda:0", **kw)
    tr = cfg.training
    toks = O.zipf_tokens(tr.batch_size * tr.seq_len * (case["steps"] + 2) + 1, cfg.model.vocab_size, seed=tr.seed)
    batches = [b for _, b in zip(range(case["steps"]), O.batches(toks, tr.batch_size, tr.seq_len))]
    return case, cfg, params, eng, batches, np.load(GOLDEN / f"{name}.npz")


def _grads_match(eng, case, params, batch):
    oracle = O.OracleTrainer(O.ModelCfg(**case["model"]), O.TrainCfg(**case["train"]), {k: v.clone() for k, v in params.items()})
    loss, grads = eng.loss_and_grads(batch)
    ref_loss, ref_grads, _ = oracle.loss_and_grads(*batch)
    assert abs(loss - float(ref_loss)) <= 1e-2 * abs(float(ref_loss)) and sorted(grads) == sorted(ref_grads)
    for n, g in grads.items():
        err, scale = (g.cpu() - ref_grads[n]).abs().max().item(), ref_grads[n].abs().max().item()
        assert err <= 2e-2 * max(scale, 1e-3) + 2e-4, (n, err, scale)


def _curve_matches(eng, batches, gold):
    losses = np.array([eng.train_step(b).loss for b in batches])
    rel = np.abs(losses - gold["losses"]) / np.abs(gold["losses"])
    assert rel.max() <= 1e-2, (rel.max(), losses, gold["losses"])


def test_recursive_exact_with_fixed_recipe_schedule():
    case, cfg, params, eng, batches, gold = _run("small_exact_schedule", use_cuda_graph=False)
    _grads_match(eng, case, params, batches[0])
    _, _, _, graphed, _, _ = _run("small_exact_schedule")
    _curve_matches(graphed, batches, gold)


def test_recursive_exact_carries_variant_macro_operator():
    case, cfg, params, eng, batches, gold = _run("small_exact_variant")
    _curve_matches(eng, batches, gold)
    for n, t in params.items():
        if n.startswith("macro."):
            assert torch.equal(eng.params[n].cpu(), t), n


def test_deferred_grouped_exact_mode():
    case, cfg, params, eng, batches, gold = _run("small_deferred", use_cuda_graph=False)
    _grads_match(eng, case, params, batches[0])
    _, _, _, graphed, _, _ = _run("small_deferred")
    _curve_matches(graphed, batches, gold)


def test_svd_ffn_slots_mode_equals_mask_mode_and_the_reference():
    """`candidate_mode="slots"` (layers.py:504-527): the same selected neurons and output as mask mode, and the
    reference's slots-mode output on the golden inputs."""
    from speedup_thingy_b200.svd_ffn import SVDFactorSparseFFN
    from tests.golden.cases import SVD_FFN, svd_ffn_inputs
    c, t = SVD_FFN, svd_ffn_inputs()
    gold = np.load(GOLDEN / "svd_ffn.npz")
    outs = {}
    for mode in ("mask", "slots"):
        dev = lambda k: t[k].to("cuda:0")  # noqa: E731
        m = SVDFactorSparseFFN(dev("w_up"), dev("w_gate"), dev("w_down"), t["up_a"], t["up_b"], t["gate_a"], t["gate_b"],
                               top_k=c["top_k"], up_m=c["up_m"], gate_m=c["gate_m"], product_m=c["product_m"], max_tokens=64,
                               candidate_mode=mode)
        outs[mode] = (m.forward(t["x"].to("cuda:0")).cpu(), m.selected[:33].cpu().clone(), m.candidate_slots)
    assert torch.equal(outs["mask"][0], outs["slots"][0]) and torch.equal(outs["mask"][1], outs["slots"][1])
    assert outs["slots"][2] == int(gold["candidate_slots_slots"])
    ref = torch.from_numpy(gold["out_slots"])
    assert (outs["slots"][0].view_as(ref) - ref).abs().max() <= 2e-2 * ref.abs().max()
