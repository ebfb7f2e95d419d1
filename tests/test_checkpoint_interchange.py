"""Checkpoints move between the reference and the engine in both directions (reference format:
training.py:1656-1701).  Needs the reference sources, which exist only in the build container: skipped elsewhere."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REF_SRC = os.environ.get("RTE_REFERENCE_SRC", str(Path(__file__).resolve().parents[2] / "reference" / "src"))
pytestmark = pytest.mark.skipif(not Path(REF_SRC, "recursive_training_engine").is_dir(),
                                reason="reference sources not present")

from oracle import rte_oracle as O  # noqa: E402
from speedup_thingy_b200.checkpoint import load_checkpoint, optimizer_layout, save_checkpoint  # noqa: E402
from speedup_thingy_b200.config import ExperimentConfig, ModelConfig, OutputConfig, TrainingConfig  # noqa: E402
from speedup_thingy_b200.engine import TrainEngine, init_parameters  # noqa: E402
from tests.emul_ops import EmulOps  # noqa: E402
from tests.golden.cases import GOLDEN_CASES  # noqa: E402


def _reference_engine(case, run_dir):
    sys.path.insert(0, REF_SRC)
    from tests.golden.make_golden import load_oracle_init_into_reference, reference_experiment
    from recursive_training_engine.training import TrainEngine as RefEngine
    from tests.golden.cases import oracle_cfgs
    ref = RefEngine(reference_experiment(case, run_dir), device=torch.device("cpu"))
    load_oracle_init_into_reference(ref, oracle_cfgs(case)[0], seed=case["train"]["seed"])
    return ref


def _engine(case):
    model = {k: v for k, v in case["model"].items() if k != "shortlist_clusters"}
    cfg = ExperimentConfig(ModelConfig(**model), TrainingConfig(**case["train"]), OutputConfig(**case.get("output", {})))
    params = init_parameters(cfg.model, seed=cfg.training.seed, num_clusters=cfg.output.num_clusters)
    return cfg, TrainEngine(cfg, params, device="cpu", ops=EmulOps(), use_cuda_graph=False)


def _batches(cfg, n):
    tr = cfg.training
    toks = O.zipf_tokens(tr.batch_size * tr.seq_len * (n + 1) + 1, cfg.model.vocab_size, seed=tr.seed)
    it = O.batches(toks, tr.batch_size, tr.seq_len)
    return [next(it) for _ in range(n)]


def test_engine_checkpoint_loads_into_the_reference_and_training_continues(tmp_path):
    case = GOLDEN_CASES["small_routed"]
    cfg, eng = _engine(case)
    batches = _batches(cfg, 3)
    for b in batches[:2]:
        eng.train_step(b)
    save_checkpoint(eng, tmp_path / "engine.pt", data_cursor=17)
    ref = _reference_engine(case, str(tmp_path))
    assert ref.load_checkpoint(tmp_path / "engine.pt") == 17
    assert ref.global_step == 2 and ref.tokens_seen == eng.tokens_seen
    ref_params = dict(ref.recursive_model.named_parameters())
    for n, t in eng.params.items():
        assert torch.equal(ref_params[n].detach(), t), n
    # optimizer: the reference's groups line up with the layout, and stepped parameters carry the engine's moments
    layout = [n for _, ps in optimizer_layout(eng) for n in ps]
    ref_order = [p for g in ref.optimizer.param_groups for p in g["params"]]
    assert len(layout) == len(ref_order)
    by_id = {id(p): n for n, p in ref_params.items()}
    assert [by_id[id(p)] for p in ref_order] == layout
    for p in ref_order:
        n = by_id[id(p)]
        if n in eng.trainable:
            st = ref.optimizer.state[p]
            assert float(st["step"]) == 2.0 and torch.equal(st["exp_avg"], eng.exp_avg[n]), n
        else:
            assert p not in ref.optimizer.state or not ref.optimizer.state[p]
    # one more step on each side from the same state
    a = eng.train_step(batches[2]).loss
    b = float(ref.train_step(batches[2]).loss)
    assert abs(a - b) <= 1e-2 * abs(b), (a, b)


def test_reference_checkpoint_loads_into_the_engine(tmp_path):
    case = GOLDEN_CASES["small_routed"]
    cfg, eng = _engine(case)
    ref = _reference_engine(case, str(tmp_path))
    batches = _batches(cfg, 3)
    for b in batches[:2]:
        ref.train_step(b)
    ref.save_checkpoint(tmp_path / "reference.pt", data_cursor=5)
    assert load_checkpoint(eng, tmp_path / "reference.pt") == 5
    assert eng.global_step == 2
    for n, p in ref.recursive_model.named_parameters():
        assert torch.equal(eng.params[n], p.detach()), n
    stepped = {n for n, p in ref.recursive_model.named_parameters() if ref.optimizer.state.get(p)}
    assert stepped == set(eng.trainable)
    for n, p in ref.recursive_model.named_parameters():
        if n in eng.trainable:
            assert torch.equal(eng.exp_avg_sq[n], ref.optimizer.state[p]["exp_avg_sq"]), n
    a = eng.train_step(batches[2]).loss
    b = float(ref.train_step(batches[2]).loss)
    assert abs(a - b) <= 1e-2 * abs(b), (a, b)


def test_reference_shortlist_checkpoint_refreshes_the_cluster_router(tmp_path):
    """The shortlist head's cluster router is in no optimiser group, so its bf16 copy changes only on load: after a
    reference checkpoint is loaded, the engine ranks clusters with the loaded weights."""
    case = GOLDEN_CASES["small_shortlist"]
    cfg, eng = _engine(case)
    ref = _reference_engine(case, str(tmp_path))
    router = ref.recursive_model.shortlist_head.cluster_router.weight
    with torch.no_grad():
        router.copy_(torch.randn(router.shape, generator=torch.Generator().manual_seed(123)) * 0.5)
    ref.save_checkpoint(tmp_path / "reference.pt", data_cursor=0)
    before = eng.cluster_w16.clone()
    load_checkpoint(eng, tmp_path / "reference.pt")
    assert torch.equal(eng.cluster_w16.float(), router.detach().to(torch.bfloat16).float())
    assert not torch.equal(before, eng.cluster_w16)
    eng.loss_and_grads(_batches(cfg, 1)[0])
    scores = eng.hidden16.float() @ eng.cluster_w16.float().t()
    want = O.topk_lowest(scores, eng.sl_tc)[1]
    assert torch.equal(eng.top_clusters.long(), want)


def test_checkpoint_payload_needs_no_package_and_refuses_steps_in_flight(tmp_path):
    case = GOLDEN_CASES["small_routed"]
    cfg, eng = _engine(case)
    save_checkpoint(eng, tmp_path / "a.pt")
    payload = torch.load(tmp_path / "a.pt", map_location="cpu", weights_only=False)
    assert isinstance(payload["config"], dict) and payload["config"]["model"]["d_model"] == cfg.model.d_model
    eng.submit(_batches(cfg, 1)[0])
    with pytest.raises(RuntimeError, match="in flight"):
        save_checkpoint(eng, tmp_path / "b.pt")
    eng.collect()
    save_checkpoint(eng, tmp_path / "b.pt")


@pytest.mark.parametrize("name", ["small_bernoulli", "small_schedule"])
def test_audit_sampler_state_survives_a_checkpoint(tmp_path, name):
    """The Bernoulli sampler's last residual and audit-coverage average, and the count schedule's count and slope
    memory, are part of the checkpoint (audit.py:38-60): a resumed engine audits the same samples and reports the same
    losses as the one that kept running, and the reference reads the state under its own keys."""
    case = GOLDEN_CASES[name]
    cfg, eng = _engine(case)
    batches = _batches(cfg, 5)
    for b in batches[:3]:
        eng.train_step(b)
    save_checkpoint(eng, tmp_path / "mid.pt")
    _, resumed = _engine(case)
    load_checkpoint(resumed, tmp_path / "mid.pt")
    for b in batches[3:]:
        x, y = eng.train_step(b), resumed.train_step(b)
        assert x.loss == y.loss and x.metrics["audit_count"] == y.metrics["audit_count"]
        assert torch.equal(eng.last_audit["chosen"], resumed.last_audit["chosen"])
    state = torch.load(tmp_path / "mid.pt", weights_only=False)["audit"]
    ref = _reference_engine(case, str(tmp_path))
    ref.load_checkpoint(tmp_path / "mid.pt")
    if name == "small_bernoulli":
        assert state["last_sample_mode"] == "bernoulli" and state["recent_residual"] > 0
        assert ref.audit_engine.recent_residual == state["recent_residual"]
        assert torch.equal(ref.audit_engine.recipe_audit_ema, state["recipe_audit_ema"])
        assert float(state["recipe_audit_ema"].sum()) > 0
    else:
        assert state["fixed_count"] == int(np.load(Path(__file__).parent / "golden" / f"{name}.npz")["audit_next_count_step2"])
        assert ref.audit_engine.last_hidden_mse == state["last_hidden_mse"] > 0
        assert ref.audit_engine.last_macro_norm == state["last_macro_norm"] > 0


def test_variant_macro_operator_checkpoints_move_both_ways(tmp_path):
    """recursive_exact on a model with a variant macro operator (extra, untouched parameters; `update_scale` a
    parameter instead of a buffer): the engine's checkpoint loads into the reference's model strictly, the
    reference's into the engine, and both continue with the same loss."""
    case = GOLDEN_CASES["small_exact_variant"]
    cfg, eng = _engine(case)
    batches = _batches(cfg, 3)
    for b in batches[:2]:
        eng.train_step(b)
    save_checkpoint(eng, tmp_path / "engine.pt")
    ref = _reference_engine(case, str(tmp_path))
    ref.load_checkpoint(tmp_path / "engine.pt")
    ref_params = dict(ref.recursive_model.named_parameters())
    assert sorted(ref_params) == sorted(eng.params)
    for n, t in eng.params.items():
        assert torch.equal(ref_params[n].detach(), t), n
    a = eng.train_step(batches[2]).loss
    b = float(ref.train_step(batches[2]).loss)
    assert abs(a - b) <= 1e-2 * abs(b), (a, b)
    ref.save_checkpoint(tmp_path / "reference.pt")
    _, back = _engine(case)
    load_checkpoint(back, tmp_path / "reference.pt")
    for n, p in ref.recursive_model.named_parameters():
        assert torch.equal(back.params[n], p.detach()), n
    assert back.global_step == 3
