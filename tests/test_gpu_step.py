"""Whole-step parity on a B200: the CUDA engine against the CPU oracle and the reference-generated
golden loss curve.  Tolerances from the north star: gradients max-abs 2e-2 of their scale (bf16),
training loss within 1 % relative over the run."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import rte_oracle as O
from speedup_thingy_b200.config import ExperimentConfig, ModelConfig, OutputConfig, TrainingConfig
from speedup_thingy_b200.engine import TrainEngine, init_parameters, parameter_shapes
from tests.golden.cases import GOLDEN_CASES
from tests.test_engine_host import CASES, _check_alignment, _drop_absent_core, _macro_scaled, _oracle, _pair, _share_top_clusters

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _engine(model, train, output=None, **kw):
    model = {k: v for k, v in model.items() if k != "shortlist_clusters"}
    cfg = ExperimentConfig(ModelConfig(**model), TrainingConfig(**train), OutputConfig(**(output or {})))
    params = init_parameters(cfg.model, seed=cfg.training.seed, num_clusters=cfg.output.num_clusters)
    return cfg, params, TrainEngine(cfg, params, device="cuda:0", **kw)


def _stream(cfg, steps):
    tr = cfg.training
    toks = O.zipf_tokens(tr.batch_size * tr.seq_len * (steps + 2) + 1, cfg.model.vocab_size, seed=tr.seed)
    return O.batches(toks, tr.batch_size, tr.seq_len)


@pytest.mark.parametrize("name", list(CASES))
def test_first_step_loss_and_grads_match_oracle(name):
    model, train, *rest = CASES[name]
    cfg, params, eng = _engine(model, train, *rest, use_cuda_graph=False)
    _, ocfg, _ = _pair(name)
    okeys = O.TrainCfg.__dataclass_fields__
    oracle = _oracle(cfg, ocfg, O.TrainCfg(**{**{k: v for k, v in train.items() if k in okeys}, "grad_clip_norm": None}), params)
    batch = next(_stream(cfg, 2))
    loss, grads = eng.loss_and_grads(batch)
    _share_top_clusters(eng, oracle)
    ref_loss, ref_grads, info = oracle.loss_and_grads(*batch)
    assert abs(loss - float(ref_loss)) <= 1e-2 * abs(float(ref_loss))
    grads = _drop_absent_core(eng, grads)
    _check_alignment(eng, info)
    assert sorted(grads) == sorted(ref_grads)
    for n, g in grads.items():
        err = (g.cpu() - ref_grads[n]).abs().max().item()
        scale = ref_grads[n].abs().max().item()
        assert err <= 2e-2 * max(scale, 1e-3) + 2e-4, (n, err, scale)
    if not eng.dense:
        assert torch.equal(eng.route["recipe_id"].cpu().long(), info["hot"]["route"]["recipe_id"])
        assert torch.equal(eng.route["depth"].cpu().long(), info["hot"]["route"]["depth"])


def test_consistency_term_matches_oracle_with_material_macro_weights():
    """lambda_cons * mse(Phi_2k(h0,h0), Phi_k(Phi_k(h0,h0),h0)) on the device (three stride pairs, its own stream, Phi on a
    state other than h0): loss, the term itself and every gradient against the oracle, with macro weights for which the
    term changes the macro operator's gradients by more than half; then graph replays equal the eager step."""
    cfg, ocfg, otr = _pair("macro_consistency")
    tr = cfg.training
    params = _macro_scaled(init_parameters(cfg.model, seed=tr.seed, num_clusters=cfg.output.num_clusters))
    eng = TrainEngine(cfg, params, device="cuda:0", use_cuda_graph=False)
    nc = {**otr.__dict__, "grad_clip_norm": None}
    with_cons = _oracle(cfg, ocfg, O.TrainCfg(**nc), params)
    without = _oracle(cfg, ocfg, O.TrainCfg(**{**nc, "lambda_cons": 0.0}), params)
    batch = next(_stream(cfg, 2))
    loss, grads = eng.loss_and_grads(batch)
    ref_loss, ref_grads, info = with_cons.loss_and_grads(*batch)
    _, base_grads, _ = without.loss_and_grads(*batch)
    assert (ref_grads["macro.u"] - base_grads["macro.u"]).abs().max() > 0.5 * base_grads["macro.u"].abs().max()
    assert abs(loss - float(ref_loss)) <= 1e-2 * abs(float(ref_loss))
    assert abs(eng.last_consistency - float(info["aux"]["cons"])) <= 2e-2 * float(info["aux"]["cons"])
    for n, g in grads.items():
        err = (g.cpu() - ref_grads[n]).abs().max().item()
        scale = ref_grads[n].abs().max().item()
        assert err <= 2e-2 * max(scale, 1e-3) + 2e-4, (n, err, scale)
    # the captured step (the branch runs on its own stream inside the graph) follows the eager one
    e1 = TrainEngine(cfg, params, device="cuda:0", use_cuda_graph=False)
    e2 = TrainEngine(cfg, params, device="cuda:0", use_cuda_graph=True)
    it1, it2 = _stream(cfg, 6), _stream(cfg, 6)
    for _ in range(5):
        a, b = e1.train_step(next(it1)).loss, e2.train_step(next(it2)).loss
        assert abs(a - b) <= 1e-5 * abs(a), (a, b)
    assert e2._graph is not None


def test_c1_loss_curve_matches_reference_golden():
    case = GOLDEN_CASES["c1_macro"]
    train = {**case["train"], "audit_fixed_count_per_batch": None}
    cfg, params, eng = _engine(case["model"], train)
    gold = np.load(GOLDEN / "c1_macro.npz")["losses"]
    it = _stream(cfg, case["steps"])
    losses = np.array([eng.train_step(next(it)).loss for _ in range(case["steps"])])
    rel = np.abs(losses - gold) / np.abs(gold)
    assert rel.max() <= 1e-2, (rel.max(), losses, gold)
    assert eng.backend_status()["mode"] == "cuda_sm100a_ext" and not eng.backend_status()["uses_reference_fallback"]
    assert eng.kernel_launches_per_step and eng.kernel_launches_per_step > 20


def test_200_step_training_loss_within_one_percent():
    case = GOLDEN_CASES["c1_macro"]
    train = {**case["train"], "audit_fixed_count_per_batch": None}
    cfg, params, eng = _engine(case["model"], train)
    oracle = O.OracleTrainer(O.ModelCfg(**case["model"]), O.TrainCfg(**train), {k: v.clone() for k, v in params.items()})
    it = _stream(cfg, 200)
    rels = []
    for step in range(200):
        batch = next(it)
        a, b = eng.train_step(batch).loss, oracle.train_step(*batch)
        rels.append(abs(a - b) / abs(b))
    assert max(rels) <= 1e-2, max(rels)
    untouched = [n for n, _ in parameter_shapes(cfg.model) if n not in eng.trainable]
    for n in untouched:                      # grad-less parameters are never decayed or stepped
        assert torch.equal(eng.params[n].cpu(), params[n]), n


def test_shortlist_loss_curve_matches_reference_golden():
    """recursive_macro_shortlist with one audited sample per batch: the shortlist ids are bit-exact whenever the
    top clusters agree, and the loss curve follows the reference's within 1 %."""
    case = GOLDEN_CASES["small_shortlist"]
    cfg, params, eng = _engine(case["model"], case["train"], case["output"])
    gold = np.load(GOLDEN / "small_shortlist.npz")
    it = _stream(cfg, case["steps"])
    losses = []
    for step in range(case["steps"]):
        tokens, targets = next(it)
        losses.append(eng.train_step((tokens, targets)).loss)
        top = eng.top_clusters.view(eng.B, eng.S, -1).cpu().long()
        gen = torch.Generator().manual_seed(cfg.training.seed + step)
        rnd = torch.randint(0, cfg.model.vocab_size, (eng.B, eng.S, cfg.output.random_negatives), generator=gen)
        want = O.dedupe_preserve_first(O.shortlist_candidates(targets, top, rnd, cfg.model.vocab_size,
                                                              O.OutputCfg(**case["output"])), cfg.output.shortlist_max_tokens)
        assert torch.equal(eng.shortlist_ids.view(eng.B, eng.S, -1).cpu().long(), want)
    rel = np.abs(np.array(losses) - gold["losses"]) / np.abs(gold["losses"])
    assert rel.max() <= 1e-2, (rel.max(), losses, gold["losses"])


def test_count_schedule_follows_the_reference_trajectory_through_graph_replays():
    """Fixed-count schedule (audit.py:137-185) on the golden case the reference ran: the audited count goes 2, 4, 2, 1,
    2, 4, 8, 8 inside a replay built for the whole batch; the captured step graph serves every count (the host only
    restages slot lists and weights), each step audits the reference's subset and reports its loss within 1 %."""
    case = GOLDEN_CASES["small_schedule"]
    cfg, params, eng = _engine(case["model"], case["train"])
    gold = np.load(GOLDEN / "small_schedule.npz")
    it = _stream(cfg, case["steps"])
    counts, losses = [], []
    for step, r in enumerate(eng.train_steps(next(it) for _ in range(case["steps"]))):
        mask = torch.zeros(eng.B, dtype=torch.bool)
        mask[eng.last_audit["chosen"]] = True
        assert np.array_equal(mask.numpy(), gold[f"audit_mask_step{step}"]), step
        assert r.metrics["audit_schedule_next_count"] == float(gold[f"audit_next_count_step{step}"]), step
        for key in ("hidden_cosine_exact_macro", "loss_residual", "audit_residual_var", "macro_norm", "exact_norm"):
            ref = float(gold[f"audit_metric_step{step}/{key}"])
            assert abs(r.metrics[key] - ref) <= 5e-2 * max(abs(ref), 0.05), (step, key, r.metrics[key], ref)
        counts.append(int(r.metrics["audit_count"]))
        losses.append(r.loss)
    assert counts == [2, 4, 2, 1, 2, 4, 8, 8] and eng._graph is not None
    rel = np.abs(np.array(losses) - gold["losses"]) / np.abs(gold["losses"])
    assert rel.max() <= 1e-2, (rel.max(), losses, gold["losses"])


def test_recursive_exact_loss_curve_matches_reference_golden():
    """`recursive_exact` (every sample through the banked recurrent core, two banks, router-chosen depth) against
    the loss curve the reference produced."""
    case = GOLDEN_CASES["small_exact"]
    cfg, params, eng = _engine(case["model"], case["train"])
    gold = np.load(GOLDEN / "small_exact.npz")["losses"]
    it = _stream(cfg, case["steps"])
    losses = np.array([eng.train_step(next(it)).loss for _ in range(case["steps"])])
    rel = np.abs(losses - gold) / np.abs(gold)
    assert rel.max() <= 1e-2, (rel.max(), losses, gold)
    for n in ("macro.v", "macro.u"):                      # the macro operator is not on this path: untouched
        assert torch.equal(eng.params[n].cpu(), params[n])


def test_recursive_exact_at_c3_shapes_runs_and_learns():
    model = dict(vocab_size=2048, d_model=512, n_heads=8, d_ff=2048, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
                 attn_banks=1, ffn_banks=1, head_groups=8, ffn_groups=16, active_head_groups=4, active_ffn_groups=4,
                 recipe_count=5, macro_rank=32)
    train = dict(mode="recursive_exact", lr=1e-3, weight_decay=0.1, batch_size=32, seq_len=64, seed=0, fixed_depth=4)
    cfg, params, eng = _engine(model, train)
    it = _stream(cfg, 6)
    losses = [eng.train_step(next(it)).loss for _ in range(6)]
    assert all(np.isfinite(losses)) and losses[-1] < losses[0]
    eng.ops.check_status()


def test_checkpoint_round_trip_resumes_the_same_run(tmp_path):
    """Reference-format checkpoint (training.py:1656-1701) written by one engine and read by a fresh one: weights,
    Adam moments and step counters carry over, so both continue with the same losses."""
    from speedup_thingy_b200.checkpoint import load_checkpoint, save_checkpoint
    model, train = CASES["macro_routed_clip"]
    cfg, params, a = _engine(model, train)
    it = _stream(cfg, 6)
    batches = [next(it) for _ in range(5)]
    for b in batches[:3]:
        a.train_step(b)
    save_checkpoint(a, tmp_path / "ck.pt", data_cursor=3)
    _, _, b_eng = _engine(model, {**train, "seed": train["seed"] + 1})          # different initial weights
    assert load_checkpoint(b_eng, tmp_path / "ck.pt") == 3 and b_eng.global_step == 3
    for n in a.params:
        assert torch.equal(a.params[n], b_eng.params[n]), n
    for batch in batches[3:]:
        la, lb = a.train_step(batch).loss, b_eng.train_step(batch).loss
        assert abs(la - lb) <= 1e-4 * abs(la), (la, lb)


def test_graph_replay_equals_eager():
    model, train = CASES["macro_routed_clip"]
    cfg, params, eager = _engine(model, train, use_cuda_graph=False)
    _, _, graphed = _engine(model, train, use_cuda_graph=True)
    it = _stream(cfg, 5)
    for _ in range(4):
        batch = next(it)
        a, b = eager.train_step(batch).loss, graphed.train_step(batch).loss
        assert abs(a - b) <= 1e-4 * abs(a)


def test_pipelined_train_steps_equal_synchronous_steps():
    """Two steps in flight (`train_steps`) against one `train_step` per batch, graph replays, pinned host batches:
    identical losses and weights, with an audited sample per step."""
    model, train = CASES["macro_audit_two_banks"]
    cfg, params, a = _engine(model, train)
    _, _, b = _engine(model, train)
    batches = [tuple(t.pin_memory() for t in x) for _, x in zip(range(8), _stream(cfg, 9))]
    ra = [a.train_step(x).loss for x in batches]
    rb = [r.loss for r in b.train_steps(iter(batches))]
    assert ra == rb
    assert a.global_step == b.global_step == 8 and a.tokens_seen == b.tokens_seen
    for n in a.params:
        assert torch.equal(a.params[n], b.params[n]), n


def test_c3_shapes_one_step_finite_and_close():
    """BASELINE configs[2] shapes without the audited sample: one step against the fp32 oracle."""
    model = dict(vocab_size=2048, d_model=512, n_heads=8, d_ff=2048, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
                 attn_banks=1, ffn_banks=1, head_groups=8, ffn_groups=16, active_head_groups=2, active_ffn_groups=4,
                 recipe_count=5, macro_rank=32)
    train = dict(mode="recursive_macro", lr=1e-3, weight_decay=0.1, batch_size=16, seq_len=64, seed=0, fixed_depth=4)
    cfg, params, eng = _engine(model, train, use_cuda_graph=False)
    oracle = O.OracleTrainer(O.ModelCfg(**model), O.TrainCfg(**train), {k: v.clone() for k, v in params.items()})
    batch = next(_stream(cfg, 2))
    ref_loss, ref_grads, _ = oracle.loss_and_grads(*batch)
    loss, grads = eng.loss_and_grads(batch)
    assert abs(loss - float(ref_loss)) <= 1e-2 * abs(float(ref_loss))
    for n, g in grads.items():
        err = (g.cpu() - ref_grads[n]).abs().max().item()
        scale = ref_grads[n].abs().max().item()
        assert err <= 2e-2 * max(scale, 1e-3) + 2e-4, (n, err, scale)
