"""Pins the CPU oracle (oracle/rte_oracle.py) against fixtures produced by the
reference implementation itself (tests/golden/make_golden.py)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import rte_oracle as O
from tests.golden.cases import GOLDEN_CASES, oracle_cfgs, oracle_output_cfg

GOLDEN = Path(__file__).resolve().parent / "golden"


def _run(name):
    case = GOLDEN_CASES[name]
    cfg, tr = oracle_cfgs(case)
    gold = np.load(GOLDEN / f"{name}.npz")
    trainer = O.OracleTrainer(cfg, tr, O.init_params(cfg, seed=tr.seed), oc=oracle_output_cfg(case))
    stream = O.zipf_tokens(tr.batch_size * tr.seq_len * (case["steps"] + 2) + 1, cfg.vocab_size, seed=tr.seed)
    it = O.batches(stream, tr.batch_size, tr.seq_len)
    return case, cfg, tr, gold, trainer, it


@pytest.mark.parametrize("name", list(GOLDEN_CASES))
def test_first_step_matches_reference(name):
    case, cfg, tr, gold, trainer, it = _run(name)
    tokens, targets = next(it)
    loss, grads, info = trainer.loss_and_grads(tokens, targets)
    assert abs(float(loss) - gold["losses"][0]) <= 2e-5 * max(1.0, abs(gold["losses"][0]))
    np.testing.assert_allclose(info["hot"]["loss_per_sample"].detach().numpy(), gold["hot_loss_per_sample"],
                               rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(info["hot"]["logits"].detach().flatten()[:32].numpy(), gold["logits_head"],
                               rtol=1e-4, atol=2e-6)
    if cfg.topology != "dense":
        route = info["hot"]["route"]
        assert np.array_equal(route["recipe_id"].numpy(), gold["recipe_id"])
        assert np.array_equal(route["recipe_id_by_pass"].numpy(), gold["recipe_id_by_pass"])
        assert np.array_equal(route["depth"].numpy(), gold["depth"])
        np.testing.assert_allclose(route["recipe_logits"].detach().numpy(), gold["recipe_logits"], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(info["hot"]["h0"].detach().flatten()[:32].numpy(), gold["h0_head"], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(info["hot"]["recurrent_hidden"].detach().flatten()[:32].numpy(), gold["phi_head"],
                                   rtol=1e-4, atol=1e-6)
    if "shortlist" in gold:
        assert np.array_equal(info["hot"]["shortlist"]["shortlist"].numpy(), gold["shortlist"])
    if "audit_mask" in gold:
        assert np.array_equal(info["mask"].numpy(), gold["audit_mask"])
        np.testing.assert_allclose(info["exact"]["loss_per_sample"].detach().numpy(), gold["exact_loss_per_sample"],
                                   rtol=2e-5, atol=2e-5)
        np.testing.assert_allclose(info["corrected"].detach().numpy(), gold["corrected_loss_per_sample"],
                                   rtol=2e-4, atol=2e-4)
        for key, val in info["aux"].items():
            assert abs(float(val) - float(gold[f"macro_aux/{key}"])) <= 1e-5 + 1e-4 * abs(float(gold[f"macro_aux/{key}"])), key
        reported = dict(info.get("alignment", {}), **info.get("residual", {}))
        assert "audit_metric/logit_kl_exact_macro" not in gold or "logit_kl_exact_macro" in reported
        for key, val in reported.items():          # macro_alignment_metrics, residual statistics (macro.py:499-546, audit.py:306-310)
            if f"audit_metric/{key}" in gold:
                ref = float(gold[f"audit_metric/{key}"])
                assert abs(val - ref) <= 1e-6 + 2e-4 * abs(ref), (key, val, ref)
    # exactly the parameters the reference gave a gradient to, with the same gradients
    assert sorted(grads) == sorted(str(n) for n in gold["grad_names"])
    for n, g in grads.items():
        ref_sumsq = float(gold[f"grad_sumsq/{n}"])
        assert abs(float(g.double().pow(2).sum()) - ref_sumsq) <= 1e-3 * ref_sumsq + 1e-12, n
        np.testing.assert_allclose(g.flatten()[:16].numpy(), gold[f"grad_head/{n}"], rtol=2e-3, atol=2e-6, err_msg=n)


@pytest.mark.parametrize("name", list(GOLDEN_CASES))
def test_loss_curve_and_final_weights_match_reference(name):
    case, cfg, tr, gold, trainer, it = _run(name)
    losses = [trainer.train_step(*next(it)) for _ in range(case["steps"])]
    np.testing.assert_allclose(np.array(losses), gold["losses"], rtol=2e-4, atol=2e-5)
    sumsq = np.array([trainer.params[n].double().pow(2).sum().item() for n, _ in O.param_shapes(cfg)])
    # (small_bernoulli: parameters that start at zero move by +-lr per Adam step on gradients of 1e-9, whose sign is
    #  rounding noise between two fp32 implementations; their sums of squares are ~1e-5 and compared absolutely)
    np.testing.assert_allclose(sumsq, gold["final_param_sumsq"], rtol=2e-4, atol=1e-6 if name == "small_bernoulli" else 1e-9)


def test_per_op_vectors():
    gold = np.load(GOLDEN / "per_op.npz")
    g = torch.Generator().manual_seed(11)
    x = torch.randn(3, 5, 24, generator=g)
    w = torch.randn(24, generator=g)
    np.testing.assert_allclose(O.rmsnorm(x, w).numpy(), gold["rmsnorm"], rtol=1e-6, atol=1e-6)
    q = torch.randn(2, 3, 7, 8, generator=g)
    k = torch.randn(2, 3, 7, 8, generator=g)
    v = torch.randn(2, 3, 7, 8, generator=g)
    cos, sin = O.rope_tables(7, 8)
    rq, rk = O.rope_apply(q, cos, sin), O.rope_apply(k, cos, sin)
    np.testing.assert_allclose(rq.numpy(), gold["rope_q"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(rk.numpy(), gold["rope_k"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(O.causal_attention(rq, rk, v).numpy(), gold["attn"], rtol=1e-5, atol=1e-6)
    logits = torch.randn(4, 6, 17, generator=g)
    tg = torch.randint(0, 17, (4, 6), generator=g)
    assert np.array_equal(tg.numpy(), gold["ce_targets"])
    np.testing.assert_allclose(O.lm_loss_per_sample(logits, tg).numpy(), gold["ce"].sum(-1), rtol=1e-5, atol=1e-5)
    p = torch.randn(37, generator=g)
    m, vv = torch.zeros(37), torch.zeros(37)
    grads = torch.randn(3, 37, generator=g)
    for i in range(3):
        O.adamw_update(p, grads[i], m, vv, i + 1, 1e-2, 0.1)
    np.testing.assert_allclose(p.numpy(), gold["adamw_p"], rtol=1e-6, atol=1e-6)


def test_lowest_index_tie_rule():
    x = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0, 0.0], [5.0, 5.0, 5.0, 5.0, 5.0, 5.0]])
    assert O.argmax_lowest(x).tolist() == [1, 0]
    vals, idx = O.topk_lowest(x, 4)
    assert idx.tolist() == [[1, 2, 4, 3], [0, 1, 2, 3]]
    assert vals.tolist() == [[3.0, 3.0, 3.0, 2.0], [5.0, 5.0, 5.0, 5.0]]


def test_cluster_pool_ffn_restatement_matches_reference_golden():
    """Routing, output and every gradient of StaticClusterPoolSwiGLU (layers.py:188-220) on the seeded case."""
    from tests.golden.cases import cluster_pool_inputs
    gold = np.load(GOLDEN / "cluster_pool.npz")
    t = cluster_pool_inputs()
    x, wug, wd = (t[k].clone().requires_grad_() for k in ("x", "wug", "wd"))
    out, assign = O.static_cluster_pool_swiglu(x, wug, wd, t["up_a"], t["gate_a"], t["centers"], t["candidate_ids"])
    (out * t["probe"]).sum().backward()
    assert np.array_equal(assign.numpy(), gold["assignments"])
    np.testing.assert_allclose(out.detach().numpy(), gold["out"], rtol=1e-5, atol=1e-6)
    for got, key in ((x.grad, "dx"), (wug.grad, "dwug"), (wd.grad, "dwd")):
        np.testing.assert_allclose(got.numpy(), gold[key], rtol=1e-4, atol=1e-5)
    # the packing restatement: ascending member order, rank-addressed gather (cluster_pool_ffn.py:162-188)
    pack, flat, counts, mx = O.cluster_pack_indices(assign, 4)
    assert int(counts.sum()) == assign.numel() and mx == int(counts.max())
    assert torch.equal(pack.reshape(-1)[flat], torch.arange(assign.numel()))


def test_svd_sparse_ffn_restatement_matches_reference_golden():
    """SVDFactorSparseFFN in mask mode (layers.py:531-637): selected neurons, candidate count, output, gradients."""
    from tests.golden.cases import SVD_FFN as c, svd_ffn_inputs
    gold = np.load(GOLDEN / "svd_ffn.npz")
    t = svd_ffn_inputs()
    leaves = {k: t[k].clone().requires_grad_() for k in ("x", "w_up", "w_gate", "w_down")}
    kw = dict(top_k=c["top_k"], up_m=c["up_m"], gate_m=c["gate_m"], product_m=c["product_m"])
    out, sel = O.svd_sparse_ffn(leaves["x"], leaves["w_up"], leaves["w_gate"], leaves["w_down"], t["up_a"], t["up_b"],
                                t["gate_a"], t["gate_b"], **kw)
    (out * t["probe"]).sum().backward()
    assert np.array_equal(sel.numpy(), gold["selected"]) and (sel.sum(-1) == c["top_k"]).all()
    flat = t["x"].reshape(-1, c["d"])
    cand = O.svd_ffn_candidates(*O.svd_ffn_hats(flat, t["up_a"], t["up_b"], t["gate_a"], t["gate_b"]),
                                t["w_down"].norm(dim=-1), c["up_m"], c["gate_m"], c["product_m"])
    assert abs(float(cand.sum(-1).float().mean()) - float(gold["avg_candidate_size"])) < 1e-6
    np.testing.assert_allclose(out.detach().numpy(), gold["out"], rtol=1e-5, atol=1e-6)
    for k, name in (("x", "dx"), ("w_up", "dw_up"), ("w_gate", "dw_gate"), ("w_down", "dw_down")):
        np.testing.assert_allclose(leaves[k].grad.numpy(), gold[name], rtol=1e-4, atol=1e-5)


def test_codebook_build_restatement_matches_reference_golden():
    """Offline cluster-pool codebook build (cli.py:3244-3389, 4741-4771, 4914-4941) against the reference's builders."""
    from tests.golden.cases import CODEBOOK, codebook_inputs
    gold = np.load(GOLDEN / "codebook.npz")
    c, t = CODEBOOK, codebook_inputs()
    factors = O.svd_factor_cache(t["wug"], c["rank"])
    wd_norm = t["wd"].norm(dim=0)
    for mode in ("sum", "upgate", "product"):
        feats, scores = O.cluster_features_and_scores(t["normed"], factors, wd_norm, c["rank"], mode)
        want = gold[f"scores_{mode}"]
        np.testing.assert_allclose(scores[: want.shape[0]].numpy(), want, rtol=2e-3, atol=2e-2)    # SVD factors: LAPACK threading
    np.testing.assert_allclose(feats.numpy(), gold["features"], rtol=2e-3, atol=1e-2)
    feats, scores = torch.from_numpy(gold["features"]), torch.from_numpy(gold["scores_sum"])
    assign, centers = O.fit_cluster_centers(feats, c["clusters"], c["iters"])
    assert np.array_equal(assign.numpy(), gold["assignments"])
    np.testing.assert_allclose(centers.numpy(), gold["centers"], rtol=1e-5, atol=1e-6)
    for agg in ("mean", "max"):
        a = O.aggregate_cluster_scores(scores, assign, c["clusters"], agg)
        np.testing.assert_allclose(a.numpy(), gold[f"aggregate_{agg}"], rtol=1e-5, atol=1e-6)
        book = O.build_cluster_pool_codebook(feats, scores, c["clusters"], c["candidate_m"], agg, c["iters"])
        # the reference leaves the order of equal scores to torch.topk: compare as sets per cluster
        for mine, ref in zip(book["candidate_ids"].numpy(), gold[f"candidate_ids_{agg}"]):
            assert set(mine.tolist()) == set(ref.tolist())
    ids = torch.from_numpy(gold["candidate_ids_mean"])
    assert np.array_equal(O.active_union_ids(ids, c["f"]).numpy(), gold["union_full"])
    # capped union: the reference leaves ties at the cap boundary to torch.topk; the restatement breaks them towards the
    # lowest id, so the two selections may differ only in ids whose score equals the boundary score
    mine, ref = set(O.active_union_ids(ids, c["f"], cap=96).tolist()), set(gold["union_cap96"].tolist())
    assert len(mine) == len(ref) == 96
    m = ids.shape[1]
    weight = torch.linspace(1.0, 1.0 / m, steps=m).unsqueeze(0).expand(*ids.shape).reshape(-1)
    score = torch.zeros(c["f"]).index_add_(0, ids.reshape(-1), weight)
    boundary = min(float(score[i]) for i in ref)
    assert all(abs(float(score[i]) - boundary) < 1e-6 for i in mine ^ ref), sorted(mine ^ ref)


def test_macro_consistency_loss_matches_reference_golden():
    """O.macro_consistency_loss against MacroOperators.consistency_loss (value, d h0, every parameter gradient)."""
    from tests.golden.cases import MACRO_CONS, macro_cons_inputs
    gold = np.load(GOLDEN / "macro_cons.npz")
    c, inp = MACRO_CONS, macro_cons_inputs()
    cfg = O.ModelCfg(d_model=c["d"], macro_rank=c["rank"], recipe_count=c["recipes"], depth_choices=c["depth_choices"],
                     t_max=max(c["depth_choices"]), macro_update_scale=c["update_scale"])
    leaves = {k: v.clone().requires_grad_(True) for k, v in inp["params"].items()}
    h0 = inp["h0"].clone().requires_grad_(True)
    loss = O.macro_consistency_loss(leaves, cfg, h0, inp["recipe_ids"])
    loss.backward()
    assert float(gold["loss"]) > 1e-4                      # the case is not a degenerate one
    assert abs(float(loss) - float(gold["loss"])) <= 1e-5 * float(gold["loss"])
    np.testing.assert_allclose(h0.grad.numpy(), gold["dh0"], rtol=1e-4, atol=1e-8)
    for name in ("d_gain", "v", "u", "bias"):
        np.testing.assert_allclose(leaves[f"macro.{name}"].grad.numpy(), gold[f"grad/{name}"], rtol=1e-4, atol=1e-8)


def test_bernoulli_sampler_follows_the_reference_step_by_step():
    """audit.py:79-132 over five optimiser steps: per step the audited mask and the inclusion probabilities (which
    carry the entropy, last-residual and coverage-deficit terms and the cap's rescaling) equal the reference's."""
    case, cfg, tr, gold, trainer, it = _run("small_bernoulli")
    capped = 0
    for step in range(case["steps"]):
        trainer.train_step(*next(it))
        info = trainer.last_info
        assert np.array_equal(info["mask"].numpy(), gold[f"audit_mask_step{step}"]), step
        np.testing.assert_allclose(info["p_inc"].numpy(), gold[f"audit_p_step{step}"], rtol=2e-4, atol=1e-6, err_msg=str(step))
        capped += int(not np.allclose(info["p_inc"].numpy(), info["audit_prob"].detach().numpy()))
    assert capped >= 1                      # the cap engaged on some steps and not on others
    assert capped < case["steps"]


def test_fixed_count_schedule_follows_the_reference_step_by_step():
    """audit.py:137-185 over eight optimiser steps: the audited subset of every step (whose size the schedule set after
    the step before), the count it chose next, and the metrics it decided on equal the reference's; the count goes
    down and up within the case."""
    case, cfg, tr, gold, trainer, it = _run("small_schedule")
    counts = []
    for step in range(case["steps"]):
        trainer.train_step(*next(it))
        info = trainer.last_info
        assert np.array_equal(info["mask"].numpy(), gold[f"audit_mask_step{step}"]), step
        assert info["audit_schedule_next_count"] == int(gold[f"audit_next_count_step{step}"]), step
        seen = dict(info["alignment"], **info["residual"])
        for key in ("hidden_cosine_exact_macro", "hidden_mse_exact_macro", "loss_residual", "audit_residual_var",
                    "delta_rms_ratio", "macro_norm", "exact_norm"):
            ref = float(gold[f"audit_metric_step{step}/{key}"])
            assert abs(seen[key] - ref) <= 1e-5 + 2e-3 * abs(ref), (step, key, seen[key], ref)
        counts.append(info["audit_count"])
    assert counts == [2, 4, 2, 1, 2, 4, 8, 8]


def test_fixed_count_schedule_decisions():
    """The decision rule alone (audit.py:137-185): every threshold can veto a reduction, a rising mse or norm vetoes it
    when the slope tests are on, the count never leaves [minimum, batch]."""
    tr = O.TrainCfg(batch_size=8, audit_fixed_count_per_batch=4, audit_schedule_enabled=True, audit_schedule_min_count=1)
    good = dict(hidden_cosine_exact_macro=0.99, loss_residual=0.01, delta_rms_ratio=1.0, hidden_mse_exact_macro=0.1,
                macro_norm=1.0, exact_norm=1.0, audit_residual_var=0.0)
    nxt = lambda cur=4, state=None, **over: O.audit_schedule_next_count(tr, cur, dict(good, **over), 8, {} if state is None else state)  # noqa: E731
    assert nxt() == 2 and nxt(cur=1) == 1 and nxt(cur=8) == 4
    for veto in (dict(hidden_mse_exact_macro=10.0), dict(macro_norm=5.0), dict(hidden_cosine_exact_macro=0.9),
                 dict(loss_residual=-0.2), dict(delta_rms_ratio=1.5), dict(delta_rms_ratio=0.5), dict(audit_residual_var=2.0)):
        assert nxt(**veto) == 8, veto
    assert nxt(cur=8, hidden_mse_exact_macro=10.0) == 8                       # capped at the batch
    state = {}
    assert nxt(state=state) == 2 and state["last_hidden_mse"] == 0.1
    assert nxt(state=state, hidden_mse_exact_macro=0.2) == 8                  # mse rose since the last audited step
    assert nxt(state=state, hidden_mse_exact_macro=0.15) == 2                 # ... and fell again
    assert nxt(state=state, macro_norm=1.2) == 8                              # norm rose
    missing = {k: v for k, v in good.items() if k != "audit_residual_var"}
    assert O.audit_schedule_next_count(tr, 4, missing, 8, {}) == 8            # a missing metric fails its test
    off = O.TrainCfg(batch_size=8, audit_fixed_count_per_batch=4)
    assert O.audit_schedule_next_count(off, 4, good, 8, {}) == 4
    default_min = O.TrainCfg(batch_size=512, audit_fixed_count_per_batch=8, audit_schedule_enabled=True)
    assert O.audit_schedule_next_count(default_min, 8, good, 512, {}) == 4    # minimum defaults to batch // 128
    assert O.audit_schedule_next_count(default_min, 4, good, 512, {}) == 4


def test_svd_ffn_slots_mode_of_the_reference_equals_its_mask_mode():
    """layers.py:473-527: with one candidate list at least top_k long no token falls short of top_k candidates, so the
    concatenated lists (slots) and their union mask hold the same set: the reference selected the same neurons and
    produced the same output in both modes on the golden inputs -- what lets one kernel serve both."""
    from pathlib import Path

    from tests.golden.cases import SVD_FFN
    gold = np.load(Path(__file__).resolve().parent / "golden" / "svd_ffn.npz")
    assert max(SVD_FFN["up_m"], SVD_FFN["gate_m"], SVD_FFN["product_m"]) >= SVD_FFN["top_k"]
    assert np.array_equal(gold["selected"], gold["selected_slots"])
    assert np.array_equal(gold["out"], gold["out_slots"])
    assert float(gold["avg_candidate_size"]) == float(gold["avg_candidate_size_slots"])
    assert int(gold["candidate_slots_slots"]) == SVD_FFN["up_m"] + SVD_FFN["gate_m"] + SVD_FFN["product_m"]


def test_svd_ffn_module_accepts_both_candidate_modes_and_refuses_the_rest():
    from speedup_thingy_b200.svd_ffn import SVDFactorSparseFFN
    w = torch.zeros(64, 32)
    a, b = torch.zeros(32, 8), torch.zeros(8, 64)
    with pytest.raises(NotImplementedError, match="candidate_mode"):
        SVDFactorSparseFFN(w, w, w, a, b, a, b, top_k=8, up_m=8, max_tokens=4, candidate_mode="triton")
    with pytest.raises(RuntimeError, match="strict_cuda"):          # a known mode gets as far as the device check
        SVDFactorSparseFFN(w, w, w, a, b, a, b, top_k=8, up_m=8, max_tokens=4, candidate_mode="slots")
