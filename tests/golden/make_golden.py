"""Generate the golden fixtures in this folder from the REFERENCE implementation.

Run in a container that has the reference checkout (it is imported, unmodified,
from ``$RTE_REFERENCE_SRC``, default: the ``reference/src`` tree beside this repository):

    python tests/golden/make_golden.py

The fixtures (`*.npz`, a few tens of KB) are what `tests/test_oracle_golden.py`
pins the CPU oracle against; the GPU box has no reference checkout, so the
fixtures are committed.  Inputs are not stored: tokens and weights are
re-derived from seeds by `oracle/rte_oracle.py` (`zipf_tokens`, `init_params`),
which this script also uses to load identical weights into the reference.
"""
from __future__ import annotations

import os
import sys
import tempfile
from dataclasses import asdict
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, os.environ.get("RTE_REFERENCE_SRC", str(ROOT.parent / "reference" / "src")))

from oracle import rte_oracle as O  # noqa: E402
from tests.golden.cases import GOLDEN_CASES, oracle_cfgs  # noqa: E402
from recursive_training_engine import config as RC  # noqa: E402
from recursive_training_engine.training import TrainEngine  # noqa: E402
from recursive_training_engine.kernels import reference as RK  # noqa: E402

def reference_experiment(case: dict, run_dir: str) -> RC.ExperimentConfig:
    m = dict(case["model"])
    m.pop("shortlist_clusters", None)
    m.setdefault("topology", "recursive")
    m["depth_choices"] = list(m["depth_choices"])
    t = dict(case["train"])
    bernoulli = t.get("audit_sampler") == "bernoulli"
    audited = t.get("audit_fixed_count_per_batch") is not None or bernoulli
    p = (t["audit_fixed_count_per_batch"] / t["batch_size"]) if (audited and not bernoulli) else 0.0
    sampler = (dict(audit_sampler="bernoulli", audit_p_min=t["audit_p_min"], audit_p_max=t["audit_p_max"],
                    audit_alpha=t.get("audit_alpha", 0.08), audit_beta=t.get("audit_beta", 0.08),
                    audit_gamma=t.get("audit_gamma", 0.08), audit_cap=t.get("audit_cap"))
               if bernoulli else dict(audit_p_min=p, audit_p_max=p, audit_alpha=0.0, audit_beta=0.0, audit_gamma=0.0))
    tr = RC.TrainingConfig(
        mode=t["mode"], lr=t["lr"], weight_decay=t["weight_decay"], batch_size=t["batch_size"],
        seq_len=t["seq_len"], seed=t["seed"], precision="fp32", fixed_depth=t.get("fixed_depth"), **sampler,
        audit_fixed_count_per_batch=t.get("audit_fixed_count_per_batch"),
        audit_mode=t.get("audit_mode", "gradient_corrected" if audited else "metric_only"),
        audit_gradient_correction=audited and t.get("audit_mode", "gradient_corrected") == "gradient_corrected",
        audit_residual_clip=t.get("audit_residual_clip"), lambda_cons=t.get("lambda_cons", 0.0),
        grad_clip_norm=t.get("grad_clip_norm"),
        fixed_recipe_schedule=list(t["fixed_recipe_schedule"]) if t.get("fixed_recipe_schedule") is not None else None,
        **{k_: v_ for k_, v_ in t.items() if k_.startswith("audit_schedule_")},
        fused_optimizer=False, foreach_optimizer=True, allow_tf32=False, log_every=10_000,
    )
    out = RC.OutputConfig(**case["output"]) if "output" in case else RC.OutputConfig()
    return RC.ExperimentConfig(model=RC.ModelConfig(**m), training=tr, output=out, run_name="golden", output_dir=run_dir)


def load_oracle_init_into_reference(engine: TrainEngine, cfg: O.ModelCfg, seed: int) -> None:
    model = engine.recursive_model if engine.recursive_model is not None else engine.dense_model
    init = O.init_params(cfg, seed=seed)
    names = [n for n, _ in model.named_parameters()]
    assert names == [n for n, _ in O.param_shapes(cfg)], "oracle parameter inventory differs from the reference's"
    with torch.no_grad():
        for name, param in model.named_parameters():
            if name in init:
                assert tuple(param.shape) == tuple(init[name].shape), name
                param.copy_(init[name])


def run_case(name: str, case: dict) -> dict[str, np.ndarray]:
    cfg, tr = oracle_cfgs(case)
    out: dict[str, np.ndarray] = {}
    with tempfile.TemporaryDirectory() as tmp:
        engine = TrainEngine(reference_experiment(case, tmp), device=torch.device("cpu"))
        load_oracle_init_into_reference(engine, cfg, seed=tr.seed)
        model = engine.recursive_model if engine.recursive_model is not None else engine.dense_model
        stream = O.zipf_tokens(tr.batch_size * tr.seq_len * (case["steps"] + 2) + 1, cfg.vocab_size, seed=tr.seed)
        it = O.batches(stream, tr.batch_size, tr.seq_len)
        losses = []
        for step in range(case["steps"]):
            tokens, targets = next(it)
            if step == 0:
                # gradients of the first step, captured just before the optimizer consumes them
                captured: dict[str, torch.Tensor] = {}
                orig = engine.optimizer.step

                def step_and_capture(*a, **k):
                    for n, prm in model.named_parameters():
                        if prm.grad is not None:
                            captured[n] = prm.grad.detach().clone()
                    return orig(*a, **k)

                engine.optimizer.step = step_and_capture
                res = engine.train_step((tokens, targets))
                engine.optimizer.step = orig
                for n, g in captured.items():
                    out[f"grad_sumsq/{n}"] = np.float64(g.double().pow(2).sum().item())
                    out[f"grad_head/{n}"] = g.flatten()[:16].numpy().copy()
                out["grad_names"] = np.array(sorted(captured), dtype=object).astype(str)
                hot = res.model_output
                out["hot_loss_per_sample"] = hot.loss_per_sample.detach().numpy().copy()
                if hot.meta.router is not None:
                    out["recipe_id"] = hot.meta.router.recipe_id.numpy().copy()
                    out["recipe_id_by_pass"] = hot.meta.router.recipe_id_by_pass.numpy().copy()
                    out["depth"] = hot.meta.router.depth.numpy().copy()
                    out["recipe_logits"] = hot.meta.router.recipe_logits.detach().numpy().copy()
                    out["h0_head"] = hot.meta.h0.detach().flatten()[:32].numpy().copy()
                    out["phi_head"] = hot.meta.recurrent_hidden.detach().flatten()[:32].numpy().copy()
                out["logits_head"] = hot.logits.detach().flatten()[:32].numpy().copy()
                if hot.meta.shortlist is not None:
                    out["shortlist"] = hot.meta.shortlist.shortlist.numpy().copy()
                if res.audit is not None and res.audit.exact is not None:
                    out["audit_mask"] = res.audit.audit_mask.numpy().copy()
                    out["exact_loss_per_sample"] = res.audit.exact.loss_per_sample.detach().numpy().copy()
                    out["corrected_loss_per_sample"] = res.audit.corrected_loss_per_sample.detach().numpy().copy()
                    for k_, v_ in res.audit.macro_aux.items():
                        out[f"macro_aux/{k_}"] = np.float64(float(v_))
                    for k_ in ("hidden_cosine_exact_macro", "hidden_mse_exact_macro", "macro_norm", "exact_norm",
                               "macro_exact_norm_ratio", "delta_cosine_exact_macro", "delta_rms_exact", "delta_rms_pred",
                               "delta_rms_ratio", "hidden_cosine", "hidden_residual_l2", "logit_kl", "logit_kl_exact_macro",
                               "audit_residual_mean", "audit_residual_std", "audit_residual_var", "loss_residual",
                               "clipped_loss_residual"):
                        if k_ in res.audit.metrics:
                            out[f"audit_metric/{k_}"] = np.float64(float(res.audit.metrics[k_]))
            else:
                res = engine.train_step((tokens, targets))
            losses.append(float(res.loss.detach()))
            if case["train"].get("audit_schedule_enabled"):
                out[f"audit_mask_step{step}"] = res.audit.audit_mask.numpy().copy()
                out[f"audit_next_count_step{step}"] = np.int64(int(res.audit.metrics["audit_schedule_next_count"]))
                for k_ in ("hidden_cosine_exact_macro", "hidden_mse_exact_macro", "loss_residual", "audit_residual_var",
                           "delta_rms_ratio", "macro_norm", "exact_norm"):
                    out[f"audit_metric_step{step}/{k_}"] = np.float64(float(res.audit.metrics[k_]))
            if case["train"].get("audit_sampler") == "bernoulli":
                out[f"audit_mask_step{step}"] = res.audit.audit_mask.numpy().copy()
                out[f"audit_p_step{step}"] = res.audit.p_audit.detach().numpy().copy()
        out["losses"] = np.array(losses, dtype=np.float64)
        final = {n: p_.detach() for n, p_ in model.named_parameters()}
        out["final_param_sumsq"] = np.array(
            [final[n].double().pow(2).sum().item() for n, _ in O.param_shapes(cfg)], dtype=np.float64)
        engine.close()
    print(f"{name}: losses {losses[0]:.6f} -> {losses[-1]:.6f}")
    return out


def per_op_vectors() -> dict[str, np.ndarray]:
    """Outputs of the reference's stand-alone kernel definitions on seeded inputs."""
    g = torch.Generator().manual_seed(11)
    out: dict[str, np.ndarray] = {}
    x = torch.randn(3, 5, 24, generator=g)
    w = torch.randn(24, generator=g)
    out["rmsnorm"] = RK.k_fused_rmsnorm(x, w)[0].numpy()
    from recursive_training_engine.layers import RotaryEmbedding
    q = torch.randn(2, 3, 7, 8, generator=g)
    k = torch.randn(2, 3, 7, 8, generator=g)
    v = torch.randn(2, 3, 7, 8, generator=g)
    rq, rk = RotaryEmbedding(8)(q, k)
    out["rope_q"], out["rope_k"] = rq.numpy(), rk.numpy()
    out["attn"] = RK.k_flash_causal_dense(rq, rk, v).numpy()
    logits = torch.randn(4, 6, 17, generator=g)
    tg = torch.randint(0, 17, (4, 6), generator=g)
    out["ce"] = RK.k_cross_entropy_unreduced(logits, tg).numpy()
    out["ce_targets"] = tg.numpy()
    # AdamW: three steps of torch.optim.AdamW on one tensor (the optimiser the reference builds)
    p = torch.nn.Parameter(torch.randn(37, generator=g))
    opt = torch.optim.AdamW([p], lr=1e-2, weight_decay=0.1)
    grads = torch.randn(3, 37, generator=g)
    for i in range(3):
        p.grad = grads[i].clone()
        opt.step()
    out["adamw_p"] = p.detach().numpy().copy()
    # hot-path budget estimators (metrics.py:69-94) on BASELINE config 1
    from recursive_training_engine import metrics as RM
    mc = reference_experiment(GOLDEN_CASES["c1_macro"], tempfile.gettempdir()).model
    out["budget"] = np.array([RM.estimate_hot_active_param_equiv_per_token(mc, shortlist_size=None, include_output=True),
                              RM.estimate_hot_active_param_equiv_per_token(mc, shortlist_size=128, include_output=True),
                              float(RM.dense_aligned_param_count(mc))], dtype=np.float64)
    return out


def cluster_pool_vectors() -> dict[str, np.ndarray]:
    """The reference's StaticClusterPoolSwiGLU (layers.py:119-220) on the seeded inputs of
    tests/golden/cases.py::cluster_pool_inputs: routing, output, and gradients of sum(out * probe)."""
    from recursive_training_engine.layers import DenseSwiGLU, StaticClusterPoolSwiGLU
    from tests.golden.cases import cluster_pool_inputs
    t = cluster_pool_inputs()
    d, f = t["wd"].shape
    from types import SimpleNamespace
    dense = DenseSwiGLU(SimpleNamespace(d_model=d, d_ff=f))          # the constructor reads these two fields only
    with torch.no_grad():
        dense.wug.weight.copy_(t["wug"])
        dense.wd.weight.copy_(t["wd"])
    mod = StaticClusterPoolSwiGLU(dense, {"up_a": t["up_a"], "gate_a": t["gate_a"]},
                                  {"centers": t["centers"], "candidate_ids": t["candidate_ids"]}, rank=t["up_a"].shape[1])
    x = t["x"].clone().requires_grad_()
    out = mod(x)
    (out * t["probe"]).sum().backward()
    from recursive_training_engine.kernels.cluster_pool_ffn import route_to_static_centers
    assign = route_to_static_centers(t["x"].reshape(-1, d), t["up_a"], t["gate_a"], t["centers"])
    return {"out": out.detach().numpy(), "assignments": assign.numpy(), "dx": x.grad.numpy(),
            "dwug": mod.wug.weight.grad.numpy(), "dwd": mod.wd.weight.grad.numpy()}


def svd_ffn_vectors() -> dict[str, np.ndarray]:
    """The reference's SVDFactorSparseFFN (layers.py:342-643, mask mode) on tests/golden/cases.py::svd_ffn_inputs."""
    from recursive_training_engine.layers import SVDFactorSparseFFN
    from tests.golden.cases import SVD_FFN, svd_ffn_inputs
    c, t = SVD_FFN, svd_ffn_inputs()
    mod = SVDFactorSparseFFN(c["d"], c["f"], rank=c["rank"], top_k=c["top_k"], up_m=c["up_m"], gate_m=c["gate_m"],
                             product_m=c["product_m"], candidate_mode="mask", refresh_on_init=False)
    with torch.no_grad():
        for k in ("w_up", "w_gate", "w_down", "up_a", "up_b", "gate_a", "gate_b"):
            getattr(mod, k).copy_(t[k])
    x = t["x"].clone().requires_grad_()
    out, aux = mod(x, return_aux=True)
    (out * t["probe"]).sum().backward()
    sel = torch.zeros(x.shape[0] * x.shape[1], c["f"], dtype=torch.bool).scatter_(-1, aux["selected_ids"], True)
    # the same module in slots mode (layers.py:504-527: the three lists concatenated, first occurrences valid)
    mod.candidate_mode = "slots"
    with torch.no_grad():
        out_slots, aux_slots = mod(t["x"], return_aux=True)
    sel_slots = torch.zeros_like(sel).scatter_(-1, aux_slots["selected_ids"], True)
    return {"out": out.detach().numpy(), "selected": sel.numpy(), "avg_candidate_size": np.float64(aux["avg_candidate_size"]),
            "dx": x.grad.numpy(), "dw_up": mod.w_up.grad.numpy(), "dw_gate": mod.w_gate.grad.numpy(),
            "dw_down": mod.w_down.grad.numpy(), "out_slots": out_slots.numpy(), "selected_slots": sel_slots.numpy(),
            "avg_candidate_size_slots": np.float64(aux_slots["avg_candidate_size"]),
            "candidate_slots_slots": np.float64(aux_slots["candidate_slots"])}


def codebook_vectors() -> dict[str, np.ndarray]:
    """The reference's offline codebook builders (cli.py: `_build_svd_factor_cache` 3244-3261 restated inline for one
    weight pair, `_svd_cluster_features_and_scores` 3357-3389, `_fit_cluster_centers_from_features` 3297-3323,
    `_aggregate_cluster_scores` 3326-3351, the top-M of 4756-4760, `_active_union_ids_from_codebook` 4914-4941) on
    tests/golden/cases.py::codebook_inputs."""
    from types import SimpleNamespace

    from recursive_training_engine import cli as RCLI
    from tests.golden.cases import CODEBOOK, codebook_inputs
    c, t = CODEBOOK, codebook_inputs()
    up_w, gate_w = t["wug"].chunk(2, dim=0)
    factors = {}
    for name, mat in (("up", up_w.t().contiguous()), ("gate", gate_w.t().contiguous())):
        u, s, vh = torch.linalg.svd(mat, full_matrices=False)
        factors[f"{name}_a"], factors[f"{name}_b"] = u[:, :c["rank"]] * s[:c["rank"]], vh[:c["rank"], :]
    wd_lin = torch.nn.Linear(c["f"], c["d"], bias=False)
    with torch.no_grad():
        wd_lin.weight.copy_(t["wd"])
    block = SimpleNamespace(mlp=SimpleNamespace(wd=wd_lin))
    out = {}
    for mode in ("sum", "upgate", "product"):
        feats, scores = RCLI._svd_cluster_features_and_scores(block, t["normed"], factors, rank=c["rank"], score_mode=mode)
        out[f"scores_{mode}"] = scores.numpy() if mode == "sum" else scores[:16].numpy()     # other modes: a 16-row sample
    out["features"] = feats.numpy()
    scores = torch.from_numpy(out["scores_sum"])
    assign, centers = RCLI._fit_cluster_centers_from_features(feats, cluster_count=c["clusters"], iters=c["iters"])
    out["assignments"], out["centers"] = assign.numpy(), centers.numpy()
    for agg in ("mean", "max"):
        a = RCLI._aggregate_cluster_scores(scores, assign, cluster_count=c["clusters"], aggregation=agg)
        out[f"aggregate_{agg}"] = a.numpy()
        out[f"candidate_ids_{agg}"] = torch.topk(a, k=c["candidate_m"], dim=-1).indices.numpy()
    ids = torch.from_numpy(out["candidate_ids_mean"])
    out["union_full"] = RCLI._active_union_ids_from_codebook(ids, hidden=c["f"]).numpy()
    out["union_cap96"] = RCLI._active_union_ids_from_codebook(ids, hidden=c["f"], cap=96).numpy()
    return out


def macro_consistency_vectors() -> dict[str, np.ndarray]:
    """MacroOperators.consistency_loss (macro.py:342-359) and its gradients on seeded inputs."""
    from recursive_training_engine.macro import MacroOperators
    from tests.golden.cases import MACRO_CONS, macro_cons_inputs
    c, inp = MACRO_CONS, macro_cons_inputs()
    mc = RC.ModelConfig(topology="recursive", vocab_size=96, d_model=c["d"], n_heads=4, d_ff=64, n_dense_layers=2, n_prelude=1,
                        n_coda=1, attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2,
                        active_ffn_groups=2, macro_rank=c["rank"], recipe_count=c["recipes"],
                        depth_choices=list(c["depth_choices"]), t_max=max(c["depth_choices"]),
                        macro_update_scale=c["update_scale"])
    macro = MacroOperators(mc)
    with torch.no_grad():
        macro.d_gain.copy_(inp["params"]["macro.d_gain"])
        macro.v.copy_(inp["params"]["macro.v"])
        macro.u.copy_(inp["params"]["macro.u"])
        macro.bias.copy_(inp["params"]["macro.bias"])
    h0 = inp["h0"].clone().requires_grad_(True)
    loss = macro.consistency_loss(h0, h0, inp["recipe_ids"])
    loss.backward()
    out = {"loss": np.float64(float(loss)), "dh0": h0.grad.numpy().copy()}
    for name, prm in (("d_gain", macro.d_gain), ("v", macro.v), ("u", macro.u), ("bias", macro.bias)):
        out[f"grad/{name}"] = prm.grad.numpy().copy()
    return out


def main() -> None:
    torch.set_num_threads(4)
    only = set(sys.argv[1:])                     # e.g. `make_golden.py cluster_pool` rewrites that file alone
    for name, case in GOLDEN_CASES.items():
        if not only or name in only:
            np.savez_compressed(HERE / f"{name}.npz", **run_case(name, case))
    for name, fn in (("per_op", per_op_vectors), ("cluster_pool", cluster_pool_vectors),
                     ("svd_ffn", svd_ffn_vectors), ("codebook", codebook_vectors), ("macro_cons", macro_consistency_vectors)):
        if not only or name in only:
            np.savez_compressed(HERE / f"{name}.npz", **fn())
    print("written to", HERE)


if __name__ == "__main__":
    main()
