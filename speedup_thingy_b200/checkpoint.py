"""Checkpoints in the reference's on-disk format (training.py:1656-1701): a ``torch.save`` payload with the model
``state_dict`` under the reference's parameter names, a ``torch.optim.AdamW`` ``state_dict`` laid out like the
reference's parameter groups (training.py:302-339: embedding, prelude, core, macro, coda + final norm, router), and
the step counters -- so a run can move between the reference and this engine in either direction.
"""
from __future__ import annotations

import dataclasses
import logging
from pathlib import Path

import torch

from .engine import TrainEngine

log = logging.getLogger(__name__)


def optimizer_layout(engine: TrainEngine) -> list[tuple[str, list[str]]]:
    """(group name, parameter names) in the order the reference builds its optimizer; parameters no group owns
    (the shortlist head's cluster router) are left out exactly as there."""
    names = list(engine.params)
    if engine.dense:
        return [("dense", names)]
    pick = lambda *prefixes: [n for n in names if n.startswith(prefixes)]  # noqa: E731
    groups = [("embedding", pick("embed.")), ("prelude", pick("prelude.")), ("core", pick("core.")),
              ("macro", pick("macro.")), ("coda", pick("coda.") + pick("final_norm.")), ("router", pick("router."))]
    return [(g, p) for g, p in groups if p]


def optimizer_state_dict(engine: TrainEngine) -> dict:
    """The AdamW state as ``torch.optim.AdamW(...).state_dict()`` would give it for the reference's groups: only
    parameters that have taken a step carry state (``step``, ``exp_avg``, ``exp_avg_sq``)."""
    tr = engine.tr
    layout = optimizer_layout(engine)
    cpu_params = {n: torch.nn.Parameter(torch.empty(0)) for _, ps in layout for n in ps}
    groups = []
    for gname, ps in layout:
        lr = tr.lr_for(gname if gname != "dense" else "dense")
        groups.append({"params": [cpu_params[n] for n in ps], "lr": lr, "base_lr": lr, "name": gname})
    opt = torch.optim.AdamW(groups, weight_decay=tr.weight_decay, foreach=True)
    steps = engine.plan.step_count.to("cpu")
    slot = {n: i for i, n in enumerate(engine.trainable)}
    for n, p in cpu_params.items():
        if n in slot and int(steps[slot[n]]) > 0:
            opt.state[p] = {"step": torch.tensor(float(steps[slot[n]])), "exp_avg": engine.exp_avg[n].detach().to("cpu").clone(),
                            "exp_avg_sq": engine.exp_avg_sq[n].detach().to("cpu").clone()}
    return opt.state_dict()


def audit_state_dict(engine: TrainEngine) -> dict:
    """The audit sampler's running state under the reference's keys (audit.py:38-48): the last residual and the
    audit-coverage average of the Bernoulli sampler, mse / norm of the last audited step for the count schedule --
    plus `fixed_count`, the schedule's current count (the reference keeps that in its live configuration only)."""
    a = engine.audit
    if a is None:
        return {}
    last = getattr(engine, "last_audit", None) or {}
    out: dict = {"last_sample_mode": "bernoulli" if a.bernoulli else "fixed_count",
                 "last_candidate_count": int(last.get("candidates", last.get("audited", a.n if not a.padded else 0))),
                 "last_capped_fraction": 0.0, "recent_residual": 0.0, "recipe_audit_ema": None,
                 "last_hidden_mse": None, "last_macro_norm": None}
    if a.bernoulli:
        cand, aud = int(last.get("candidates", 0)), int(last.get("audited", 0))
        out.update(recent_residual=float(a.recent.detach().cpu()), recipe_audit_ema=a.audit_ema.detach().to("cpu").clone(),
                   last_capped_fraction=float(cand - aud) / max(cand, 1))
    if a.scheduled:
        out.update(last_hidden_mse=a.schedule_state.get("mse"), last_macro_norm=a.schedule_state.get("norm"),
                   fixed_count=int(a.count))
    return out


def load_audit_state(engine: TrainEngine, state: dict) -> None:
    """Counterpart of `audit_state_dict` (audit.py:50-60); keys a checkpoint lacks leave the fresh state."""
    a = engine.audit
    if a is None or not state:
        return
    if a.bernoulli:
        a.recent.fill_(float(state.get("recent_residual", 0.0)))
        ema = state.get("recipe_audit_ema")
        if isinstance(ema, torch.Tensor) and ema.numel() == a.audit_ema.numel():
            a.audit_ema.copy_(ema.to(a.audit_ema.dtype))
        else:
            a.audit_ema.zero_()
    if a.scheduled:
        a.schedule_state = {"mse": state.get("last_hidden_mse"), "norm": state.get("last_macro_norm")}
        if state.get("fixed_count") is not None:
            a.count = int(state["fixed_count"])
    a._prepared = None                      # whatever was staged for the next step belonged to the old state


def save_checkpoint(engine: TrainEngine, path: str | Path, *, data_cursor: int | None = None) -> None:
    """Writes the reference's payload.  The configuration is stored as plain nested dicts (the reference's loader
    never reads it back, training.py:1681-1701), so the file unpickles where this package is not importable."""
    if engine._pending:
        # global_step advances at submit, tokens_seen / usage_ema at collect: a snapshot in between is inconsistent
        raise RuntimeError("steps are in flight: collect() them before saving a checkpoint")
    if engine.world > 1:
        # data parallel: every rank holds the same weights and optimiser state after the all-reduced step, so one
        # rank writes the file and the others wait for it (call this on every rank)
        import torch.distributed as dist
        if dist.get_rank(engine.pg) != 0:
            dist.barrier(group=engine.pg)
            return
    model = {n: t.detach().to("cpu").clone() for n, t in engine.params.items()}
    if not engine.dense:
        # the reference model's two persistent buffers (macro.py:99-122): the per-key update scale the macro kernels
        # read, and the teacher statistic only the reference's distillation tooling writes
        if "macro.update_scale" not in model:          # (a trainable parameter in the operator's variants, macro.py:99-108)
            model["macro.update_scale"] = engine.macro_scale.detach().to("cpu").clone()
        model["macro.teacher_delta_rms"] = engine.macro_teacher_delta_rms.clone()
    payload = {"config": dataclasses.asdict(engine.config), "model": model,
               "optimizer": optimizer_state_dict(engine), "global_step": engine.global_step,
               "global_micro_step": engine._micro, "tokens_seen": engine.tokens_seen, "audit": audit_state_dict(engine),
               "aligned_lm_phase": "aligned_lm", "data_cursor": data_cursor, "usage_ema": engine.usage_ema.clone(),
               "torch_rng_state": torch.get_rng_state()}
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    torch.save(payload, p)
    if engine.world > 1:
        import torch.distributed as dist
        dist.barrier(group=engine.pg)


def load_checkpoint(engine: TrainEngine, path: str | Path) -> int | None:
    """Loads a checkpoint written by `save_checkpoint` or by the reference's ``TrainEngine.save_checkpoint``.
    Returns the data cursor.  State of parameters this mode does not train is ignored, as is any buffer of the
    reference model that is not a parameter here."""
    payload = torch.load(path, map_location="cpu", weights_only=False)
    model = payload.get("model") or {}
    missing = [n for n in engine.params if n not in model]
    if missing:
        raise KeyError(f"checkpoint lacks parameters: {missing[:4]}{' ...' if len(missing) > 4 else ''}")
    for n, t in engine.params.items():
        if tuple(model[n].shape) != tuple(t.shape):
            raise ValueError(f"{n}: checkpoint shape {tuple(model[n].shape)} != {tuple(t.shape)}")
        t.copy_(model[n].to(t.dtype))
    for n, sh in engine.shadow.items():
        engine.ops.cast_bf16(engine.params[n], sh)
    if engine.shortlist:
        # the shortlist head's cluster router is in no optimiser group: its bf16 copy changes only here
        engine.ops.cast_bf16(engine.params["shortlist_head.cluster_router.weight"], engine.cluster_w16)
    if not engine.dense:
        if "macro.update_scale" in model:
            engine.macro_scale.copy_(model["macro.update_scale"].to(engine.macro_scale.dtype))
        if "macro.teacher_delta_rms" in model:
            engine.macro_teacher_delta_rms.copy_(model["macro.teacher_delta_rms"])
    opt = payload.get("optimizer")
    steps = torch.zeros_like(engine.plan.step_count, device="cpu")
    for n in engine.trainable:
        engine.exp_avg[n].zero_()
        engine.exp_avg_sq[n].zero_()
    if opt is not None:
        order = [n for _, ps in optimizer_layout(engine) for n in ps]
        saved = [i for g in opt["param_groups"] for i in g["params"]]
        if len(saved) == len(order):                     # same grouping: indices line up with our parameter order
            slot = {n: i for i, n in enumerate(engine.trainable)}
            for idx, n in zip(saved, order):
                st = opt["state"].get(idx)
                if st is not None and n in slot:
                    engine.exp_avg[n].copy_(st["exp_avg"])
                    engine.exp_avg_sq[n].copy_(st["exp_avg_sq"])
                    steps[slot[n]] = int(float(st["step"]))
        else:
            # a different grouping (e.g. a macro-only optimizer, or a build with a separate output group): weights
            # load, the optimizer starts fresh (training.py:1683-1689)
            log.warning("checkpoint %s: optimizer state has %d parameter slots, this engine's layout %d; "
                        "optimizer state discarded, moments and step counters start from zero", path, len(saved), len(order))
    engine.plan.step_count.copy_(steps)
    engine.global_step = int(payload.get("global_step", 0))
    engine.tokens_seen = int(payload.get("tokens_seen", 0))
    engine._micro = int(payload.get("global_micro_step", engine.global_step * engine.accum))
    engine._tokens_scheduled = engine.tokens_seen * engine.world        # the LR schedule resumes where it stopped
    engine._write_lr_table(engine.tr.lr_scale(engine._tokens_scheduled))
    engine._refresh_static_param_sq()
    if isinstance(payload.get("usage_ema"), torch.Tensor) and payload["usage_ema"].shape == engine.usage_ema.shape:
        engine.usage_ema.copy_(payload["usage_ema"])
    load_audit_state(engine, payload.get("audit") or {})
    return payload.get("data_cursor")
