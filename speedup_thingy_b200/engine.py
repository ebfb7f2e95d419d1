"""Host side of the accelerated training step.

``TrainEngine`` mirrors the reference's ``TrainEngine.train_step`` for the modes ``recursive_macro``
(training.py:1336-1476 -> models.py:681-723) and ``dense_exact`` (training.py:742-769): same parameter
names and shapes (a ``state_dict`` of either side loads into the other), same loss assembly, same
AdamW semantics (parameters that receive no gradient are left untouched).  Everything numerical runs
in hand-written sm_100a kernels behind the C ABI; the forward AND backward sequences are written out
explicitly here (no autograd), all buffers are allocated once, and the whole step -- forward, backward,
gradient norm, AdamW with bf16 shadow refresh -- is captured in one CUDA graph and replayed per step.

PyTorch is used for device memory, streams and graph capture only.
"""
from __future__ import annotations

import contextlib
import os

import math
from dataclasses import dataclass, field
from typing import Any

import torch

from . import _abi as A
from .config import ExperimentConfig, ModelConfig, TrainingConfig, check_supported
from .ops import AdamWPlan

LR_GROUPS = ["embedding", "prelude", "core", "macro", "coda", "output", "router", "dense"]
# groups whose gradient / parameter norms are reported (training.py:386-443): the optimizer's groups, with the core's
# per-pass FiLM vectors and per-pass scales counted separately as well (they also belong to "core")
METRIC_GROUPS = LR_GROUPS + ["pass_film", "pass_scale"]


def metric_group_of(name: str, topology: str) -> int:
    if name.startswith(("core.pass_gamma", "core.pass_beta")):
        return METRIC_GROUPS.index("pass_film")
    if name in ("core.pass_attn_scale", "core.pass_mlp_scale"):
        return METRIC_GROUPS.index("pass_scale")
    return METRIC_GROUPS.index(lr_group_of(name, topology))


# --------------------------------------------------------------------------- parameters
def _block_shapes(prefix: str, cfg: ModelConfig) -> list[tuple[str, tuple]]:
    d, f = cfg.d_model, cfg.d_ff
    return [(f"{prefix}.norm1.weight", (d,)), (f"{prefix}.attn.wqkv.weight", (3 * d, d)),
            (f"{prefix}.attn.wo.weight", (d, d)), (f"{prefix}.norm2.weight", (d,)),
            (f"{prefix}.mlp.wug.weight", (2 * f, d)), (f"{prefix}.mlp.wd.weight", (d, f))]


def macro_param_shapes(cfg) -> list[tuple[str, tuple]]:
    """Parameters of ``MacroOperators`` in registration order for every variant the reference builds (macro.py:42-124):
    the bounded-residual operator with its optional hidden layer, gate, delta-to-h0 / depth-embedding inputs and
    trainable update scale, and the v2 delta-radius operator.  Only the plain bounded-residual form is ever
    EVALUATED by this code; the others are carried (checkpoints, parameter counts) by modes that do not call the
    macro operator."""
    r, k, d, m = cfg.recipe_count, len(cfg.depth_choices), cfg.d_model, cfg.macro_rank
    g = lambda name, default: getattr(cfg, name, default)      # noqa: E731
    delta = g("macro_include_delta_to_h0", False)
    depth_emb, hidden = g("macro_use_depth_embedding", False), max(m, m * g("macro_hidden_mult", 1))
    out: list[tuple[str, tuple]] = []
    if g("macro_type", "bounded_residual") == "v2_delta_radius":
        n_in = 3 * d + (d if (delta or g("macro_use_delta_to_h0", False)) else 0) + (d if depth_emb else 0)
        if depth_emb:
            out.append(("macro.depth_embed", (k, d)))
        if g("macro_use_recipe_embedding", False):
            n_in += d
            out.append(("macro.recipe_embed", (r, d)))
        return out + [("macro.v", (r, k, n_in, hidden)), ("macro.v2", (r, k, hidden, m)), ("macro.u", (r, k, m, d)),
                      ("macro.bias", (r, k, d)), ("macro.rho_base_raw", (r, k)), ("macro.rho_head", (r, k, d, 1))]
    n_in = 3 * d + (d if delta else 0) + (d if depth_emb else 0)
    gated = g("macro_use_gated_update", False)
    legacy = (g("macro_hidden_mult", 1) == 1 and not gated and not delta and not depth_emb
              and g("macro_update_scale_init", 1.0) == 1.0)          # then `update_scale` is a buffer, not a parameter
    if depth_emb:
        out.append(("macro.depth_embed", (k, d)))
    out += [("macro.d_gain", (r, k, d)), ("macro.v", (r, k, n_in, hidden))]
    if hidden != m:
        out.append(("macro.v2", (r, k, hidden, m)))
    out.append(("macro.u", (r, k, m, d)))
    if not legacy:
        out.append(("macro.update_scale", (r, k, d)))
    out.append(("macro.bias", (r, k, d)))
    if gated:
        out += [("macro.gate_v", (r, k, n_in, m)), ("macro.gate_u", (r, k, m, d)), ("macro.gate_bias", (r, k, d))]
    return out


def parameter_shapes(cfg: ModelConfig, num_clusters: int = 64) -> list[tuple[str, tuple]]:
    """Parameter names and shapes in the reference's registration order (models.py:78-93, 125-151);
    `num_clusters` sizes the shortlist head's cluster router (output.py:29)."""
    d, f, v = cfg.d_model, cfg.d_ff, cfg.vocab_size
    out: list[tuple[str, tuple]] = [("embed.weight", (v, d))]
    if cfg.topology == "dense":
        for i in range(cfg.n_dense_layers):
            out += _block_shapes(f"blocks.{i}", cfg)
        return out + [("final_norm.weight", (d,))]
    hid, r, k, t, m = cfg.router_hidden_dim, cfg.recipe_count, len(cfg.depth_choices), cfg.t_max, cfg.macro_rank
    head_slots = max(1, cfg.head_groups // cfg.active_head_groups)
    ffn_slots = max(1, cfg.ffn_groups // cfg.active_ffn_groups)
    for i in range(cfg.n_prelude):
        out += _block_shapes(f"prelude.{i}", cfg)
    out += [("router.pass_recipe_bias", (t, r)), ("router.pass_factor_bias", (t, hid))]

    def mlp(name: str, n_in: int, n_mid: int, n_out: int):
        return [(f"router.{name}.0.weight", (n_mid, n_in)), (f"router.{name}.0.bias", (n_mid,)),
                (f"router.{name}.2.weight", (n_out, n_mid)), (f"router.{name}.2.bias", (n_out,))]

    out += mlp("recipe_mlp", d, hid, r) + mlp("factor_mlp", d, hid, hid)
    for name, o in (("attn_bank_head", cfg.attn_banks), ("ffn_bank_head", cfg.ffn_banks),
                    ("head_slot_head", head_slots), ("ffn_slot_head", ffn_slots)):
        out += [(f"router.{name}.weight", (o, hid)), (f"router.{name}.bias", (o,))]
    out += mlp("depth_mlp", d, hid, k)
    out += [("core.pass_gamma1", (t, d)), ("core.pass_beta1", (t, d)), ("core.pass_gamma2", (t, d)),
            ("core.pass_beta2", (t, d)), ("core.pass_attn_scale", (t,)), ("core.pass_mlp_scale", (t,)),
            ("core.alpha_inj", ()), ("core.norm1.weight", (d,)), ("core.attn.wqkv", (cfg.attn_banks, d, 3 * d)),
            ("core.attn.wo", (cfg.attn_banks, d, d)), ("core.norm2.weight", (d,)),
            ("core.mlp.wug", (cfg.ffn_banks, d, 2 * f)), ("core.mlp.wd", (cfg.ffn_banks, f, d))]
    out += macro_param_shapes(cfg)
    for i in range(cfg.n_coda):
        out += _block_shapes(f"coda.{i}", cfg)
    return out + [("final_norm.weight", (d,)), ("shortlist_head.cluster_router.weight", (num_clusters, d))]


def init_parameters(cfg: ModelConfig, seed: int = 0, std: float = 0.02, num_clusters: int = 64) -> dict[str, torch.Tensor]:
    """Seeded benchmark initialisation: tensors with >= 2 dims ~ N(0, std) from one CPU generator in
    registration order; norm gains and per-pass scales 1; the input-skip gain 0.1; biases 0."""
    gen = torch.Generator().manual_seed(seed)
    params: dict[str, torch.Tensor] = {}
    for name, shape in parameter_shapes(cfg, num_clusters):
        if len(shape) >= 2:
            params[name] = torch.randn(shape, generator=gen, dtype=torch.float32) * std
        elif name.endswith(("norm1.weight", "norm2.weight", "final_norm.weight", "pass_attn_scale", "pass_mlp_scale")):
            params[name] = torch.ones(shape, dtype=torch.float32)
        elif name == "core.alpha_inj":
            params[name] = torch.tensor(0.1, dtype=torch.float32)
        else:
            params[name] = torch.zeros(shape, dtype=torch.float32)
    return params


def lr_group_of(name: str, topology: str) -> str:
    if topology == "dense":
        return "dense"
    for prefix, group in (("embed.", "embedding"), ("prelude.", "prelude"), ("core.", "core"), ("macro.", "macro"),
                          ("coda.", "coda"), ("final_norm.", "coda"), ("lm_head.", "output"), ("router.", "router"),
                          ("shortlist_head.", "output")):
        if name.startswith(prefix):
            return group
    raise KeyError(name)


# --------------------------------------------------------------------------- hot-path budget (host arithmetic)
def dense_block_param_count(cfg: ModelConfig) -> int:
    """metrics.py:12-14."""
    d = cfg.d_model
    return 4 * d * d + 3 * d * cfg.d_ff + 4 * d


def dense_aligned_param_count(cfg: ModelConfig) -> int:
    """Parameters of the dense model of the same width and depth (metrics.py:17-23,75-76; tied embeddings)."""
    return cfg.vocab_size * cfg.d_model + cfg.n_dense_layers * dense_block_param_count(cfg) + cfg.d_model


def hot_budget(cfg: ModelConfig, tr: TrainingConfig, shortlist_size: int | None) -> dict[str, float]:
    """training.py:707-740 with metrics.py:69-94: parameter-equivalents and FLOPs one token touches on the hot path
    (prelude + coda blocks, one macro operator, the output rows it scores); raises when a configured budget is exceeded."""
    d = cfg.d_model
    active = float((cfg.n_prelude + cfg.n_coda) * dense_block_param_count(cfg)
                   + d + 3 * d * cfg.macro_rank + cfg.macro_rank * d + d
                   + (cfg.vocab_size if shortlist_size is None else float(shortlist_size)) * d)
    flops = 2.0 * active
    limit = tr.max_active_param_equiv_per_token
    if tr.target_speedup_vs_dense is not None:
        target = dense_aligned_param_count(cfg) / tr.target_speedup_vs_dense
        limit = target if limit is None else min(limit, target)
    if limit is not None and active > limit:
        raise RuntimeError(f"recursive hot path exceeds active parameter budget: {active:.1f} > {limit:.1f}")
    if tr.max_hotpath_flops_per_token is not None and flops > tr.max_hotpath_flops_per_token:
        raise RuntimeError(f"recursive hot path exceeds FLOPs/token budget: {flops:.1f} > {tr.max_hotpath_flops_per_token:.1f}")
    return {"active_param_equiv_per_token": active, "hotpath_flops_per_token_est": flops,
            "active_param_budget": limit if limit is not None else 0.0}


# --------------------------------------------------------------------------- data-parallel teardown
def teardown_data_parallel(engine: "TrainEngine | None", watchdog_s: float = 30.0) -> None:
    """Ends a data-parallel run in the order NCCL needs.  A communicator keeps a reference for every collective that
    was captured into a CUDA graph, and destroying it waits until those graphs are gone; destroying it while a step
    graph (or work queued on the communication stream) still exists therefore blocks forever.  So: drain the device,
    drop the engine's graphs, run the garbage collector so that the graph objects are really destroyed, drain again,
    meet the other ranks in a last barrier, and only then destroy the process group.  Should the destroy still not
    return within `watchdog_s` seconds, the process exits (everything a caller wants to keep must be written before
    this call)."""
    import gc
    import sys
    import threading

    import torch.distributed as dist

    if engine is not None:
        engine.close()
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if not (dist.is_available() and dist.is_initialized()):
        return
    dist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if engine is not None and getattr(engine, "_peer", None) is not None:
        engine._peer.close()              # every rank is past its last exchange: unmap the peers' memory ...
        dist.barrier()
        engine._peer.flag_mem.free()      # ... and only then release what the peers had mapped
        engine._peer.stage_mem.free()
        engine._grad_mem.free()           # (the engine's gradient views dangle from here on: it is closed)
        engine._peer = engine._grad_mem = None
    sys.stdout.flush()
    sys.stderr.flush()

    def give_up() -> None:
        sys.stderr.write(f"teardown_data_parallel: destroy_process_group did not return in {watchdog_s:.0f} s; exiting\n")
        sys.stderr.flush()
        os._exit(0)

    timer = threading.Timer(watchdog_s, give_up)
    timer.daemon = True
    timer.start()
    dist.destroy_process_group()
    timer.cancel()


# --------------------------------------------------------------------------- results
@dataclass
class TrainStepResult:
    loss: float
    metrics: dict[str, Any] = field(default_factory=dict)


class _Block:
    """Saved activations of one pre-norm transformer block (layers.py:646-656)."""

    def __init__(self, prefix: str, M: int, cfg: ModelConfig, B: int, S: int, device):
        d, f = cfg.d_model, cfg.d_ff
        bf, f32 = torch.bfloat16, torch.float32
        e = lambda *shape, dtype=bf: torch.empty(*shape, dtype=dtype, device=device)  # noqa: E731
        self.prefix = prefix
        self.M, self.B, self.S = M, B, S
        self.n1, self.n2, self.y = e(M, d), e(M, d), e(M, d)
        self.qkv, self.ug, self.z = e(M, 3 * d), e(M, 2 * f), e(M, f)
        self.u, self.out = e(M, d, dtype=f32), e(M, d, dtype=f32)
        self.rstd1, self.rstd2 = e(M, dtype=f32), e(M, dtype=f32)
        self.lse = e(B * cfg.n_heads * S, dtype=f32)
        self.x_in: torch.Tensor | None = None


class _Temps:
    """Scratch tensors of one block-backward pass over M tokens (reused by every block)."""

    def __init__(self, M: int, cfg: ModelConfig, device):
        d, f = cfg.d_model, cfg.d_ff
        bf, f32 = torch.bfloat16, torch.float32
        self.dug = torch.empty(M, 2 * f, dtype=bf, device=device)
        self.dz16 = torch.empty(M, f, dtype=bf, device=device)
        self.dn16, self.dy16, self.dx16 = (torch.empty(M, d, dtype=bf, device=device) for _ in range(3))
        self.dqkv = torch.empty(M, 3 * d, dtype=bf, device=device)
        self.dxa, self.dxb, self.dxc = (torch.empty(M, d, dtype=f32, device=device) for _ in range(3))
        self.partial = torch.empty(8 * 148, d, dtype=f32, device=device)
        self.partial2 = torch.empty(8 * 148, d, dtype=f32, device=device)      # second norm backward of a block


class TrainEngine:
    def __init__(self, config: ExperimentConfig, params: dict[str, torch.Tensor] | None = None, *,
                 device: str | torch.device = "cuda:0", ops=None, use_cuda_graph: bool = True,
                 process_group=None, bucket_cap_mb: float | None = None, swiglu_fuse_max_rows: int = 1024,
                 grad_metrics: bool = True, audit_capacity: int | None = None):
        check_supported(config)          # NotImplementedError naming every configured value this path lacks
        self.config = config
        self.cfg, self.tr = config.model, config.training
        self.device = torch.device(device)
        if ops is None:
            from .ops import CudaOps  # raises when CUDA or the library is missing: no fallback
            ops = CudaOps(self.device)
        self.ops = ops
        self.use_cuda_graph = bool(use_cuda_graph) and self.device.type == "cuda"
        self._eager_steps_left = 0
        self._dp_paused = False      # True while one rank runs local passes (profiling) that others do not join
        # data parallelism: one process per GPU, the batch in `training.batch_size` is this rank's shard
        self.pg = process_group
        self.world = 1
        if process_group is not None:
            import torch.distributed as dist
            self.world = dist.get_world_size(process_group)
        if self.world > 1:
            # NCCL sets up its channels lazily on the first collectives (allocations, host synchronisation),
            # which must not happen inside stream capture: run the first steps launch by launch, and capture
            # the collective-bearing graph afterwards (RTE_DP_GRAPH=0 keeps every step eager).  A process that holds
            # such a graph should call close() before it destroys the process group.
            self._eager_steps_left = 3
            if os.environ.get("RTE_DP_GRAPH", "1") == "0":
                self.use_cuda_graph = False
        cfg, tr = self.cfg, self.tr
        # gradient accumulation (training.py:445-455): every micro-batch contributes 1/accum of its gradient, the
        # optimiser runs on every accum-th call
        self.accum = int(tr.grad_accum_steps)
        self.loss_div = self.world * self.accum         # what every loss weight is divided by
        self._micro = 0
        self.grad_metrics = bool(grad_metrics)
        self.B, self.S = tr.batch_size, tr.seq_len
        self.M = self.B * self.S
        self.dense = cfg.topology == "dense"
        if self.dense != (tr.mode == "dense_exact"):
            raise ValueError("mode dense_exact needs topology 'dense'; recursive_macro needs 'recursive'")
        self.swiglu_fuse_max_rows = int(os.environ.get("RTE_SWIGLU_FUSE_MAX_ROWS", swiglu_fuse_max_rows))
        self.oc = config.output
        self.shortlist = tr.mode == "recursive_macro_shortlist"
        self.n_clusters = self.oc.num_clusters
        # every sample runs the banked recurrent core (training.py:771-797), as t_max passes or -- `deferred` -- as one
        # grouped block that sums the scheduled recipes (training.py:823-877)
        self.deferred = tr.mode == "recursive_deferred_grouped_exact"
        self.exact = tr.mode == "recursive_exact" or self.deferred
        self.audit_k = int(tr.audit_fixed_count_per_batch or 0) if tr.audits_enabled else 0
        # Bernoulli sampler (audit.py:79-132): the audited count varies per step, so the replay gets a fixed capacity --
        # the cap when one is set, otherwise the count B * p_max can reach plus six standard deviations (beyond it the
        # step raises through the status word rather than audit a different subset than the one drawn)
        self.audit_bernoulli = (not self.dense and not self.exact and tr.audits_enabled
                                and tr.audit_fixed_count_per_batch is None)
        if self.audit_bernoulli:
            pm = min(max(float(tr.audit_p_max), 0.0), 1.0)
            bound = int(math.ceil(self.B * pm + 6.0 * math.sqrt(self.B * pm * (1.0 - pm)) + 1.0))
            self.audit_k = min(self.B, bound if tr.audit_cap is None else int(tr.audit_cap))
        # Fixed-count schedule (audit.py:137-185): the count halves or doubles between steps, up to the whole batch; the
        # replay's buffers get the capacity `audit_capacity` (default: the batch), slots beyond the step's count idle
        self.audit_scheduled = (not self.dense and not self.exact and bool(self.audit_k)
                                and not self.audit_bernoulli and tr.audit_schedule_enabled)
        if self.audit_scheduled:
            self.audit_count0 = min(self.audit_k, self.B)
            self.audit_k = self.B if audit_capacity is None else int(audit_capacity)
            if not self.audit_count0 <= self.audit_k <= self.B:
                raise ValueError(f"audit_capacity must lie between the initial audit count {self.audit_count0} and the batch size")
        self.audit_padded = self.audit_bernoulli or self.audit_scheduled
        # audit_mode "metric_only" / "distill_only" run the exact subset without gradients (audit.py:295-298): the replay
        # stops after its forward, the control variate leaves the loss, only the distillation terms reach the hot pass
        self.audit_grad = bool(self.audit_k) and tr.audit_mode == "gradient_corrected"
        if self.exact and (self.audit_k or self.dense):
            raise ValueError("recursive_exact: recursive topology, no audit (the whole batch is exact)")
        if self.audit_k:
            if self.dense:
                raise ValueError("the exact audit belongs to the recursive model")
            if self.S % 2:
                raise NotImplementedError("audit: seq_len must be even")
        if cfg.d_model % 8 or cfg.d_ff % 64 or cfg.vocab_size % 8 or cfg.head_dim not in (8, 16, 32, 64, 128):
            raise NotImplementedError("kernel size limits: d_model % 8 == 0, d_ff % 64 == 0, vocab % 8 == 0, "
                                      "head_dim in {8,16,32,64,128}")
        if self.S > 256:
            raise NotImplementedError("seq_len <= 256")
        dev, f32, bf = self.device, torch.float32, torch.bfloat16
        init = params if params is not None else init_parameters(cfg, seed=tr.seed, num_clusters=self.n_clusters)
        self._shapes = [(n, sh) for n, sh in parameter_shapes(cfg, self.n_clusters) if n in init]
        self.params = {n: init[n].detach().to(dev, f32).contiguous().clone() for n, _ in self._shapes}
        self.global_step = 0
        self.tokens_seen = 0
        self.usage_ema = torch.zeros(cfg.recipe_count, dtype=f32)

        # ---- which parameters receive a gradient in this mode (everything else is never touched)
        names = [n for n, _ in self._shapes]
        if self.dense:
            self.trainable = names
        else:
            used = ("embed.", "prelude.", "coda.", "final_norm.") + (() if self.exact else ("macro.",))
            self.trainable = [n for n in names if n.startswith(used)]
            if not tr.disable_router_aux:
                self.trainable += [n for n in names if n.startswith(("router.recipe_mlp.", "router.depth_mlp."))]
            if self.audit_grad or self.exact:
                from .audit import CORE_PARAMS
                self.trainable += CORE_PARAMS
        # gradients live in one flat buffer, laid out in the order the backward pass completes them, so that
        # data-parallel buckets are contiguous slices that can be all-reduced while backward continues
        order = self._grad_completion_order()
        assert sorted(order) == sorted(self.trainable)
        offsets, total = {}, 0
        for n in order:
            offsets[n] = total
            total += -(-self.params[n].numel() // 64) * 64          # 256-byte aligned slots
        self._grad_offsets = offsets
        # Gradient exchange: one kernel per rank over NVLink peer memory (peer_comm.PeerAllReduce) on GPUs, which
        # needs the gradient buffer in memory the other ranks can map; RTE_DP_COMM=nccl keeps the library all-reduce
        # (also what CPU / gloo process groups use).
        self._peer = self._grad_mem = None
        peer_comm = (self.world > 1 and dev.type == "cuda" and os.environ.get("RTE_DP_COMM", "peer") == "peer"
                     and hasattr(ops, "lib"))
        if peer_comm:
            from .peer_comm import PeerMemory
            # (128 more floats behind the gradients: the small vectors the step exchanges besides them)
            self._grad_mem = PeerMemory(ops, (max(total, 64) + 128) * 4)
            self.grad_flat = self._grad_mem.tensor(f32)[:max(total, 64)]
        else:
            self.grad_flat = torch.zeros(max(total, 64), dtype=f32, device=dev)
        self.grads = {n: self.grad_flat[offsets[n]: offsets[n] + self.params[n].numel()].view(self.params[n].shape)
                      for n in self.trainable}
        self._buckets: list[tuple[int, int]] = []                   # [start, end) element ranges of grad_flat
        self._bucket_of: dict[str, int] = {}
        self._bucket_pending: list[int] = []
        self._bucket_size: list[int] = []
        # Bucket size: 25 MB.  With an audited sample every bucket becomes complete only near the end of backward (the
        # replay contributes late to all of them), so the exchange is mostly exposed and few large exchanges beat many
        # small ones (2 ranks, c3: 25 MB 1.93 ms per step, 7 MB 2.16 ms, 2 MB 2.29 ms).  RTE_BUCKET_MB overrides.
        if bucket_cap_mb is None:
            bucket_cap_mb = float(os.environ.get("RTE_BUCKET_MB", 25.0))
        self.bucket_cap_mb = float(bucket_cap_mb)
        cap = max(int(bucket_cap_mb * 1024 * 1024 / 4), 1)
        start = 0
        # With an audited sample the gradients become final in three groups -- coda / final norm / macro operator once
        # the replay's head backward has been merged, the recurrent core (and router) when the replay leaves the core,
        # prelude and embedding at the last join -- so a bucket never straddles two of them.
        def ready_group(name: str) -> int:
            if not self.audit_grad:
                return 0
            return 1 if name.startswith(("core.", "router.")) else 2 if name.startswith(("prelude.", "embed.")) else 0

        prev_group = None
        for n in order:
            end = offsets[n] + -(-self.params[n].numel() // 64) * 64
            same_group, prev_group = ready_group(n) == prev_group, ready_group(n)
            if self._buckets and same_group and end - self._buckets[-1][0] <= cap:
                self._buckets[-1] = (self._buckets[-1][0], end)
            else:
                self._buckets.append((offsets[n], end))
            self._bucket_of[n] = len(self._buckets) - 1
        self._bucket_size = [sum(1 for n in order if self._bucket_of[n] == i) for i in range(len(self._buckets))]
        # (high priority: an exchange is short, sits on the step's critical path once backward has finished, and all of
        # its blocks must have run before it can tell the peers anything)
        comm_prio = int(os.environ.get("RTE_COMM_PRIORITY", "-1"))
        self._comm_stream = torch.cuda.Stream(device=dev, priority=comm_prio) if (self.world > 1 and dev.type == "cuda") else None
        if peer_comm:
            from .peer_comm import PeerAllReduce
            self._peer = PeerAllReduce(ops, self._grad_mem, process_group)
        self.exp_avg = {n: torch.zeros_like(self.params[n]) for n in self.trainable}
        self.exp_avg_sq = {n: torch.zeros_like(self.params[n]) for n in self.trainable}

        # ---- bf16 shadows of the GEMM weights (refreshed by the AdamW kernel)
        self.shadow: dict[str, torch.Tensor] = {}
        for n in names:
            if n == "embed.weight" or n.endswith((".attn.wqkv.weight", ".attn.wo.weight", ".mlp.wug.weight", ".mlp.wd.weight")):
                self.shadow[n] = torch.empty_like(self.params[n], dtype=bf)
        if self.audit_k or self.exact:
            from .audit import CORE_SHADOWED
            for n in CORE_SHADOWED:
                self.shadow[n] = torch.empty_like(self.params[n], dtype=bf)
        entries = [dict(p=self.params[n], g=self.grads[n], m=self.exp_avg[n], v=self.exp_avg_sq[n],
                        shadow=self.shadow.get(n), lr_group=LR_GROUPS.index(lr_group_of(n, cfg.topology)),
                        metric_group=metric_group_of(n, cfg.topology))
                   for n in self.trainable]
        self.plan = AdamWPlan(entries, len(LR_GROUPS), dev, n_metric_groups=len(METRIC_GROUPS))
        # Bernoulli sampler: on a step that audited nobody the recurrent core receives no gradient, and the reference's
        # optimiser then leaves it alone (`grad is None`: no decay, no moments, no step count).  `_core_absent` stays 1
        # while no micro-batch of the current accumulation cycle has audited anybody.
        self._core_absent = self._none_audited = self._absent_mask = None
        if self.audit_padded and self.audit_grad:
            from .audit import CORE_PARAMS
            self._core_absent = torch.ones(1, dtype=torch.int32, device=dev)
            self._none_audited = torch.zeros(1, dtype=torch.int32, device=dev)
            self._absent_mask = torch.tensor([1 if n in CORE_PARAMS else 0 for n in self.trainable], dtype=torch.uint8, device=dev)
        self._lr_stage = None                            # pinned staging of the per-step learning-rate table
        self._tokens_scheduled = 0                       # tokens of the steps submitted so far (LR schedule, all ranks)
        self._write_lr_table()
        self.skip_flag = torch.zeros(1, dtype=torch.int32, device=dev)      # set by the non-finite guard of a step
        self.accum_flat = torch.zeros_like(self.grad_flat) if self.accum > 1 else None
        self._refresh_static_param_sq()

        # ---- activations
        M, d, V, B, S = self.M, cfg.d_model, cfg.vocab_size, self.B, self.S
        e = lambda *shape, dtype=f32: torch.empty(*shape, dtype=dtype, device=dev)  # noqa: E731
        self.tokens = torch.zeros(B, S, dtype=torch.int64, device=dev)
        self.targets = torch.zeros(B, S, dtype=torch.int64, device=dev)
        self.embed_accum = torch.zeros(cfg.vocab_size * cfg.d_model, dtype=torch.int64, device=dev)   # embed_bwd scratch
        self.x0 = e(M, d)
        if self.dense:
            self.blocks = [_Block(f"blocks.{i}", M, cfg, B, S, dev) for i in range(cfg.n_dense_layers)]
            self.prelude, self.coda = self.blocks, []
        else:
            self.prelude = [_Block(f"prelude.{i}", M, cfg, B, S, dev) for i in range(cfg.n_prelude)]
            self.coda = [_Block(f"coda.{i}", M, cfg, B, S, dev) for i in range(cfg.n_coda)]
            self.blocks = self.prelude + self.coda
        self.hidden16, self.rstd_f = e(M, d, dtype=bf), e(M)
        self.logits = e(M, V, dtype=bf)
        # Everything the host reads back after a step lives in ONE buffer, so that it is one device-to-host copy:
        #   scalars[8] | loss_per_sample[B] | recipe_id[B] (int32) | audit terms[k,4] | audit exact_loss[k] | kl_sum[1]
        #   | per metric group (sum grad^2, sum param^2)
        k_a = self.audit_k or 0
        n_mg = len(METRIC_GROUPS)
        # (Bernoulli sampler, scheduled count: + audited sample ids[k] (int32) | 1 / inclusion probability[k] | sampler
        #  statistics[4];  every audit: + alignment sums[k,8] (macro.py:499-546)
        self._audit_extra = 8 * k_a + ((2 * k_a + 4) if self.audit_padded else 0)
        self._results = torch.zeros(8 + 2 * B + 5 * k_a + 1 + self._audit_extra + 2 * n_mg, dtype=f32, device=dev)
        self.loss_tok = e(M)
        # [0]=sum loss, [1]=aux load, [2]=aux depth, [3]=sumsq, [4]=clip, [5]=1.0 when the step was dropped (non-finite)
        self.scalars = self._results[0:8]
        self.loss_per_sample = self._results[8:8 + B]
        self._metric_sums = self._results[8 + 2 * B + 5 * k_a + 1 + self._audit_extra:].view(n_mg, 2)
        self.row_weight = torch.full((B,), 1.0 / (B * S * self.loss_div), dtype=f32, device=dev)
        # backward temporaries
        self.tmp = _Temps(M, cfg, dev)
        # Weight-gradient launches of the hot pass run on their own stream beside the data-gradient chain (they fill the
        # SMs that attention / norm / macro-operator kernels leave idle).  What they read must then outlive the chain's
        # reuse of scratch: every block gets its own scratch set and its own bf16 input-gradient buffer.
        self._hot_param_stream = torch.cuda.Stream(device=dev) if (dev.type == "cuda" and hasattr(ops, "param_stream")) else None
        # The parameter-gradient halves of the macro operator and of the router (long SIMT kernels) get a stream of
        # their own, so that the weight-gradient GEMMs keep following the data-gradient chain closely.
        self._misc_param_stream = (torch.cuda.Stream(device=dev)
                                   if (self._hot_param_stream is not None and not self.dense) else None)
        n_blocks = len(self.blocks) if self.dense else cfg.n_prelude + cfg.n_coda
        if self._hot_param_stream is not None:
            self.block_tmps = [self.tmp] + [_Temps(M, cfg, dev) for _ in range(n_blocks - 1)]
            self.grad16 = [self.tmp.dx16] + [torch.empty(M, d, dtype=bf, device=dev) for _ in range(n_blocks + 1)]
        else:
            self.block_tmps = [self.tmp] * n_blocks
            self.grad16 = [self.tmp.dx16] * (n_blocks + 2)
        t_ = self.tmp
        self.dug, self.dn16, self.dy16, self.dx16, self.dqkv = t_.dug, t_.dn16, t_.dy16, t_.dx16, t_.dqkv
        self.dxa, self.dxb, self.dxc, self.partial = t_.dxa, t_.dxb, t_.dxc, t_.partial
        self.partial_final = torch.empty_like(self.partial)     # the final norm's column partials (its reduction is deferred too)
        self.gn_partial = e(self.plan.total_chunks)
        max_ws = 0
        for (mm, nn) in ((3 * d, d), (d, d), (2 * cfg.d_ff, d), (d, cfg.d_ff), (V, d)):
            max_ws = max(max_ws, ops.pick_splits(mm, nn, M) * mm * nn)
        ops.split_workspace(max_ws)
        if not self.dense:
            r, k, m, hid = cfg.recipe_count, len(cfg.depth_choices), cfg.macro_rank, cfg.router_hidden_dim
            self.h_phi = e(M, d)
            self.phi_rstd, self.phi_pooled, self.phi_act = e(M), e(B * d + B * m), e(M, m)
            self.phi_scratch = e(ops.phi_bwd_scratch_floats(B, S, d, m))
            # transposed macro-operator weights for its tensor-core forward, refreshed every step (CudaOps only)
            self.phi_wt = (e(cfg.recipe_count * len(cfg.depth_choices) * 4 * d * m)
                           if hasattr(ops, "macro_phi_prepare") and dev.type == "cuda" else None)
            self._init_consistency(e)
            self.macro_scale = torch.ones(r, k, d, dtype=f32, device=dev)   # `update_scale` buffer (macro.py:99-108)
            self.macro_teacher_delta_rms = torch.zeros(r, k)               # carried through checkpoints only (macro.py:122)
            self.depth_values = torch.tensor(list(cfg.depth_choices), dtype=torch.int32, device=dev)
            i32 = torch.int32
            self.route = dict(pooled=e(B, d), r_hidden_pre=e(B, hid), d_hidden_pre=e(B, hid), recipe_logits=e(B, r),
                              recipe_probs=e(B, r), depth_probs=e(B, k), expected_depth=e(B), router_entropy=e(B),
                              recipe_id=self._results[8 + B:8 + 2 * B].view(i32), recipe_id_by_pass=e(B, cfg.t_max, dtype=i32),
                              depth_id=e(B, dtype=i32), depth=e(B, dtype=i32))
            self.router_scratch = e(A.ROUTER_MAX_R + B * (2 * hid + r + k + A.ROUTER_DPOOLED_PARTS * d) + 4)
            self._mean_prob = torch.zeros(A.ROUTER_MAX_R, dtype=f32, device=dev)
            if self._grad_mem is not None:              # exchanged by the peer kernel: lives in the shared allocation
                self._mean_prob_lo = self.grad_flat.numel() + 32         # (clear of the last bucket's staging overhang)
                self._mean_prob = self._grad_mem.tensor(f32)[self._mean_prob_lo:self._mean_prob_lo + A.ROUTER_MAX_R]
        if self.shortlist:
            oc, i32 = self.oc, torch.int32
            if "shortlist_head.cluster_router.weight" not in self.params:
                raise ValueError("recursive_macro_shortlist needs shortlist_head.cluster_router.weight")
            self.sl_tc = min(oc.shortlist_top_clusters, oc.num_clusters)
            self.cluster_w16 = torch.empty(oc.num_clusters, d, dtype=bf, device=dev)
            ops.cast_bf16(self.params["shortlist_head.cluster_router.weight"], self.cluster_w16)
            self.cluster_logits = e(M, oc.num_clusters)
            self.top_clusters = e(M, self.sl_tc, dtype=i32)
            self.random_negs = torch.zeros(M, max(oc.random_negatives, 1), dtype=i32, device=dev)
            self.shortlist_ids = e(M, oc.shortlist_max_tokens, dtype=i32)
            self.shortlist_dups = e(M, dtype=i32)
        self.audit = None
        # The replay is a long chain of small launches beside a hot pass that fills every SM: its stream gets the
        # higher priority and the persistent GEMM leaves a few SMs free, so a replay kernel never waits for a whole
        # hot-pass kernel to drain (measured: -2.5 % step time).
        self._side_stream = torch.cuda.Stream(device=dev, priority=-1) if (self.audit_k and dev.type == "cuda") else None
        if self._side_stream is not None and hasattr(ops, "gemm_max_ctas"):
            ops.gemm_max_ctas = max(ops.sm_count - int(os.environ.get("RTE_SIDE_SMS", "8")), 1)
        self._param_stream = torch.cuda.Stream(device=dev) if (self.audit_k and dev.type == "cuda") else None
        self._merge_stream = torch.cuda.Stream(device=dev) if (self.audit_k and dev.type == "cuda") else None
        self.exact_core = None
        if self.exact:
            from .audit import AuditReplay
            self.exact_core = AuditReplay(self, B, direct_grads=True)         # the replay machinery over the whole batch
            self.exact_core.idx.copy_(torch.arange(B, dtype=torch.int32))
            if self.deferred:
                # models.py:551-566: one recipe per branch of the grouped block -- `fixed_recipe` (default 1) repeated
                # `fixed_depth` (default t_max) times, or the head of `fixed_recipe_schedule` with its last entry repeated
                depth = max(1, min(int(tr.fixed_depth or cfg.t_max), cfg.t_max))
                first = int(tr.fixed_recipe if tr.fixed_recipe is not None else 1)
                sched = [int(r) for r in (tr.fixed_recipe_schedule or [])][:depth] or [first]
                if tr.fixed_recipe_schedule is None:
                    sched = [first] * depth
                sched += [sched[-1]] * (depth - len(sched))
                if any(not 0 <= r < cfg.recipe_count for r in sched):
                    raise ValueError(f"deferred grouped recipe outside [0, {cfg.recipe_count})")
                self.exact_schedule = sched
                self.exact_core.deferred_depth = depth
                self.exact_core.fixed_rid = (torch.tensor(sched + [0] * (cfg.t_max - depth), dtype=torch.int32).view(-1, 1)
                                             .expand(cfg.t_max, B).contiguous().to(dev))
            elif tr.fixed_recipe_schedule is not None:
                # models.py:230-247, 449-451: pass t runs recipe schedule[t] for every sample, whatever the router chose
                sched = [int(r) for r in tr.fixed_recipe_schedule]
                if len(sched) < cfg.t_max:
                    raise ValueError(f"fixed_recipe_schedule length {len(sched)} is shorter than t_max={cfg.t_max}")
                if any(not 0 <= r < cfg.recipe_count for r in sched):
                    raise ValueError(f"fixed_recipe_schedule recipe outside [0, {cfg.recipe_count})")
                self.exact_schedule = sched[:cfg.t_max]
                self.exact_core.fixed_rid = (torch.tensor(self.exact_schedule, dtype=torch.int32).view(-1, 1)
                                             .expand(cfg.t_max, B).contiguous().to(dev))
        if self.audit_k:
            from .audit import AuditReplay
            self.audit = AuditReplay(self, self.audit_k)
            r0, k_a = 8 + 2 * B, self.audit_k
            self.audit.terms = self._results[r0:r0 + 4 * k_a].view(k_a, 4)
            self.audit.exact_loss = self._results[r0 + 4 * k_a:r0 + 5 * k_a]
            self.audit.kl_sum = self._results[r0 + 5 * k_a:r0 + 5 * k_a + 1]
            self.audit.align = self._results[r0 + 5 * k_a + 1:r0 + 13 * k_a + 1].view(k_a, 8)
            if self.audit_padded:
                x0 = r0 + 13 * k_a + 1
                self.audit.sampler_block = self._results[x0:x0 + 2 * k_a + 4]       # the three views below, contiguous
                self.audit.idx = self._results[x0:x0 + k_a].view(torch.int32)
                self.audit.inv_p = self._results[x0 + k_a:x0 + 2 * k_a]
                self.audit.stats = self._results[x0 + 2 * k_a:x0 + 2 * k_a + 4]
        for n, sh in self.shadow.items():
            ops.cast_bf16(self.params[n], sh)
        if hasattr(ops, "rope_table"):
            ops.rope_table(S, cfg.head_dim)          # built once, before any stream capture
        # the hot-path budget depends on the configuration only: checked once, before anything runs (training.py:1389-1392)
        self._budget = {} if (self.dense or self.exact) else hot_budget(cfg, tr, self.oc.shortlist_max_tokens if self.shortlist else None)
        self._graphs: dict[str, Any] = {}                  # captured step graphs: "step" (with optimiser), "micro"
        self._host: dict[str, Any] | None = None           # results of the step collected last
        self._host_slots = None
        self._slot_next = 0
        self._pending: list[dict[str, Any]] = []
        self._launches_per_step: int | None = None

    # ------------------------------------------------------------------ data-parallel gradient exchange
    def _grad_completion_order(self) -> list[str]:
        """Trainable parameter names in the order `_forward_backward` finishes their gradients."""
        cfg = self.cfg

        def block(prefix: str) -> list[str]:
            return [f"{prefix}.mlp.wd.weight", f"{prefix}.mlp.wug.weight", f"{prefix}.norm2.weight",
                    f"{prefix}.attn.wo.weight", f"{prefix}.attn.wqkv.weight", f"{prefix}.norm1.weight"]

        order = ["final_norm.weight"]
        if self.dense:
            for i in reversed(range(cfg.n_dense_layers)):
                order += block(f"blocks.{i}")
        else:
            for i in reversed(range(cfg.n_coda)):
                order += block(f"coda.{i}")
            if not self.exact:
                order += ["macro.d_gain", "macro.v", "macro.u", "macro.bias"]
            if self.audit_grad or self.exact:
                from .audit import CORE_PARAMS
                order += CORE_PARAMS
            if not self.tr.disable_router_aux:
                for mlp in ("recipe_mlp", "depth_mlp"):
                    order += [f"router.{mlp}.0.weight", f"router.{mlp}.0.bias", f"router.{mlp}.2.weight", f"router.{mlp}.2.bias"]
            for i in reversed(range(cfg.n_prelude)):
                order += block(f"prelude.{i}")
        return order + ["embed.weight"]

    def _begin_backward(self) -> None:
        self._bucket_pending = list(self._bucket_size)
        self._ready_events: list = []

    def _grad_ready(self, *names: str, after=None) -> None:
        """Marks gradients as final; a bucket whose last gradient arrived is summed across ranks on the
        communication stream (NCCL over NVLink) while the compute stream carries on with backward.
        `after`: an event (recorded on another stream) that these gradients additionally depend on."""
        if self.world == 1 or self._dp_paused:
            return
        import torch.distributed as dist
        if after is not None:
            self._ready_events.append(after)      # every later bucket launch of this step waits for it too (cheap, monotone)
        for n in names:
            i = self._bucket_of[n]
            self._bucket_pending[i] -= 1
            if self._bucket_pending[i] == 0:
                lo, hi = self._buckets[i]
                view = self.grad_flat[lo:hi]
                if self._comm_stream is None:
                    dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.pg)
                else:
                    self._comm_stream.wait_stream(torch.cuda.current_stream(self.device))
                    for ev in self._ready_events:
                        self._comm_stream.wait_event(ev)
                    if self._hot_param_stream is not None:       # weight gradients are produced there
                        self._comm_stream.wait_stream(self._hot_param_stream)
                    if self._misc_param_stream is not None:
                        self._comm_stream.wait_stream(self._misc_param_stream)
                    with torch.cuda.stream(self._comm_stream):
                        probes = getattr(self, "_dp_probes", None)       # optional: event pairs around every exchange
                        if probes is not None:
                            e0 = torch.cuda.Event(enable_timing=True, external=True)
                            e0.record(self._comm_stream)
                        if self._peer is not None:
                            self._peer.all_reduce_(lo, hi, slot=i % (A.COMM_MAX_SLOTS - 1))     # the last slot: the router's vector
                        else:
                            dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.pg)
                        if probes is not None:
                            e1 = torch.cuda.Event(enable_timing=True, external=True)
                            e1.record(self._comm_stream)
                            probes.append((f"bucket{i}", (hi - lo) * 4, e0, e1))

    def _global_mean_prob(self):
        """Under data parallelism: the recipe probabilities' mean over the GLOBAL batch (R floats summed across the
        ranks on the current stream), which the load-balance loss squares (metrics.py:103-105); None on one rank."""
        if self.world == 1 or self._dp_paused:
            return None
        import torch.distributed as dist
        R = self.cfg.recipe_count
        self.ops.router_mean_prob(self.route["recipe_probs"], self._mean_prob, 1.0 / (self.B * self.world), B=self.B, R=R)
        if self._peer is not None:
            self._peer.all_reduce_(self._mean_prob_lo, self._mean_prob_lo + A.ROUTER_MAX_R, slot=A.COMM_MAX_SLOTS - 1)
        else:
            dist.all_reduce(self._mean_prob, op=dist.ReduceOp.SUM, group=self.pg)
        return self._mean_prob

    def _finish_backward(self) -> None:
        if self._comm_stream is not None and not self._dp_paused:
            torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)

    # ------------------------------------------------------------------ side stream of the audit replay
    def _on_side(self):
        import contextlib
        if self._side_stream is None:
            return contextlib.nullcontext()
        return torch.cuda.stream(self._side_stream)

    def _side_wait_main(self) -> None:
        if self._side_stream is not None:
            self._side_stream.wait_stream(torch.cuda.current_stream(self.device))

    def _side_event(self):
        """An event at the current end of the replay's stream (None without one: single-stream order then holds)."""
        if self._side_stream is None:
            return None
        ev = torch.cuda.Event()
        ev.record(self._side_stream)
        return ev

    def _main_wait_side(self, event=None) -> None:
        """The hot pass waits for the replay's stream (or only for `event` recorded on it)."""
        if self._side_stream is None:
            return
        main = torch.cuda.current_stream(self.device)
        probes = getattr(self, "_join_probes", None)        # optional: event pairs that time how long the hot pass idles here
        if probes is not None:
            e0 = torch.cuda.Event(enable_timing=True, external=True)
            e0.record(main)
        if event is not None:
            main.wait_event(event)
        else:
            main.wait_stream(self._side_stream)
        if probes is not None:
            e1 = torch.cuda.Event(enable_timing=True, external=True)
            e1.record(main)
            probes.append(("wait", e0, e1))

    # ------------------------------------------------------------------ small helpers
    def _write_lr_table(self, scale: float = 1.0) -> None:
        """Per-group learning rates x the schedule's factor -> the device table the AdamW kernel reads.  Per step the
        values go through pinned staging (three buffers in rotation, as many as steps can be in flight plus one), so the
        copy is stream-ordered in front of the step that uses it."""
        lrs = torch.tensor([self.tr.lr_for(g) * scale for g in LR_GROUPS], dtype=torch.float32)
        self._lr_now = {g: float(v) for g, v in zip(LR_GROUPS, lrs)}
        if self._lr_stage is None:
            pin = self.device.type == "cuda"
            self._lr_stage = [torch.empty(len(LR_GROUPS), dtype=torch.float32, pin_memory=pin) for _ in range(3)]
            self._lr_stage_next = 0
        h = self._lr_stage[self._lr_stage_next]
        self._lr_stage_next = (self._lr_stage_next + 1) % 3
        h.copy_(lrs)
        self.plan.lr_table.copy_(h, non_blocking=True)

    def _refresh_static_param_sq(self) -> None:
        """Sum of squares, per metric group, of the parameters the optimiser never touches in this mode (they count
        towards the reference's per-group parameter norms, training.py:386-443, and only change on a checkpoint load)."""
        out = [0.0] * len(METRIC_GROUPS)
        for n, p in self.params.items():
            if n not in self.trainable and not n.startswith("shortlist_head."):
                out[metric_group_of(n, self.cfg.topology)] += float(p.double().pow(2).sum())
        self._static_param_sq = out

    def _router_weight_dict(self) -> dict[str, torch.Tensor]:
        p = self.params
        return dict(r_w0=p["router.recipe_mlp.0.weight"], r_b0=p["router.recipe_mlp.0.bias"],
                    r_w2=p["router.recipe_mlp.2.weight"], r_b2=p["router.recipe_mlp.2.bias"],
                    d_w0=p["router.depth_mlp.0.weight"], d_b0=p["router.depth_mlp.0.bias"],
                    d_w2=p["router.depth_mlp.2.weight"], d_b2=p["router.depth_mlp.2.bias"],
                    pass_recipe_bias=p["router.pass_recipe_bias"])

    # ------------------------------------------------------------------ macro consistency term
    def _init_consistency(self, e) -> None:
        """Buffers of the consistency term lambda_cons * mse(Phi_2k(h0, h0), Phi_k(Phi_k(h0, h0), h0)) over the stride pairs
        (k, 2k) of the depth choices (macro.py:126,342-359; added on every step of the macro modes, audit.py:370-379)."""
        cfg, tr, dev = self.cfg, self.tr, self.device
        strides = list(cfg.depth_choices)
        self.cons_pairs = ([(i, strides.index(v * 2)) for i, v in enumerate(strides) if v * 2 in strides]
                           if (tr.lambda_cons != 0.0 and not self.exact) else [])
        self._cons_stream = None
        if not self.cons_pairs:
            return
        B, M, d, m = self.B, self.M, cfg.d_model, cfg.macro_rank
        i32 = torch.int32
        self.cons_src = [torch.full((B,), a, dtype=i32, device=dev) for a, _ in self.cons_pairs]
        self.cons_dst = [torch.full((B,), c, dtype=i32, device=dev) for _, c in self.cons_pairs]
        self.cons_out = [e(M, d) for _ in range(3)]                       # direct, mid, twice
        self.cons_saved = [(e(M), e(B * d + B * m), e(M, m)) for _ in range(3)]          # rstd, pooled(+pa), act of each
        self.cons_g, self.cons_gneg = e(M, d), e(M, d)                    # coef * (direct - twice) and its negative
        self.cons_dmid, self.cons_dh, self.cons_dh0 = e(M, d), e(M, d), e(M, d)
        self.cons_scratch = e(self.ops.phi_bwd_scratch_floats(B, self.S, d, m))
        self.cons_partial = e(1024)
        # parameter gradients of the term: a mirror of the macro operator's slice of the flat gradient buffer (same
        # relative offsets, so one add merges it) plus a scratch mirror each backward overwrites
        names = ["macro.d_gain", "macro.v", "macro.u", "macro.bias"]
        lo = min(self._grad_offsets[n] for n in names)
        hi = max(self._grad_offsets[n] + -(-self.params[n].numel() // 64) * 64 for n in names)
        self.cons_range = (lo, hi)
        self.cons_pg_flat, self.cons_pg_tmp_flat = e(hi - lo), e(hi - lo)

        def views(flat):
            return {n.split(".")[1].replace("d_gain", "gain"): flat[self._grad_offsets[n] - lo: self._grad_offsets[n] - lo + self.params[n].numel()]
                    .view(self.params[n].shape) for n in names}
        self.cons_pg_tmp = views(self.cons_pg_tmp_flat)
        if dev.type == "cuda":
            self._cons_stream = torch.cuda.Stream(device=dev)

    def _consistency_branch(self, h0: torch.Tensor):
        """Forward and backward of the consistency term, on its own stream beside the rest of the step: needs h0, the
        routed recipe ids and the prepared macro weights; leaves d h0 in `cons_dh0`, the parameter gradients in
        `cons_pg_flat`, the summed squared difference in scalars[6].  Returns the event that marks them complete."""
        o, cfg, tr = self.ops, self.cfg, self.tr
        B, S, M, d, m = self.B, self.S, self.M, cfg.d_model, cfg.macro_rank
        R, K, P = cfg.recipe_count, len(cfg.depth_choices), len(self.cons_pairs)
        dims = dict(B=B, S=S, d=d, m=m, K=K)
        pd, rid, s_cfg = self._phi_param_dict(), self.route["recipe_id"], cfg.macro_update_scale
        coef = 2.0 * tr.lambda_cons / (P * M * d * self.loss_div)           # d(lambda * mse)/d direct, this rank's share
        cs = self._cons_stream
        if cs is not None:
            cs.wait_stream(torch.cuda.current_stream(self.device))
        ctx = torch.cuda.stream(cs) if cs is not None else contextlib.nullcontext()
        with ctx:
            o.fill_(self.cons_dh0, 0.0)
            o.fill_(self.cons_pg_flat, 0.0)
            direct, mid, twice = self.cons_out
            (r_d, p_d, a_d), (r_m, p_m, a_m), (r_t, p_t, a_t) = self.cons_saved
            for i in range(P):
                src, dst = self.cons_src[i], self.cons_dst[i]
                o.macro_phi_fwd(h0, pd, rid, dst, s_cfg, direct, r_d, p_d, a_d, **dims)
                o.macro_phi_fwd(h0, pd, rid, src, s_cfg, mid, r_m, p_m, a_m, **dims)
                o.macro_phi_fwd_hx(mid, h0, pd, rid, src, s_cfg, twice, r_t, p_t, a_t, **dims)
                o.sqdiff_grad(direct, twice, coef, self.cons_g, self.cons_partial, self.scalars[6:7], accumulate=i > 0)
                o.sqdiff_grad(twice, direct, coef, self.cons_gneg, self.cons_partial, self.scalars[7:8], accumulate=False)
                # d twice = -g: through Phi_k(mid, h0) into mid and h0 ...
                o.macro_phi_bwd_hx(mid, h0, self.cons_gneg, pd, rid, src, s_cfg, r_t, p_t, a_t, self.cons_dmid, self.cons_dh0,
                                   self.cons_pg_tmp, self.cons_scratch, R=R, **dims)
                o.add_(self.cons_pg_flat, self.cons_pg_tmp_flat)
                # ... d mid through Phi_k(h0, h0) ...
                o.macro_phi_bwd(h0, self.cons_dmid, pd, rid, src, s_cfg, r_m, p_m, a_m, self.cons_dh, self.cons_pg_tmp,
                                self.cons_scratch, R=R, **dims)
                o.add_(self.cons_dh0, self.cons_dh)
                o.add_(self.cons_pg_flat, self.cons_pg_tmp_flat)
                # ... and d direct = +g through Phi_2k(h0, h0)
                o.macro_phi_bwd(h0, self.cons_g, pd, rid, dst, s_cfg, r_d, p_d, a_d, self.cons_dh, self.cons_pg_tmp,
                                self.cons_scratch, R=R, **dims)
                o.add_(self.cons_dh0, self.cons_dh)
                o.add_(self.cons_pg_flat, self.cons_pg_tmp_flat)
            done = None
            if cs is not None:
                done = torch.cuda.Event()
                done.record(cs)
        return done

    def _phi_param_dict(self) -> dict[str, torch.Tensor]:
        p = self.params
        return dict(gain=p["macro.d_gain"], v=p["macro.v"], u=p["macro.u"], bias=p["macro.bias"], scale=self.macro_scale,
                    wt=getattr(self, "phi_wt", None))

    # ------------------------------------------------------------------ one transformer block
    def _router_grad_dict(self) -> dict[str, torch.Tensor]:
        g = self.grads
        return dict(r_w0=g["router.recipe_mlp.0.weight"], r_b0=g["router.recipe_mlp.0.bias"],
                    r_w2=g["router.recipe_mlp.2.weight"], r_b2=g["router.recipe_mlp.2.bias"],
                    d_w0=g["router.depth_mlp.0.weight"], d_b0=g["router.depth_mlp.0.bias"],
                    d_w2=g["router.depth_mlp.2.weight"], d_b2=g["router.depth_mlp.2.bias"])

    @staticmethod
    def _router_grad_names() -> list[str]:
        return [f"router.{m}.{i}.{k}" for m in ("recipe_mlp", "depth_mlp") for i in (0, 2) for k in ("weight", "bias")]

    def _fuse_swiglu(self, rows: int) -> bool:
        """SwiGLU inside the tcgen05 GEMM's epilogue only between the few-row kernel's range and the large-M range."""
        return getattr(self.ops, "small_gemm_rows", 0) < rows <= self.swiglu_fuse_max_rows

    def _block_fwd(self, blk: _Block, x_in: torch.Tensor) -> torch.Tensor:
        o, cfg, p, sh, M = self.ops, self.cfg, self.params, self.shadow, blk.M
        d, f, pre = cfg.d_model, cfg.d_ff, blk.prefix.split("@")[0]
        blk.x_in = x_in
        o.rmsnorm_fwd(x_in, p[f"{pre}.norm1.weight"], blk.n1, blk.rstd1)
        o.gemm(blk.n1, sh[f"{pre}.attn.wqkv.weight"], blk.qkv, M=M, N=3 * d, K=d)
        o.attn_fwd(blk.qkv, blk.y, blk.lse, B=blk.B, S=blk.S, n_heads=cfg.n_heads, head_dim=cfg.head_dim)
        o.gemm(blk.y, sh[f"{pre}.attn.wo.weight"], blk.u, M=M, N=d, K=d, epilogue=A.EPI_F32, residual=x_in)
        o.rmsnorm_fwd(blk.u, p[f"{pre}.norm2.weight"], blk.n2, blk.rstd2)
        if self._fuse_swiglu(M):
            o.gemm(blk.n2, sh[f"{pre}.mlp.wug.weight"], blk.z, M=M, N=2 * f, K=d, epilogue=A.EPI_SWIGLU_FWD, out2=blk.ug, pair=f)
        else:       # at large M the plain-store GEMM plus one vectorised pass beats the fused epilogue (measured);
                    # with few rows the plain-store product runs in the few-row kernel, which has no such epilogue
            o.gemm(blk.n2, sh[f"{pre}.mlp.wug.weight"], blk.ug, M=M, N=2 * f, K=d)
            o.swiglu_fwd(blk.ug, blk.z, M, f)
        o.gemm(blk.z, sh[f"{pre}.mlp.wd.weight"], blk.out, M=M, N=d, K=f, epilogue=A.EPI_F32, residual=blk.u)
        return blk.out

    def _block_bwd(self, blk: _Block, dout: torch.Tensor, dout16: torch.Tensor, dx: torch.Tensor,
                   dx16: torch.Tensor | None, du: torch.Tensor, tmp: "_Temps | None" = None,
                   accumulate: bool = False, mark_ready: bool = True, grads: dict | None = None, ws=None) -> None:
        """dout/dout16: gradient wrt the block output (f32 and its bf16 copy); writes dx (f32) and dx16.
        `accumulate` adds the weight gradients to what is already there (second pass over shared weights)."""
        o, cfg, p, sh, M = self.ops, self.cfg, self.params, self.shadow, blk.M
        g = grads if grads is not None else self.grads
        t = tmp if tmp is not None else self.tmp
        d, f, pre = cfg.d_model, cfg.d_ff, blk.prefix.split("@")[0]
        ready = self._grad_ready if mark_ready else (lambda *names: None)
        # --- MLP: x_out = u + wd(up * silu(gate)),  (up | gate) = wug(norm2(u))
        if self._fuse_swiglu(M):
            o.gemm(dout16, sh[f"{pre}.mlp.wd.weight"], t.dug, M=M, N=f, K=d, b_mn=True, epilogue=A.EPI_SWIGLU_BWD,
                   residual=blk.ug, pair=f)
        else:
            o.gemm(dout16, sh[f"{pre}.mlp.wd.weight"], t.dz16, M=M, N=f, K=d, b_mn=True)
            o.swiglu_bwd(blk.ug, t.dz16, t.dug, M, f)
        o.gemm_wgrad(dout16, blk.z, g[f"{pre}.mlp.wd.weight"], M=d, N=f, K=M, accumulate=accumulate, ws=ws)
        ready(f"{pre}.mlp.wd.weight")
        o.gemm(t.dug, sh[f"{pre}.mlp.wug.weight"], t.dn16, M=M, N=d, K=2 * f, b_mn=True)
        o.gemm_wgrad(t.dug, blk.n2, g[f"{pre}.mlp.wug.weight"], M=2 * f, N=d, K=M, accumulate=accumulate, ws=ws)
        ready(f"{pre}.mlp.wug.weight")
        o.rmsnorm_bwd(blk.u, p[f"{pre}.norm2.weight"], blk.rstd2, t.dn16, dout, du, t.dy16,
                      g[f"{pre}.norm2.weight"], t.partial, accumulate_dw=accumulate)
        ready(f"{pre}.norm2.weight")
        du16 = t.dy16
        # --- attention: u = x + wo(attn(rope(q), rope(k), v)),  (q | k | v) = wqkv(norm1(x))
        o.gemm(du16, sh[f"{pre}.attn.wo.weight"], t.dn16, M=M, N=d, K=d, b_mn=True)
        o.gemm_wgrad(du16, blk.y, g[f"{pre}.attn.wo.weight"], M=d, N=d, K=M, accumulate=accumulate, ws=ws)
        ready(f"{pre}.attn.wo.weight")
        o.attn_bwd(blk.qkv, blk.y, t.dn16, blk.lse, t.dqkv, B=blk.B, S=blk.S, n_heads=cfg.n_heads,
                   head_dim=cfg.head_dim)
        o.gemm(t.dqkv, sh[f"{pre}.attn.wqkv.weight"], t.dn16, M=M, N=d, K=3 * d, b_mn=True)
        o.gemm_wgrad(t.dqkv, blk.n1, g[f"{pre}.attn.wqkv.weight"], M=3 * d, N=d, K=M, accumulate=accumulate, ws=ws)
        ready(f"{pre}.attn.wqkv.weight")
        o.rmsnorm_bwd(blk.x_in, p[f"{pre}.norm1.weight"], blk.rstd1, t.dn16, du, dx, dx16,
                      g[f"{pre}.norm1.weight"], t.partial2, accumulate_dw=accumulate)
        ready(f"{pre}.norm1.weight")

    # ------------------------------------------------------------------ forward + backward
    def _forward_backward_exact(self, forward_only: bool = False) -> None:
        """`recursive_exact`: embed -> prelude -> router -> t_max banked passes for every sample -> coda -> logits ->
        cross entropy (models.py:202-228, 416-512), then the same chain backwards; one stream."""
        o, cfg, p, g, tr, a = self.ops, self.cfg, self.params, self.grads, self.tr, self.exact_core
        M, d, B, S = self.M, cfg.d_model, self.B, self.S
        tokens = self.tokens.view(-1)
        o.embed_fwd(tokens, p["embed.weight"], self.x0)
        x = self.x0
        for blk in self.prelude:
            x = self._block_fwd(blk, x)
        h0 = x
        fixed_depth_id = None if tr.fixed_depth is None else list(cfg.depth_choices).index(tr.fixed_depth)
        o.router_fwd(h0, self._router_weight_dict(), self.depth_values, self.route, B=B, S=S, d=d,
                     hid=cfg.router_hidden_dim, R=cfg.recipe_count, K=len(cfg.depth_choices), T=cfg.t_max,
                     fixed_recipe=tr.fixed_recipe, fixed_depth_id=fixed_depth_id)
        if self.deferred:
            a.forward_deferred(h0)
        else:
            a.forward_replay(h0)
        o.ce_fwd_bwd(a.logits, a.targets_a, a.row_weight_a, S, a.loss_tok, a.logits)
        o.segment_sum(a.loss_tok, self.loss_per_sample, B, S)
        o.segment_sum(self.loss_per_sample, self.scalars[0:1], 1, B)
        if forward_only:
            return
        # ---------------- backward
        self._begin_backward()
        if self.deferred:
            a.backward_deferred(a.backward_head())
        else:
            a.backward_core(a.backward_head())
        dcur, dalt = a.dh0_acc, self.dxb
        o.add_(dcur, a.dh_first)                          # d h0 = through the alpha*h0 injections + through h[0]
        if not tr.disable_router_aux:
            rg = {f"{m_[0]}_{k_}": g[f"router.{m_}.{i_}.{w_}"] for m_ in ("recipe_mlp", "depth_mlp")
                  for i_, w_, k_ in ((0, "weight", "w0"), (0, "bias", "b0"), (2, "weight", "w2"), (2, "bias", "b2"))}
            o.router_aux_bwd(self._router_weight_dict(), self.route, self.depth_values, tr.lambda_load / self.loss_div,
                             tr.lambda_depth / self.loss_div, self.scalars[1:3], rg, dcur, self.router_scratch, B=B, S=S,
                             d=d, hid=cfg.router_hidden_dim, R=cfg.recipe_count, K=len(cfg.depth_choices),
                             mean_prob=self._global_mean_prob())
        g16 = self.grad16
        o.cast_bf16(dcur, g16[0])
        for j, blk in enumerate(reversed(self.prelude)):
            self._block_bwd(blk, dcur, g16[j], dalt, g16[j + 1], self.dxc, tmp=self.block_tmps[j], mark_ready=False)
            dcur, dalt = dalt, dcur
        o.embed_bwd(tokens, dcur, g["embed.weight"], self.embed_accum)
        self._grad_ready(*self.trainable)
        self._finish_backward()

    def _forward_backward(self, forward_only: bool = False) -> None:
        """`forward_only` (evaluation): stops after the per-sample losses; the caller switches the audit replay off."""
        if self.exact:
            return self._forward_backward_exact(forward_only)
        o, cfg, p, sh, g, tr = self.ops, self.cfg, self.params, self.shadow, self.grads, self.tr
        M, d, V, B, S = self.M, cfg.d_model, cfg.vocab_size, self.B, self.S
        tokens, targets = self.tokens.view(-1), self.targets.view(-1)
        # ---------------- forward
        o.embed_fwd(tokens, p["embed.weight"], self.x0)
        x = self.x0
        for blk in self.prelude:
            x = self._block_fwd(blk, x)
        if not self.dense:
            h0 = x
            fixed_depth_id = None if tr.fixed_depth is None else list(cfg.depth_choices).index(tr.fixed_depth)
            if self.audit is not None and not self.audit.bernoulli:
                if self.audit.own_prelude:
                    # copies of the prelude's saved activations for the audited samples (read by the replay's own
                    # prelude backward, much later): on the replay's weight-gradient stream, idle during forward
                    ps = self._param_stream
                    if ps is not None:
                        ps.wait_stream(torch.cuda.current_stream(self.device))
                        with torch.cuda.stream(ps):
                            self.audit.gather_prelude()
                    else:
                        self.audit.gather_prelude()
                # the replay's first launches need h0 only: they run beside the router
                self._side_wait_main()
                with self._on_side():
                    self.audit.forward_replay_head(h0)
                if self.audit.scheduled and self._core_absent is not None:
                    self._core_absent.mul_(self._none_audited)      # (a schedule whose minimum is 0 can stop auditing)
            o.router_fwd(h0, self._router_weight_dict(), self.depth_values, self.route, B=B, S=S, d=d,
                         hid=cfg.router_hidden_dim, R=cfg.recipe_count, K=len(cfg.depth_choices), T=cfg.t_max,
                         fixed_recipe=tr.fixed_recipe, fixed_depth_id=fixed_depth_id)
            self._router_early = None
            if not tr.disable_router_aux and self._misc_param_stream is not None and self._hot_param_stream is not None:
                # The auxiliary losses' backward needs no upstream gradient: all of it except the add into d h0 runs
                # here, on the parameter-gradient stream, beside the rest of the forward pass.
                ms = self._misc_param_stream
                ms.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(ms):
                    o.router_aux_bwd_early(self._router_weight_dict(), self.route, self.depth_values, tr.lambda_load / self.loss_div,
                                           tr.lambda_depth / self.loss_div, self.scalars[1:3], self._router_grad_dict(),
                                           self.router_scratch, B=B, S=S, d=d, hid=cfg.router_hidden_dim,
                                           R=cfg.recipe_count, K=len(cfg.depth_choices), mean_prob=self._global_mean_prob())
                    self._router_early = torch.cuda.Event()
                    self._router_early.record(ms)
            if self.audit is not None and self.audit.bernoulli and not forward_only:
                # the subset is drawn from this step's routing (entropy, recipes): sampler first, then what the
                # fixed-count path had started before the router
                self.audit.sample()
                ps = self._param_stream
                if self.audit.own_prelude and ps is not None:
                    ps.wait_stream(torch.cuda.current_stream(self.device))
                    with torch.cuda.stream(ps):
                        self.audit.gather_prelude()
                elif self.audit.own_prelude:
                    self.audit.gather_prelude()
                self._side_wait_main()
                with self._on_side():
                    self.audit.forward_replay_head(h0)
            if self.audit is not None:
                # exact replay of the audited samples: needs only h0 and the routing, so it runs beside the macro
                # operator and the rest of the hot pass
                self._side_wait_main()
                with self._on_side():
                    self.audit.forward_replay(h0, head_done=True)
            if self.phi_wt is not None:
                o.macro_phi_prepare(self._phi_param_dict())
            self._cons_done, self._cons_pending = None, False
            if self.cons_pairs and not forward_only:
                self._cons_done, self._cons_pending = self._consistency_branch(h0), True
            o.macro_phi_fwd(h0, self._phi_param_dict(), self.route["recipe_id"], self.route["depth_id"],
                            cfg.macro_update_scale, self.h_phi, self.phi_rstd, self.phi_pooled, self.phi_act,
                            B=B, S=S, d=d, m=cfg.macro_rank, K=len(cfg.depth_choices))
            x = self.h_phi
            if self.audit is not None:
                self.audit.forward_distill(self.h_phi)           # (picks its stream itself)
            for blk in self.coda:
                x = self._block_fwd(blk, x)
        x_last = x
        o.rmsnorm_fwd(x_last, p["final_norm.weight"], self.hidden16, self.rstd_f)
        if self.shortlist:
            # cluster router -> top clusters -> shortlist -> gathered-row logits + CE (output.py:72-136); the gradient
            # comes back as a dense, otherwise-zero [M, V] row block so that backward is the full-vocabulary one
            oc = self.oc
            o.gemm(self.hidden16, self.cluster_w16, self.cluster_logits, M=M, N=oc.num_clusters, K=d, epilogue=A.EPI_F32)
            o.topk_lowest_index(self.cluster_logits, self.sl_tc, self.top_clusters)
            o.shortlist_build(targets, self.top_clusters, self.random_negs, self.shortlist_ids, self.shortlist_dups,
                              V=V, C=oc.num_clusters, TC=self.sl_tc, HN=oc.hard_negatives, RN=oc.random_negatives,
                              K=oc.shortlist_max_tokens)
            if V <= 240 * oc.shortlist_max_tokens:
                # small vocabulary: all V dot products as one tensor-core GEMM (2*d*V FLOP per token at ~1 PFLOP/s) cost
                # less than gathering K weight rows per token from L2 (K*d*2 bytes at a few TB/s); same bf16 logits
                o.gemm(self.hidden16, sh["embed.weight"], self.logits, M=M, N=V, K=d)
                o.shortlist_ce_from_logits(self.logits, self.shortlist_ids, self.row_weight, S, self.loss_tok)
            else:
                o.shortlist_ce(self.hidden16, sh["embed.weight"], self.shortlist_ids, self.row_weight, S, self.loss_tok, None,
                               self.logits)
        else:
            o.gemm(self.hidden16, sh["embed.weight"], self.logits, M=M, N=V, K=d)
            if self.audit is not None:
                self.audit.save_hot_logits()
                fwd_probe = getattr(self, "_fwd_probe", None)       # optional: (end of the replay's forward, hot logits ready)
                if fwd_probe is not None and self._side_stream is not None:
                    pe = (torch.cuda.Event(enable_timing=True, external=True), torch.cuda.Event(enable_timing=True, external=True))
                    pe[0].record(self._side_stream)
                    pe[1].record(torch.cuda.current_stream(self.device))
                    fwd_probe.append(pe)
                # the replay's KL term needs the saved hot logits only: it runs beside the hot cross entropy
                self._side_wait_main()
                with self._on_side():
                    self.audit.forward_kl()
                    kl_done = self._side_event()
                    self.audit.report()
            o.ce_fwd_bwd(self.logits, targets, self.row_weight, S, self.loss_tok, self.logits)   # logits -> dlogits in place
        o.segment_sum(self.loss_tok, self.loss_per_sample, B, S)
        o.segment_sum(self.loss_per_sample, self.scalars[0:1], 1, B)
        if forward_only:
            return
        if self.audit is not None:
            if self.shortlist:
                self._side_wait_main()
                with self._on_side():
                    kl_done = self._side_event()
                    self.audit.report()
            # join: the hot backward needs the distillation gradients (KL rows of dlogits, endpoint terms), not the
            # replay's own cross entropy, which starts the replay's backward on its stream
            a = self.audit
            self._main_wait_side(kl_done)
            clip = a.grad and a.clip is not None
            if clip:
                self._side_wait_main()            # the clip decision reads the hot pass's per-sample losses
            else:
                a.add_kl_grad()
            clip_done = None
            with self._on_side():
                probes = getattr(self, "_join_probes", None)
                if probes is not None:
                    s0 = torch.cuda.Event(enable_timing=True, external=True)
                    s0.record(torch.cuda.current_stream(self.device))
                a.forward_ce()
                if clip:
                    a.clip_exact()
                    clip_done = self._side_event()
                if a.grad:
                    self.audit_dh_exact = a.backward_head()
                    a.backward_core(self.audit_dh_exact)
                if probes is not None:
                    s1 = torch.cuda.Event(enable_timing=True, external=True)
                    s1.record(torch.cuda.current_stream(self.device))
                    probes.append(("replay_backward", s0, s1))
            if clip:
                # residual clip: both cross-entropy launches wrote unit-weight gradients; the audited rows of the hot
                # dlogits get their factor now that the exact losses exist (then the KL rows, which it must not touch)
                self._main_wait_side(clip_done)
                a.clip_hot()
                a.add_kl_grad()
        # ---------------- backward
        self._begin_backward()
        dlogits = self.logits
        o.gemm(dlogits, sh["embed.weight"], self.dn16, M=M, N=d, K=V, b_mn=True)
        o.gemm_wgrad(dlogits, self.hidden16, g["embed.weight"], M=V, N=d, K=M)
        hot = self._hot_param_stream

        def defer(on: bool) -> None:        # weight-gradient launches of the hot pass -> their own stream
            if hot is not None:
                o.param_stream = hot if on else None

        g16 = self.grad16
        defer(True)
        o.rmsnorm_bwd(x_last, p["final_norm.weight"], self.rstd_f, self.dn16, None, self.dxa, g16[0],
                      g["final_norm.weight"], self.partial_final)
        audited = self.audit is not None and self.audit.grad       # the replay contributes gradients of its own
        if not audited:
            self._grad_ready("final_norm.weight")
        dcur, dalt = self.dxa, self.dxb
        tail = self.coda if not self.dense else self.blocks
        for i, blk in enumerate(reversed(tail)):
            self._block_bwd(blk, dcur, g16[i], dalt, g16[i + 1], self.dxc, tmp=self.block_tmps[i], mark_ready=not audited)
            dcur, dalt = dalt, dcur
        defer(False)
        n_tail = len(tail)
        hot_w_done = None
        if audited and self._side_stream is not None:
            # the coda's weight gradients are queued: the replay adds its share to them once this point has passed
            hot_w_done = torch.cuda.Event()
            hot_w_done.record(hot if hot is not None else torch.cuda.current_stream(self.device))
        if self.audit is not None:
            # distillation gradient on the hot endpoint of the audited samples, then the replay's own
            # logits / final-norm / coda backward (their weight gradients add to the hot pass's)
            if self.audit.distill_done is not None:
                torch.cuda.current_stream(self.device).wait_event(self.audit.distill_done)
            o.scatter_add_rows(dcur, self.audit.idx_scatter, self.audit.dhot_extra, self.audit.n, S * d)
        if not self.dense:
            # Phi backward writes dh0 into `dalt`; the router's auxiliary losses add their share
            # (its parameter-gradient half goes to the parameter-gradient stream: backward only waits for dh0)
            split = hot is not None
            misc = self._misc_param_stream if (split and self._misc_param_stream is not None) else hot
            if split:
                o.param_stream = misc
            o.macro_phi_bwd_split(self.prelude[-1].out if self.prelude else self.x0, dcur, self._phi_param_dict(),
                                  self.route["recipe_id"], self.route["depth_id"], cfg.macro_update_scale, self.phi_rstd,
                                  self.phi_pooled, self.phi_act, dalt,
                                  dict(gain=g["macro.d_gain"], v=g["macro.v"], u=g["macro.u"], bias=g["macro.bias"]),
                                  self.phi_scratch, B=B, S=S, d=d, m=cfg.macro_rank, R=cfg.recipe_count,
                                  K=len(cfg.depth_choices))
            if split:
                o.param_stream = None
            if getattr(self, "_cons_pending", False):
                # the consistency term's share: d h0 on the chain, the parameter gradients behind the macro operator's own
                clo, chi = self.cons_range
                if self._cons_done is not None:
                    torch.cuda.current_stream(self.device).wait_event(self._cons_done)
                o.add_(dalt, self.cons_dh0)
                if split:
                    with torch.cuda.stream(misc):
                        if self._cons_done is not None:
                            misc.wait_event(self._cons_done)
                        o.add_(self.grad_flat[clo:chi], self.cons_pg_flat)
                else:
                    o.add_(self.grad_flat[clo:chi], self.cons_pg_flat)
            # (the communication stream waits for the weight-gradient stream too, so marking here is safe)
            self._grad_ready("macro.d_gain", "macro.v", "macro.u", "macro.bias")
            dcur, dalt = dalt, dcur
            if audited:
                from .audit import CORE_PARAMS
                # The replay's backward ran beside the hot backward.  On ITS stream: once the hot pass's coda weight
                # gradients are in place it adds its share of the shared gradients, then (own_prelude) carries its
                # d h0 rows through the prelude itself.  The hot pass only waits where it needs a result.
                head_done = None
                with self._on_side():
                    if self.audit.own_prelude:
                        head_done = self.audit.merge_head(hot_w_done)
                        core_done = self.audit.finish_core(head_done, hot_w_done)
                        self.audit.backward_prelude()
                    else:
                        if hot_w_done is not None:
                            self._side_stream.wait_event(hot_w_done)
                        self.audit.merge_shared()
                        core_done = self._side_event()
                    side_done = self._side_event()
                if not self.audit.own_prelude:
                    self._main_wait_side(side_done)
                    self.audit.merge_tail(dcur)
                names = ["final_norm.weight"]
                for blk in reversed(self.coda):
                    pre = blk.prefix
                    names += [f"{pre}.mlp.wd.weight", f"{pre}.mlp.wug.weight", f"{pre}.norm2.weight",
                              f"{pre}.attn.wo.weight", f"{pre}.attn.wqkv.weight", f"{pre}.norm1.weight"]
                if head_done is not None:
                    # coda and final norm are final as soon as the replay's head backward has been merged: their bucket
                    # leaves while the replay is still inside the core
                    self._grad_ready(*names, after=head_done)
                    self._grad_ready(*CORE_PARAMS, after=core_done)
                else:
                    self._grad_ready(*names, *CORE_PARAMS, after=core_done)
            if not tr.disable_router_aux:
                # under data parallelism each rank contributes 1/world of the auxiliary losses' gradient on its own
                # samples, with the load-balance term's batch mean taken over ALL shards (`_global_mean_prob`)
                dims = dict(B=B, S=S, d=d, hid=cfg.router_hidden_dim, R=cfg.recipe_count, K=len(cfg.depth_choices))
                if self._router_early is not None:
                    torch.cuda.current_stream(self.device).wait_event(self._router_early)
                    o.router_aux_add_dh0(dcur, self.router_scratch, **dims)
                else:
                    if split:
                        o.param_stream = misc
                    o.router_aux_bwd_split(self._router_weight_dict(), self.route, self.depth_values, tr.lambda_load / self.loss_div,
                                           tr.lambda_depth / self.loss_div, self.scalars[1:3], self._router_grad_dict(), dcur,
                                           self.router_scratch, mean_prob=self._global_mean_prob(), **dims)
                    if split:
                        o.param_stream = None
                self._grad_ready(*self._router_grad_names())
            o.cast_bf16(dcur, g16[n_tail])
            defer(True)
            late = audited and self.audit.own_prelude       # their other share arrives at the last join
            for j, blk in enumerate(reversed(self.prelude)):
                self._block_bwd(blk, dcur, g16[n_tail + j], dalt, g16[n_tail + j + 1], self.dxc, tmp=self.block_tmps[n_tail + j],
                                mark_ready=not late)
                dcur, dalt = dalt, dcur
            defer(False)
        o.embed_bwd(tokens, dcur, g["embed.weight"], self.embed_accum)
        if audited and self.audit.own_prelude:
            # last join: the replay's prelude and embedding gradients meet the hot pass's
            self._main_wait_side(side_done)
            if hot is not None:
                torch.cuda.current_stream(self.device).wait_stream(hot)
            self.audit.merge_tail(None)
            for blk in reversed(self.prelude):
                pre = blk.prefix
                self._grad_ready(f"{pre}.mlp.wd.weight", f"{pre}.mlp.wug.weight", f"{pre}.norm2.weight",
                                 f"{pre}.attn.wo.weight", f"{pre}.attn.wqkv.weight", f"{pre}.norm1.weight")
        self._grad_ready("embed.weight")
        if self.audit is not None and not audited:
            self._main_wait_side(self._side_event())          # the replay's forward results are part of the step's results
        if hot is not None:
            torch.cuda.current_stream(self.device).wait_stream(hot)
            if self._misc_param_stream is not None:
                torch.cuda.current_stream(self.device).wait_stream(self._misc_param_stream)
        self._finish_backward()

    def _loss_guard(self) -> None:
        """Device-side `torch.isfinite(loss)` (training.py:448): flags the step when any piece the loss is assembled from
        -- summed token loss, auxiliary terms, per-sample losses, the audited terms -- or, with clipping, the
        gradient's sum of squares is not finite.  (The reference checks the loss only; a non-finite gradient norm
        under clipping would write NaN into every weight there, so dropping that step too is the stricter reading.)"""
        B, k_a = self.B, self.audit_k or 0
        r = self._results
        audit_part = r[8 + 2 * B: 8 + 2 * B + 5 * k_a + 1] if k_a else None       # (terms of unused slots are finite too)
        self.ops.nonfinite_guard([r[0:8], r[8:8 + B], audit_part], self.skip_flag, self.scalars[5:6])

    def _optimizer_step(self) -> None:
        o, tr = self.ops, self.tr
        clip = None
        if tr.grad_clip_norm is not None:
            o.grad_norm(self.plan, self.gn_partial, self.scalars[3:4], float(tr.grad_clip_norm), self.scalars[4:5])
            clip = self.scalars[4:5]
        self._loss_guard()
        o.adamw(self.plan, 0.9, 0.999, 1e-8, tr.weight_decay, clip, skip=self.skip_flag,
                metric_out=self._metric_sums if self.grad_metrics else None,
                absent_flag=self._core_absent, absent_mask=self._absent_mask)
        if self._core_absent is not None:
            self._core_absent.fill_(1)

    def _accumulate(self, last: bool) -> None:
        """Gradient accumulation: a micro-batch's gradients join `accum_flat` (unless its loss was not finite); on the
        cycle's last micro-batch the sum moves into the gradient buffer the optimiser reads."""
        if self.accum == 1:
            return
        o = self.ops
        if not last:
            self._loss_guard()
            o.add_guarded_(self.accum_flat, self.grad_flat, self.skip_flag)
        else:
            o.add_(self.grad_flat, self.accum_flat)
            o.fill_(self.accum_flat, 0.0)

    # ------------------------------------------------------------------ public API
    def _load_batch(self, batch) -> None:
        tokens, targets = batch
        if tuple(tokens.shape) != (self.B, self.S) or tuple(targets.shape) != (self.B, self.S):
            raise ValueError(f"batch must be [{self.B}, {self.S}] int64 token ids")
        self.tokens.copy_(tokens, non_blocking=True)
        self.targets.copy_(targets, non_blocking=True)
        if self.audit is not None:
            self.audit.choose(self.tr.seed + 10_000 + self.global_step)
        if self.shortlist and self.oc.random_negatives > 0:
            # the reference draws them with a generator seeded by seed + step (output.py:86-94, training.py:1364)
            gen = torch.Generator().manual_seed(self.tr.seed + self.global_step)
            rn = torch.randint(0, self.cfg.vocab_size, (self.B, self.S, self.oc.random_negatives), generator=gen)
            self.random_negs.copy_(rn.view(self.M, -1).to(torch.int32), non_blocking=True)

    def _run_step_kernels(self, optimizer: bool, accumulate: bool = False) -> None:
        """`optimizer`: forward + backward + optimiser (the last micro-batch of an accumulation cycle, or every call
        without accumulation); `accumulate`: forward + backward + add into the accumulation buffer; neither: forward +
        backward only (`loss_and_grads`)."""
        def body() -> None:
            self._forward_backward()
            if optimizer:
                self._accumulate(last=True)
                self._optimizer_step()
            elif accumulate:
                self._accumulate(last=False)

        if not self.use_cuda_graph or not (optimizer or accumulate) or self._eager_steps_left > 0:
            if optimizer and self._eager_steps_left > 0:
                self._eager_steps_left -= 1
            body()
            return
        key = "step" if optimizer else "micro"
        if self._graphs.get(key) is None:
            before = self.ops.launches
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            # (capturing the hot pass on a raised-priority stream, so that its kernels are served before the
            # weight-gradient streams, was measured: +3 % step time; all streams but the replay's keep the default)
            with torch.cuda.graph(graph):
                body()
            self._graphs[key] = graph
            if optimizer:
                self._launches_per_step = self.ops.launches - before
        self._graphs[key].replay()

    @property
    def _graph(self):
        return self._graphs.get("step")

    def close(self) -> None:
        """Drops the captured step graphs (which, under data parallelism, hold NCCL kernels) after the device has
        drained, so that the process group can be torn down afterwards (see `teardown_data_parallel`)."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self._graphs.clear()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def loss_and_grads(self, batch) -> tuple[float, dict[str, torch.Tensor]]:
        """Forward + backward without the optimiser (what the parity tests compare with the oracle).  The Bernoulli
        sampler's running state (coverage average, last residual) is put back afterwards: only a training step
        advances it."""
        a = self.audit if (self.audit is not None and self.audit.bernoulli) else None
        keep = (a.audit_ema.clone(), a.recent.clone()) if a is not None else None
        self._load_batch(batch)
        self._run_step_kernels(optimizer=False)
        out = self._assemble_loss(), self.grads
        if a is not None:
            a.audit_ema.copy_(keep[0])
            a.recent.copy_(keep[1])
            if self._core_absent is not None:
                self._core_absent.fill_(1)
        return out

    def evaluate(self, batches) -> dict[str, float]:
        """Forward-only evaluation over an iterable of [B,S] (tokens, targets) batches, as `rte evaluate` does for one
        batch (cli.py:193-319): the mode's own forward (the hot macro pass for `recursive_macro*`, the banked exact
        passes for `recursive_exact`, the dense stack for `dense_exact`), no audit, no gradients, weights untouched.
        Returns the mean per-sample loss (sum over a sample's tokens) and the mean negative log-likelihood per token."""
        if self._pending:
            raise RuntimeError("steps are in flight: collect() them before evaluating")
        audit, self.audit = self.audit, None              # evaluation never replays audited samples
        total, n = 0.0, 0
        try:
            for batch in batches:
                tokens, targets = batch
                if tuple(tokens.shape) != (self.B, self.S):
                    raise ValueError(f"batch must be [{self.B}, {self.S}] int64 token ids")
                self.tokens.copy_(tokens, non_blocking=True)
                self.targets.copy_(targets, non_blocking=True)
                if self.shortlist and self.oc.random_negatives > 0:
                    gen = torch.Generator().manual_seed(self.tr.seed)       # `forward_macro(..., seed=0)` + config seed
                    rn = torch.randint(0, self.cfg.vocab_size, (self.B, self.S, self.oc.random_negatives), generator=gen)
                    self.random_negs.copy_(rn.view(self.M, -1).to(torch.int32), non_blocking=True)
                self._forward_backward(forward_only=True)
                total += float(self.loss_per_sample.sum())
                n += self.B
        finally:
            self.audit = audit
        if hasattr(self.ops, "check_status"):
            self.ops.check_status()
        mean = total / max(n, 1)
        return {"mode": self.tr.mode, "eval_loss_per_sample": mean, "eval_nll_per_token": mean / self.S, "samples": n}

    def _host_slot(self, i: int) -> dict[str, Any]:
        """Pinned host buffers for the results of one in-flight step (two slots alternate)."""
        if self._host_slots is None:
            self._host_slots = [None, None]
        if self._host_slots[i] is None:
            B, k_a = self.B, self.audit_k or 0
            cuda = self.device.type == "cuda"
            h = torch.empty(self._results.shape, dtype=torch.float32, pin_memory=cuda)
            r0 = 8 + 2 * B
            self._host_slots[i] = {
                "flat": h, "status": torch.zeros(1, dtype=torch.int32, pin_memory=cuda),
                "event": torch.cuda.Event() if cuda else None,
                "scalars": h[0:8], "loss_per_sample": h[8:8 + B], "recipe_id": h[8 + B:8 + 2 * B].view(torch.int32),
                "terms": h[r0:r0 + 4 * k_a].view(k_a, 4), "exact_loss": h[r0 + 4 * k_a:r0 + 5 * k_a],
                "kl_sum": h[r0 + 5 * k_a:r0 + 5 * k_a + 1],
                "metric_sums": h[r0 + 5 * k_a + 1 + self._audit_extra:].view(len(METRIC_GROUPS), 2)}
            if k_a:
                self._host_slots[i]["align"] = h[r0 + 5 * k_a + 1:r0 + 13 * k_a + 1].view(k_a, 8)
            if self.audit_padded:
                x0 = r0 + 13 * k_a + 1
                self._host_slots[i].update(audit_idx=h[x0:x0 + k_a].view(torch.int32), audit_inv_p=h[x0 + k_a:x0 + 2 * k_a],
                                           audit_stats=h[x0 + 2 * k_a:x0 + 2 * k_a + 4])
        return self._host_slots[i]

    def _queue_fetch(self) -> dict[str, Any]:
        """Queues, behind the step's kernels, the one device-to-host copy of everything the host reads after a step
        (plus the status word) into the next pinned slot, and records the event `_wait_fetch` waits on."""
        slot = self._host_slot(self._slot_next)
        self._slot_next ^= 1
        slot["flat"].copy_(self._results, non_blocking=True)
        if hasattr(self.ops, "status"):
            slot["status"].copy_(self.ops.status, non_blocking=True)
        if slot["event"] is not None:
            slot["event"].record(torch.cuda.current_stream(self.device))
        slot["chosen"] = self.audit.last_chosen if self.audit is not None else None
        return slot

    def _wait_fetch(self, slot: dict[str, Any]) -> dict[str, Any]:
        if slot["event"] is not None:
            slot["event"].synchronize()
        if int(slot["status"][0]) != 0:
            self.ops.check_status()                          # raises with the decoded device status
        self._host = slot
        return slot

    def _assemble_loss(self, host: dict[str, Any] | None = None) -> float:
        if host is None:
            host = self._wait_fetch(self._queue_fetch())
        vals = host["scalars"]
        loss = float(vals[0]) / (self.B * self.S)          # this rank's shard
        if self.audit is not None:
            terms = self.audit.loss_terms(host["loss_per_sample"], host, host["chosen"])
            loss += terms["correction"] / (self.B * self.S) + sum(terms["aux"].values())
            self.last_audit = terms
        if getattr(self, "cons_pairs", None):
            cons = self.tr.lambda_cons * float(vals[6]) / (len(self.cons_pairs) * self.M * self.cfg.d_model)
            loss += cons
            self.last_consistency = cons
        if not self.dense and not self.tr.disable_router_aux:
            cover = float(torch.relu(self.tr.coverage_min - self.usage_ema).square().sum()) * self.tr.lambda_cover
            loss += (float(vals[1]) + float(vals[2])) * self.loss_div + cover
        return loss

    MAX_IN_FLIGHT = 2

    @property
    def _max_in_flight(self) -> int:
        """The count schedule decides a step's audited count from the metrics of the step before: one step at a time."""
        return 1 if self.audit_scheduled else self.MAX_IN_FLIGHT

    def submit(self, batch) -> None:
        """Queues one training call on a [B,S] int64 (tokens, targets) batch and returns without waiting for the
        device: the batch copy, the step's kernels (one graph replay) and the copy of its results into pinned host
        memory are all stream-ordered.  With `grad_accum_steps` = A the call is a micro-batch: the optimiser runs on
        every A-th call.  At most `MAX_IN_FLIGHT` steps may be queued before `collect` is called; a host batch must
        stay untouched until its step has been collected."""
        if len(self._pending) >= self._max_in_flight:
            raise RuntimeError(f"{len(self._pending)} steps already in flight: call collect() first")
        self._load_batch(batch)
        lr_scale = self.tr.lr_scale(self._tokens_scheduled)        # training.py:470-490, from the tokens seen so far
        if self.tr.lr_schedule != "constant":
            self._write_lr_table(lr_scale)
        self._micro += 1
        stepping = self._micro % self.accum == 0
        self._run_step_kernels(optimizer=stepping, accumulate=not stepping)
        slot = self._queue_fetch()
        slot["stepping"], slot["lr"] = stepping, dict(self._lr_now)
        self._pending.append(slot)
        self._tokens_scheduled += self.B * self.S * self.world
        if stepping:
            self.global_step += 1
        if self.audit is not None and not self.audit.scheduled:
            # host work for the NEXT step (the seeded permutation of its audited subset) while the device runs this one
            # (under the count schedule the next step's count is only known once this step has been collected)
            self.audit.prepare(self.tr.seed + 10_000 + self.global_step)

    def _grad_metrics(self, host: dict[str, Any]) -> dict[str, float]:
        """training.py:386-443 from the per-group sums the AdamW launch left in the results buffer: gradient norm (after
        clipping) and lr * |g| / |p| per optimizer group, plus the core's per-pass FiLM / scale sub-groups."""
        sums = host["metric_sums"]
        gsq = [float(sums[i, 0]) for i in range(len(METRIC_GROUPS))]
        psq = [float(sums[i, 1]) + self._static_param_sq[i] for i in range(len(METRIC_GROUPS))]
        core, film, scale = (METRIC_GROUPS.index(x) for x in ("core", "pass_film", "pass_scale"))
        out: dict[str, float] = {}
        present = {lr_group_of(n, self.cfg.topology) for n in self.params if not n.startswith("shortlist_head.")}
        for i, name in enumerate(LR_GROUPS):
            if name not in present:
                continue
            g2, p2 = gsq[i], psq[i]
            if i == core:                 # the sub-groups are part of the core group as well
                g2, p2 = g2 + gsq[film] + gsq[scale], p2 + psq[film] + psq[scale]
            out[f"grad_norm_{name}"] = g2 ** 0.5
            out[f"update_ratio_{name}"] = host["lr"][name] * g2 ** 0.5 / max(p2 ** 0.5, 1e-12)
        if not self.dense:
            for i, name in ((film, "pass_film"), (scale, "pass_scale")):
                out[f"grad_norm_{name}"] = gsq[i] ** 0.5
                out[f"update_ratio_{name}"] = host["lr"]["core"] * gsq[i] ** 0.5 / max(psq[i] ** 0.5, 1e-12)
        return out

    def collect(self) -> TrainStepResult:
        """Waits for the oldest queued step and returns its loss and metrics (steps complete in submission order)."""
        if not self._pending:
            raise RuntimeError("no step in flight")
        host = self._wait_fetch(self._pending.pop(0))
        loss = self._assemble_loss(host)
        metrics: dict[str, Any] = {"mode": self.tr.mode, "loss": loss, "lr": host["lr"][LR_GROUPS[0] if not self.dense else "dense"]}
        skipped = float(host["scalars"][5]) != 0.0
        stepped = bool(host["stepping"]) and not skipped
        metrics["did_optimizer_step"] = stepped
        if skipped:
            # training.py:448-452: a non-finite loss drops the step; weights, moments and step counters are untouched
            # (the device flag made the AdamW launch a no-op).  Steps queued behind it were seeded with the
            # speculative step number; from here on `global_step` again counts optimiser steps taken.
            metrics["skipped_nonfinite_loss"] = 1.0
            if host["stepping"]:
                self.global_step -= 1
        elif stepped and self.grad_metrics:
            metrics.update(self._grad_metrics(host))
        if self.audit is not None:
            # audit.py:274-299, training.py:1405-1470: what the audit did this step
            la, B, S = self.last_audit, self.B, self.S
            audited = la.get("audited", self.audit.n)
            metrics.update(audit_count=float(audited), audit_rate=audited / B,
                           audit_sampler_fixed_count=0.0 if self.audit.bernoulli else 1.0,
                           audit_is_gradient_corrected=1.0 if self.audit.grad else 0.0,
                           audit_inclusion_prob=la.get("p_inclusion", self.audit.p_inc),
                           audit_requested_probability=la.get("p_requested", self.audit.p_inc),
                           audit_candidate_count=float(la.get("candidates", audited)),
                           macro_distill_loss=sum(la["aux"].values()),
                           hot_lm_loss=float(host["scalars"][0]) / (B * S),
                           corrected_lm_loss=(float(host["scalars"][0]) + la["correction"]) / (B * S),
                           corrected_metric_loss=(float(host["scalars"][0]) + la["correction_metric"]) / (B * S))
            metrics.update({f"macro_{k}_loss": v for k, v in la["aux"].items()})
            metrics.update(la.get("alignment", {}))
            metrics.update(la.get("residual", {}))
            if self.audit.scheduled:
                metrics["audit_fixed_count"] = float(self.audit.count)
                if audited:
                    self.audit.update_schedule(metrics)                  # audit.py:365: decides the next step's count
                metrics["audit_schedule_next_count"] = float(self.audit.count)
            if audited:
                metrics["exact_eval_nll"] = float(la["exact"].mean()) / S
        if getattr(self, "cons_pairs", None):
            metrics["macro_consistency_loss"] = self.last_consistency
        if not self.dense:
            ids = host["recipe_id"].long()
            if getattr(self, "exact_schedule", None) is not None:        # the schedule is what ran (models.py:480-497)
                ids = torch.tensor(self.exact_schedule, dtype=torch.long).repeat(self.B)
            counts = torch.bincount(ids, minlength=self.cfg.recipe_count).float()
            self.usage_ema.mul_(self.tr.coverage_beta).add_(counts / counts.sum().clamp_min(1.0), alpha=1.0 - self.tr.coverage_beta)
            metrics["unique_recipes_per_batch"] = int(ids.unique().numel())
            metrics.update(self._budget)
        self.tokens_seen += self.B * self.S
        metrics["tokens_seen"] = self.tokens_seen
        return TrainStepResult(loss=loss, metrics=metrics)

    def train_step(self, batch) -> TrainStepResult:
        """One optimiser step on a [B,S] int64 (tokens, targets) batch held on the host or the device."""
        if self._pending:
            raise RuntimeError("steps are in flight: collect() them before a synchronous train_step")
        self.submit(batch)
        return self.collect()

    def train_steps(self, batches):
        """Pipelined loop over an iterable of batches: yields one TrainStepResult per batch, in order, keeping
        `MAX_IN_FLIGHT` steps queued so that the host's work for a step (batch copy, launch, result read-back)
        overlaps the device's work on the one before.  Same arithmetic as calling `train_step` per batch."""
        for batch in batches:
            if len(self._pending) >= self._max_in_flight:
                yield self.collect()
            self.submit(batch)
        while self._pending:
            yield self.collect()

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict[str, torch.Tensor]:
        if self._pending:
            raise RuntimeError("steps are in flight: collect() them before reading the parameters")
        return {n: t.detach().clone() for n, t in self.params.items()}

    def backend_status(self) -> dict[str, object]:
        """Counterpart of kernels/optimized.py:27-43 for the run manifest."""
        return {"mode": getattr(self.ops, "name", "unknown"), "strict_cuda": True, "require_flash": False,
                "cuda_available": torch.cuda.is_available(), "triton_available": False,
                "uses_reference_fallback": False}

    @property
    def kernel_launches_per_step(self) -> int | None:
        return self._launches_per_step

    def profile_step(self, repeats: int = 3) -> list[tuple[str, float]]:
        """Device-side duration of every C-ABI call of one step, measured INSIDE a CUDA graph (event-record
        nodes around each call), so that host launch latency does not leak into the numbers.  Returns
        (entry point + shape tag, microseconds) in launch order, averaged over `repeats` replays; calls issued on
        the hot pass's weight-gradient stream carry the suffix "@wgrad", those of the audit replay's streams "@side"."""
        ops = self.ops
        calls: list[tuple[str, Any, Any]] = []
        call_streams: list[int] = []
        orig_call, orig_gemm = ops._call, ops.gemm
        tag = {"v": ""}

        def timed_call(name, *args):
            e0 = torch.cuda.Event(enable_timing=True, external=True)
            e1 = torch.cuda.Event(enable_timing=True, external=True)
            st = torch.cuda.current_stream(self.device)
            e0.record(st)
            orig_call(name, *args)
            e1.record(st)
            hot_ps = self._hot_param_stream.cuda_stream if self._hot_param_stream is not None else None
            misc_ps = getattr(self, "_misc_param_stream", None)
            where = "" if st.cuda_stream == main_stream else (
                "@wgrad" if st.cuda_stream == hot_ps or (misc_ps is not None and st.cuda_stream == misc_ps.cuda_stream) else "@side")
            calls.append((name + tag["v"] + where, e0, e1))
            call_streams.append(st.cuda_stream)

        def tagged_gemm(a, b, out, **kw):
            tag["v"] = f"[{kw['M']}x{kw['N']}x{kw['K']}/epi{kw.get('epilogue', 0)}" + (f"/split{kw['splits']}" if kw.get("splits", 1) > 1 else "") + "]"
            try:
                orig_gemm(a, b, out, **kw)
            finally:
                tag["v"] = ""

        ops._call, ops.gemm = timed_call, tagged_gemm
        main_stream = None
        self._dp_paused = True
        try:
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                main_stream = torch.cuda.current_stream(self.device).cuda_stream
                self._forward_backward()
                self._optimizer_step()
        finally:
            ops._call, ops.gemm = orig_call, orig_gemm
            self._dp_paused = False
        totals = [0.0] * len(calls)
        graph.replay()
        torch.cuda.synchronize(self.device)
        for _ in range(repeats):
            graph.replay()
            torch.cuda.synchronize(self.device)
            for i, (_, e0, e1) in enumerate(calls):
                totals[i] += e0.elapsed_time(e1) * 1e3
        # start of every call relative to the first one (last replay): the timeline across the streams
        first = calls[0][1]
        self.last_profile_starts = [first.elapsed_time(e0) * 1e3 for _, e0, _ in calls]
        known = {main_stream: "main"}
        for label, attr in (("hot_wgrad", "_hot_param_stream"), ("misc_wgrad", "_misc_param_stream"),
                            ("replay", "_side_stream"), ("replay_wgrad", "_param_stream"), ("comm", "_comm_stream")):
            st = getattr(self, attr, None)
            if st is not None:
                known.setdefault(st.cuda_stream, label)
        self.last_profile_streams = [known.get(x, f"stream{x:#x}") for x in call_streams]
        return [(calls[i][0], totals[i] / repeats) for i in range(len(calls))]

    def dp_timeline(self, repeats: int = 5) -> dict[str, Any]:
        """Where the gradient exchange sits inside one data-parallel step: start / end of every bucket's all-reduce on the
        communication stream, of backward and of the optimiser on the main stream, in microseconds from the start of the
        step, from event-record nodes inside a captured step (averaged over `repeats` replays).  EVERY rank must call
        this (the captured step contains the collectives)."""
        self._dp_probes = []
        marks: dict[str, Any] = {}
        ev = lambda: torch.cuda.Event(enable_timing=True, external=True)       # noqa: E731
        try:
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                main = torch.cuda.current_stream(self.device)
                marks["step_start"] = ev(); marks["step_start"].record(main)
                self._forward_backward()
                marks["backward_end"] = ev(); marks["backward_end"].record(main)
                self._optimizer_step()
                marks["step_end"] = ev(); marks["step_end"].record(main)
            probes, self._dp_probes = self._dp_probes, None
        finally:
            self._dp_probes = None
        acc: dict[str, list[float]] = {}
        graph.replay()
        torch.cuda.synchronize(self.device)
        for _ in range(repeats):
            graph.replay()
            torch.cuda.synchronize(self.device)
            t0 = marks["step_start"]
            for k in ("backward_end", "step_end"):
                acc.setdefault(k, []).append(t0.elapsed_time(marks[k]) * 1e3)
            for name, nbytes, e0, e1 in probes:
                acc.setdefault(name + ".start", []).append(t0.elapsed_time(e0) * 1e3)
                acc.setdefault(name + ".end", []).append(t0.elapsed_time(e1) * 1e3)
        del graph
        mean = {k: sum(v) / len(v) for k, v in acc.items()}
        buckets = [dict(name=name, mb=nbytes / 2 ** 20, start_us=mean[name + ".start"], end_us=mean[name + ".end"])
                   for name, nbytes, _, _ in probes]
        last_end = max((b["end_us"] for b in buckets), default=0.0)
        return {"backward_end_us": mean["backward_end"], "step_end_us": mean["step_end"], "buckets": buckets,
                "exchange_exposed_us": max(0.0, last_end - mean["backward_end"]), "bucket_cap_mb": self.bucket_cap_mb}

    def join_waits(self, repeats: int = 20) -> dict[str, Any]:
        """How long the hot pass idles at each point where it waits for the audit replay's stream, in microseconds, from
        event-record nodes placed only around those waits inside a captured step (averaged over `repeats` replays of the
        batch loaded last), with the length of that step.  A few nodes on one stream: unlike `profile_step`, this does
        not stretch the replay's long chain of launches."""
        if self._side_stream is None:
            return {"waits_us": [], "step_us": None}
        self._join_probes = []
        ev = lambda: torch.cuda.Event(enable_timing=True, external=True)       # noqa: E731
        try:
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                main = torch.cuda.current_stream(self.device)
                start = ev(); start.record(main)                                # noqa: E702
                self._forward_backward()
                self._optimizer_step()
                end = ev(); end.record(main)                                    # noqa: E702
            probes = self._join_probes
        finally:
            self._join_probes = None
        graph.replay()
        torch.cuda.synchronize(self.device)
        spans, begins, step = [0.0] * len(probes), [0.0] * len(probes), 0.0
        for _ in range(repeats):
            graph.replay()
            torch.cuda.synchronize(self.device)
            step += start.elapsed_time(end) * 1e3 / repeats
            for i, (_, e0, e1) in enumerate(probes):
                spans[i] += e0.elapsed_time(e1) * 1e3 / repeats
                begins[i] += start.elapsed_time(e0) * 1e3 / repeats
        del graph
        pick = lambda kind, vals: [round(v, 1) for (k, _, _), v in zip(probes, vals) if k == kind]      # noqa: E731
        return {"waits_us": pick("wait", spans), "at_us": pick("wait", begins), "step_us": round(step, 1),
                "replay_backward_us": pick("replay_backward", spans), "replay_backward_at_us": pick("replay_backward", begins)}

    def gemm_roofline(self, repeats: int = 5) -> dict[str, Any]:
        """Relates the algorithmic 2*M*N*K FLOPs of every tcgen05 GEMM launch of one step to its device
        duration, taken from event-record nodes around each launch inside a captured step (`profile_step`),
        i.e. under the same cache state and stream concurrency as the timed step and without host gaps.  The
        headline figures cover the hot pass (main stream and its weight-gradient stream); the audit replay's
        few-row GEMMs, which run beside it on their own streams, are reported under "side_stream"."""
        import re
        acc = {"": [0.0, 0.0, 0, {}], "@side": [0.0, 0.0, 0, {}]}      # flops, us, launches, per shape
        # the hot pass's weight-gradient GEMMs normally overlap its other kernels on their own stream, which would
        # stretch every overlapping launch's event interval: for this measurement they run in line on the main stream
        keep, self._hot_param_stream = self._hot_param_stream, None
        try:
            profile = self.profile_step(repeats)
        finally:
            self._hot_param_stream = keep
        for name, t in profile:
            m = re.match(r"rte_gemm_bf16(?:_small)?\[(\d+)x(\d+)x(\d+)/(.*)\](@side|@wgrad)?$", name)
            if not m:
                continue
            f = 2.0 * int(m.group(1)) * int(m.group(2)) * int(m.group(3))
            a = acc["@side" if m.group(5) == "@side" else ""]       # the hot pass = main stream + its weight-gradient stream
            a[0], a[1], a[2] = a[0] + f, a[1] + t, a[2] + 1
            sh = a[3].setdefault(f"{m.group(1)}x{m.group(2)}x{m.group(3)}/{m.group(4)}", [0.0, 0.0, 0])
            sh[0] += f
            sh[1] += t
            sh[2] += 1

        def table(d):
            return {k: {"launches": v[2], "us": v[1] / v[2], "tflops": v[0] / (v[1] * 1e-6) / 1e12} for k, v in d.items()}

        hot, side = acc[""], acc["@side"]
        out = {"tflops": hot[0] / (hot[1] * 1e-6) / 1e12, "launches": hot[2], "gemm_ms_per_step": hot[1] * 1e-3,
               "per_shape": table(hot[3])}
        if side[2]:
            out["side_stream"] = {"tflops": side[0] / (side[1] * 1e-6) / 1e12, "launches": side[2],
                                  "gemm_ms_per_step": side[1] * 1e-3, "per_shape": table(side[3])}
        return out
