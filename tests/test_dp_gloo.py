"""Data-parallel path on CPU: two gloo ranks, each with half of the global batch, must end up with the
gradients (and, after the optimiser, the weights) of one process that saw the whole batch -- the reference's
grad-accumulation parity (tests/test_training_fixes.py:53-75) carried over to ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from speedup_thingy_b200.config import ExperimentConfig, ModelConfig, TrainingConfig
from speedup_thingy_b200.engine import TrainEngine, init_parameters
from tests.emul_ops import EmulOps

MODEL = dict(vocab_size=96, d_model=64, n_heads=4, d_ff=128, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=8)
TRAIN = dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, seq_len=16, seed=3, fixed_depth=4,
             disable_router_aux=True, grad_clip_norm=1.0)
GLOBAL_B = 8


def _batch():
    g = torch.Generator().manual_seed(42)
    toks = torch.randint(0, MODEL["vocab_size"], (GLOBAL_B, TRAIN["seq_len"] + 1), generator=g)
    return toks[:, :-1].contiguous(), toks[:, 1:].contiguous()


def _worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    cfg = ExperimentConfig(ModelConfig(**MODEL), TrainingConfig(**{**TRAIN, "batch_size": GLOBAL_B // world}))
    params = init_parameters(cfg.model, seed=3)
    eng = TrainEngine(cfg, params, device="cpu", ops=EmulOps(), use_cuda_graph=False, process_group=dist.group.WORLD,
                      bucket_cap_mb=0.05)   # tiny buckets: several exchanges per step
    assert len(eng._buckets) > 3
    x, y = _batch()
    lo, hi = rank * (GLOBAL_B // world), (rank + 1) * (GLOBAL_B // world)
    _, grads = eng.loss_and_grads((x[lo:hi], y[lo:hi]))
    grads = {k: v.clone() for k, v in grads.items()}
    eng.train_step((x[lo:hi], y[lo:hi]))
    if rank == 0:
        torch.save({"grads": grads, "params": {k: v.clone() for k, v in eng.params.items()}}, out_path)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_one_process_on_the_global_batch(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "rank0.pt"
    mp.spawn(_worker, args=(2, port, str(out)), nprocs=2, join=True)
    got = torch.load(out)
    cfg = ExperimentConfig(ModelConfig(**MODEL), TrainingConfig(**{**TRAIN, "batch_size": GLOBAL_B}))
    single = TrainEngine(cfg, init_parameters(cfg.model, seed=3), device="cpu", ops=EmulOps(), use_cuda_graph=False)
    _, ref = single.loss_and_grads(_batch())
    ref = {k: v.clone() for k, v in ref.items()}
    single.train_step(_batch())
    assert sorted(ref) == sorted(got["grads"])
    for n in ref:
        scale = max(ref[n].abs().max().item(), 1e-6)
        assert (ref[n] - got["grads"][n]).abs().max().item() <= 2e-2 * scale + 1e-6, n
    for n, p in single.params.items():
        assert (p - got["params"][n]).abs().max().item() <= 2.1 * TRAIN["lr"], n


AUDIT_TRAIN = dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, seq_len=16, seed=3, fixed_depth=None,
                   audit_fixed_count_per_batch=1, grad_clip_norm=1.0)


SAMPLERS = {
    "fixed_count": {},
    # subset drawn on the device from the step's routing; capacity-padded replay
    "bernoulli": dict(audit_fixed_count_per_batch=None, audit_sampler="bernoulli", audit_p_min=0.3, audit_p_max=0.8,
                      audit_alpha=0.5, audit_beta=1.0, audit_gamma=0.3, audit_cap=2),
    # fixed count under the count schedule (each rank decides from its own shard's metrics: equal shards, equal counts)
    "scheduled": dict(audit_fixed_count_per_batch=2, audit_schedule_enabled=True, audit_schedule_min_count=1,
                      audit_schedule_nll_gap_threshold=0.3, audit_schedule_hidden_cosine_threshold=0.9,
                      audit_schedule_delta_rms_ratio_min=0.0, audit_schedule_delta_rms_ratio_max=10.0,
                      audit_schedule_require_negative_mse_slope=False, audit_schedule_require_negative_norm_slope=False),
}


def _replicated_worker(rank, world, port, out_path, sampler="fixed_count"):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    cfg = ExperimentConfig(ModelConfig(**MODEL), TrainingConfig(**{**AUDIT_TRAIN, **SAMPLERS[sampler], "batch_size": 4}))
    eng = TrainEngine(cfg, init_parameters(cfg.model, seed=3), device="cpu", ops=EmulOps(), use_cuda_graph=False,
                      process_group=dist.group.WORLD, bucket_cap_mb=0.05)
    x, y = _batch()
    results = [eng.train_step((x[:4], y[:4])) for _ in range(3)]
    if rank == 0:
        torch.save({"losses": [r.loss for r in results], "counts": [r.metrics["audit_count"] for r in results],
                    "params": {k: v.clone() for k, v in eng.params.items()}}, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("sampler", list(SAMPLERS))
def test_two_ranks_with_the_same_shard_equal_one_process_with_audit(tmp_path, sampler):
    """With audited samples per rank (their gradients reach the buckets from the replay's side of the step, and the
    prelude's only after the last join), two ranks that hold the SAME shard must reproduce the single-process run:
    every gradient is g/2 + g/2 -- for the fixed-count sampler, the Bernoulli sampler with a cap and the count
    schedule alike (same shard, same seeds: the same subsets and the same counts on both ranks)."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "rank0.pt"
    mp.spawn(_replicated_worker, args=(2, port, str(out), sampler), nprocs=2, join=True)
    got = torch.load(out)
    cfg = ExperimentConfig(ModelConfig(**MODEL), TrainingConfig(**{**AUDIT_TRAIN, **SAMPLERS[sampler], "batch_size": 4}))
    single = TrainEngine(cfg, init_parameters(cfg.model, seed=3), device="cpu", ops=EmulOps(), use_cuda_graph=False)
    x, y = _batch()
    results = [single.train_step((x[:4], y[:4])) for _ in range(3)]
    losses = [r.loss for r in results]
    assert [r.metrics["audit_count"] for r in results] == got["counts"]
    if sampler != "fixed_count":
        assert len(set(got["counts"])) > 1 or sampler == "bernoulli"         # the schedule moved the count
    for a, b in zip(losses, got["losses"]):
        assert abs(a - b) <= 2e-3 * abs(a), (losses, got["losses"])
    for n, p in single.params.items():
        assert (p - got["params"][n]).abs().max().item() <= 2.1 * AUDIT_TRAIN["lr"], n
        assert (p - got["params"][n]).abs().mean().item() <= 0.05 * AUDIT_TRAIN["lr"], n


ROUTED_TRAIN = dict(mode="recursive_macro", lr=2e-3, weight_decay=0.1, seq_len=16, seed=3, fixed_depth=None,
                    disable_router_aux=False, lambda_load=0.5, lambda_depth=0.05)


def _routed_params():
    """Benchmark initialisation with the recipe router's weights scaled up: the recipe probabilities differ clearly
    from sample to sample, so the batch mean (and its square) is far from the uniform fixed point."""
    params = init_parameters(ModelConfig(**MODEL), seed=3)
    params["router.recipe_mlp.0.weight"] *= 40.0
    params["router.recipe_mlp.2.weight"] *= 40.0
    return params


def _routed_worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    cfg = ExperimentConfig(ModelConfig(**MODEL), TrainingConfig(**{**ROUTED_TRAIN, "batch_size": GLOBAL_B // world}))
    eng = TrainEngine(cfg, _routed_params(), device="cpu", ops=EmulOps(), use_cuda_graph=False,
                      process_group=dist.group.WORLD, bucket_cap_mb=0.05)
    x, y = _batch()
    lo, hi = rank * (GLOBAL_B // world), (rank + 1) * (GLOBAL_B // world)
    loss, grads = eng.loss_and_grads((x[lo:hi], y[lo:hi]))
    if rank == 0:
        torch.save({"grads": {k: v.clone() for k, v in grads.items()}, "aux": eng.scalars[1:3].clone() * eng.loss_div}, out_path)
    dist.barrier()
    dist.destroy_process_group()


def test_split_batch_with_router_aux_equals_the_global_batch(tmp_path):
    """The load-balance loss squares a batch mean (metrics.py:103-105), so a shard-local mean would NOT reproduce the
    global-batch gradient: the ranks exchange the R-float mean before the square.  Two ranks on a really split batch,
    router-chosen recipes and depths, auxiliary losses on (weights raised so that they matter), against one process on
    the whole batch."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "rank0.pt"
    mp.spawn(_routed_worker, args=(2, port, str(out)), nprocs=2, join=True)
    got = torch.load(out)
    cfg = ExperimentConfig(ModelConfig(**MODEL), TrainingConfig(**{**ROUTED_TRAIN, "batch_size": GLOBAL_B}))
    single = TrainEngine(cfg, _routed_params(), device="cpu", ops=EmulOps(), use_cuda_graph=False)
    _, ref = single.loss_and_grads(_batch())
    assert float(single.scalars[1]) > 1e-3          # the term is active: the probabilities are far from uniform
    assert abs(float(single.scalars[1]) - float(got["aux"][0])) <= 1e-5 * abs(float(single.scalars[1])) + 1e-8      # the load-balance loss itself
    router = [n for n in ref if n.startswith("router.recipe_mlp")]
    assert router
    for n in ref:
        scale = max(ref[n].abs().max().item(), 1e-6)
        tol = 1e-4 if n in router else 2e-2          # the router only sees the auxiliary losses: exact up to fp32 order
        assert (ref[n] - got["grads"][n]).abs().max().item() <= tol * scale + 1e-7, (n, scale)
