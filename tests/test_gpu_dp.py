"""Data-parallel step on two GPUs over NCCL (skipped with fewer): two ranks holding the SAME shard must reproduce the
single-GPU run -- every gradient is g/2 + g/2 -- through the eager steps, the capture of the collective-bearing graph
and its replays, with an audited sample (whose gradients reach the buckets from the replay's stream)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from speedup_thingy_b200.config import ExperimentConfig, ModelConfig, TrainingConfig
from speedup_thingy_b200.engine import TrainEngine, init_parameters, teardown_data_parallel

pytestmark = pytest.mark.gpu

MODEL = dict(vocab_size=256, d_model=128, n_heads=4, d_ff=256, n_prelude=1, n_coda=1, t_max=4, depth_choices=(1, 2, 4),
             attn_banks=1, ffn_banks=1, head_groups=4, ffn_groups=4, active_head_groups=2, active_ffn_groups=2,
             recipe_count=5, macro_rank=32)
TRAIN = dict(mode="recursive_macro", lr=1e-3, weight_decay=0.1, batch_size=8, seq_len=32, seed=3, fixed_depth=None,
             audit_fixed_count_per_batch=1, grad_clip_norm=1.0)
STEPS = 7


def _batches():
    g = torch.Generator().manual_seed(7)
    out = []
    for _ in range(STEPS):
        toks = torch.randint(0, MODEL["vocab_size"], (TRAIN["batch_size"], TRAIN["seq_len"] + 1), generator=g)
        out.append((toks[:, :-1].contiguous(), toks[:, 1:].contiguous()))
    return out


def _worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    cfg = ExperimentConfig(ModelConfig(**MODEL), TrainingConfig(**TRAIN))
    eng = TrainEngine(cfg, init_parameters(cfg.model, seed=3), device=dev, process_group=dist.group.WORLD, bucket_cap_mb=0.25)
    losses = [eng.train_step(b).loss for b in _batches()]
    captured = eng._graph is not None
    if rank == 0:
        torch.save({"losses": losses, "captured": captured, "params": {k: v.cpu() for k, v in eng.params.items()}}, out_path)
    teardown_data_parallel(eng)      # graphs first, then the process group


def test_two_gpu_ranks_with_the_same_shard_equal_one_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "rank0.pt"
    ctx = mp.spawn(_worker, args=(2, port, str(out)), nprocs=2, join=False)
    ctx.join(timeout=300)
    got = torch.load(out)
    assert got["captured"], "the data-parallel step graph was not captured"
    cfg = ExperimentConfig(ModelConfig(**MODEL), TrainingConfig(**TRAIN))
    single = TrainEngine(cfg, init_parameters(cfg.model, seed=3), device="cuda:0")
    losses = [single.train_step(b).loss for b in _batches()]
    for a, b in zip(losses, got["losses"]):
        assert abs(a - b) <= 1e-3 * abs(a), (losses, got["losses"])
    for n, p in single.params.items():
        diff = (p.cpu() - got["params"][n]).abs()
        assert diff.max().item() <= 2.1 * TRAIN["lr"], n
        assert diff.mean().item() <= 0.02 * TRAIN["lr"], n
