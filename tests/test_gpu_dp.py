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


def _check_peer_allreduce(eng, rank, world):
    """The exchange kernel on its own: ranges of several sizes and offsets of the shared gradient buffer, filled with
    values every rank can reproduce, against the analytic sum; twice per range (the flags' epochs advance)."""
    peer, flat = eng._peer, eng.grad_flat
    n = flat.numel()
    vals = [torch.randn(n, generator=torch.Generator().manual_seed(100 + q)) for q in range(world)]
    want = sum(vals)
    ranges = [(0, min(n, 4096)), (64, min(n, 64 + 1000 * 4)), (0, n - n % 4), (n // 2 - (n // 2) % 4, n - n % 4)]
    for rep in range(2):
        for slot, (lo, hi) in enumerate(ranges):
            flat.copy_(vals[rank])
            torch.cuda.synchronize()
            dist.barrier()
            peer.all_reduce_(lo, hi, slot)
            torch.cuda.synchronize()
            dist.barrier()
            eng.ops.check_status()
            got = flat.cpu()
            assert torch.allclose(got[lo:hi], want[lo:hi], rtol=1e-6, atol=1e-6), (rep, lo, hi)
            assert torch.equal(got[:lo], vals[rank][:lo]) and torch.equal(got[hi:], vals[rank][hi:])
    flat.zero_()


def _worker(rank, world, port, out_path, comm):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["RTE_DP_COMM"] = comm
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    cfg = ExperimentConfig(ModelConfig(**MODEL), TrainingConfig(**TRAIN))
    eng = TrainEngine(cfg, init_parameters(cfg.model, seed=3), device=dev, process_group=dist.group.WORLD, bucket_cap_mb=0.25)
    assert (eng._peer is not None) == (comm == "peer")
    if eng._peer is not None:
        _check_peer_allreduce(eng, rank, world)
    losses = [eng.train_step(b).loss for b in _batches()]
    captured = eng._graph is not None
    if rank == 0:
        torch.save({"losses": losses, "captured": captured, "params": {k: v.cpu() for k, v in eng.params.items()}}, out_path)
    teardown_data_parallel(eng)      # graphs first, then the process group


@pytest.mark.parametrize("comm", ["peer", "nccl"])
def test_two_gpu_ranks_with_the_same_shard_equal_one_gpu(tmp_path, comm):
    """`comm`: the gradient exchange -- "peer" = one kernel per rank over NVLink peer memory, "nccl" = library all-reduce."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "rank0.pt"
    ctx = mp.spawn(_worker, args=(2, port, str(out), comm), nprocs=2, join=False)
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
