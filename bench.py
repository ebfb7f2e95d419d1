"""Benchmark of the `recursive_macro` training step (BASELINE metric: train tokens/sec).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU implementation of the same step on the host cores

One JSON line on stdout (rank 0).  `value` = device-timed whole-job tokens/sec with the batch already
in HBM (CUDA-graph replays between CUDA events, max over ranks); `e2e` = the same through
`TrainEngine.train_step` with pinned HOST batches (H2D copy and loss read-back inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# BASELINE.json configs[2]: recursive_macro cluster-pool config, expressed in the reference's schema.
C3_MODEL = dict(vocab_size=2048, d_model=512, n_heads=8, d_ff=2048, n_prelude=1, n_coda=1, t_max=4,
                depth_choices=(1, 2, 4), attn_banks=1, ffn_banks=1, head_groups=8, ffn_groups=16,
                active_head_groups=2, active_ffn_groups=4, recipe_count=5, macro_rank=32)
C3_TRAIN = dict(mode="recursive_macro", lr=1e-3, weight_decay=0.1, batch_size=128, seq_len=64, seed=0, fixed_depth=4,
                audit_fixed_count_per_batch=1)     # exact-audit control variate at probability 1/128
WORKLOAD = "BASELINE configs[2]: recursive_macro depth 4, d512 H8 F2048 (16x128 slabs, 4 active) V2048, batch 128x64, audit 1/128"


def step_flops_per_token(m: dict) -> float:
    """Algorithmic training FLOPs per token of the hot step: 3 x forward, forward =
    (n_prelude+n_coda) * (8 d^2 + 6 d F + 4 S d) + 8 d m + 2 d V."""
    d, f, v, s = m["d_model"], m["d_ff"], m["vocab_size"], C3_TRAIN["seq_len"]
    block = 8 * d * d + 6 * d * f + 4 * s * d
    return 3.0 * ((m["n_prelude"] + m["n_coda"]) * block + 8 * d * m["macro_rank"] + 2 * d * v)


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def mark(self) -> None:
        """Only samples taken from now on count (the sampler is started early so that nvidia-smi's start-up time does
        not eat a short timed region)."""
        self.first = len(self.rows)

    def summary(self) -> dict:
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows[getattr(self, "first", 0):]:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_port_tokens_per_sec(sample_batch: int, steps: int, threads: int) -> tuple[float, str]:
    """Times the CPU restatement of the reference step (oracle/, fp32, autograd + AdamW) on a bounded
    sample of the workload: the same model and sequence length at a reduced batch."""
    import torch

    from oracle import rte_oracle as O

    torch.set_num_threads(threads)
    train = {**C3_TRAIN, "batch_size": sample_batch}
    ocfg, otr = O.ModelCfg(**C3_MODEL), O.TrainCfg(**train)
    trainer = O.OracleTrainer(ocfg, otr, O.init_params(ocfg, seed=0))
    toks = O.zipf_tokens(sample_batch * 64 * (steps + 3) + 1, ocfg.vocab_size, seed=0)
    it = O.batches(toks, sample_batch, 64)
    trainer.train_step(*next(it))                       # warm-up
    t0 = time.perf_counter()
    for _ in range(steps):
        trainer.train_step(*next(it))
    dt = time.perf_counter() - t0
    return sample_batch * 64 * steps / dt, f"{steps} steps of batch {sample_batch}x64 (of 128x64), fp32, {threads} threads"


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    t0 = time.perf_counter()
    vals = []
    for _ in range(max(args.steps, 1)):
        v, sample = cpu_port_tokens_per_sec(sample_batch=128, steps=1, threads=threads)     # the whole 128x64 step
        vals.append(v)
        if time.perf_counter() - t0 > 150:
            break
    vals.sort()
    value = vals[len(vals) // 2]
    line = {"impl": "reference", "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": len(vals), "warmup": 1, "ms_per_step": 1000.0 * 128 * 64 / value,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "CPU port of the reference step (oracle/rte_oracle.py) on all host cores, each step "
                       "the whole 128x64 batch (fresh trainer + one warm-up step per timed step; median)"},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def probe_gemm(iters: int, warmup: int) -> None:
    """Stand-alone launches of the hot pass's GEMM shapes (one JSON line per shape): the small, fixed case the
    `ncu --set full` capture of the tcgen05 kernel is taken on.  Operands rotate over sets larger than L2."""
    import torch

    from speedup_thingy_b200 import _abi as A
    from speedup_thingy_b200.ops import CudaOps

    ops, dev = CudaOps("cuda:0"), "cuda:0"
    M, d, F, V = C3_TRAIN["batch_size"] * C3_TRAIN["seq_len"], C3_MODEL["d_model"], C3_MODEL["d_ff"], C3_MODEL["vocab_size"]
    bf, f32 = torch.bfloat16, torch.float32
    shapes = [  # name, M, N, K, a_mn, b_mn, epilogue, residual, splits
        ("qkv", M, 3 * d, d, 0, 0, A.EPI_BF16, False, 1), ("wo+residual", M, d, d, 0, 0, A.EPI_F32, True, 1),
        ("w_ug", M, 2 * F, d, 0, 0, A.EPI_BF16, False, 1), ("w_d+residual", M, d, F, 0, 0, A.EPI_F32, True, 1),
        ("logits", M, V, d, 0, 0, A.EPI_BF16, False, 1), ("dz=dy.w_d", M, F, d, 0, 1, A.EPI_BF16, False, 1),
        ("dn=dug.w_ug", M, d, 2 * F, 0, 1, A.EPI_BF16, False, 1), ("dw_ug", 2 * F, d, M, 1, 1, A.EPI_F32, False, 2),
        ("dw_qkv", 3 * d, d, M, 1, 1, A.EPI_F32, False, 6)]
    sets = 4
    for name, m, n, k, a_mn, b_mn, epi, res, splits in shapes:
        a = [torch.randn((k, m) if a_mn else (m, k), device=dev).to(bf) for _ in range(sets)]
        b = [torch.randn((k, n) if b_mn else (n, k), device=dev).to(bf) for _ in range(sets)]
        out = [torch.empty(splits * m * n, device=dev, dtype=f32 if epi == A.EPI_F32 else bf) for _ in range(sets)]
        r = [torch.randn(m, n, device=dev) for _ in range(sets)] if res else [None] * sets
        kw = dict(M=m, N=n, K=k, a_mn=bool(a_mn), b_mn=bool(b_mn), epilogue=epi, ldc=n)
        if splits > 1:
            kw.update(splits=splits, split_stride=m * n)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(warmup):
            ops.gemm(a[i % sets], b[i % sets], out[i % sets], residual=r[i % sets], **kw)
        e0.record()
        for i in range(iters):
            ops.gemm(a[i % sets], b[i % sets], out[i % sets], residual=r[i % sets], **kw)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / iters
        print(json.dumps({"gemm": name, "M": m, "N": n, "K": k, "splits": splits, "us": us, "tflops": 2.0 * m * n * k / us / 1e6}))
    ops.check_status()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--eager", action="store_true", help="launch kernels one by one instead of replaying the CUDA graph (profiling)")
    ap.add_argument("--no-roofline", action="store_true", help="skip the per-launch GEMM timing pass (profiling)")
    ap.add_argument("--probe-gemm", action="store_true", help="time the hot pass's GEMM shapes stand-alone and exit (profiling)")
    ap.add_argument("--probe-iters", type=int, default=20)
    ap.add_argument("--probe-warmup", type=int, default=3)
    args = ap.parse_args()
    if args.probe_gemm:
        probe_gemm(args.probe_iters, args.probe_warmup)
        return
    if args.impl == "reference":
        run_reference(args)
        return

    import torch

    from speedup_thingy_b200.config import ExperimentConfig, ModelConfig, TrainingConfig
    from speedup_thingy_b200.engine import TrainEngine, init_parameters

    # stdout carries exactly one JSON line: everything libraries print there (NCCL's version banner) goes to stderr
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def _emit(text: str) -> None:
        os.write(real_stdout, (text + "\n").encode())

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    cfg = ExperimentConfig(ModelConfig(**C3_MODEL), TrainingConfig(**C3_TRAIN))
    B, S = cfg.training.batch_size, cfg.training.seq_len
    params = init_parameters(cfg.model, seed=0)
    kw = {"process_group": dist.group.WORLD} if world > 1 else {}
    eng = TrainEngine(cfg, params, device=dev, use_cuda_graph=not args.eager, **kw)

    # synthetic Zipf(1.1) token stream, per-rank seed; batches cut as windows of S+1 with stride S
    ranks_ = torch.arange(1, cfg.model.vocab_size + 1, dtype=torch.float64)
    probs = (ranks_.pow(-1.1) / ranks_.pow(-1.1).sum()).float()
    gen = torch.Generator().manual_seed(rank)
    n_batches = 8
    stream = torch.multinomial(probs, B * S * n_batches + 1, replacement=True, generator=gen)
    host_batches = []
    for i in range(n_batches):
        win = stream[i * B * S: (i + 1) * B * S + 1]
        x = win[:-1].view(B, S).clone().pin_memory()
        y = win[1:].view(B, S).clone().pin_memory()
        host_batches.append((x, y))

    W, K = max(args.warmup, 3), args.steps
    clocks = ClockSampler(local).__enter__()          # running before the timed region; see ClockSampler.mark
    for i in range(W):
        eng.train_step(host_batches[i % n_batches])
    for i in range(8):          # data parallel: the first steps run eagerly (NCCL set-up); capture before timing
        if not eng.use_cuda_graph or eng._graph is not None:
            break
        eng.train_step(host_batches[i % n_batches])
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed: batch resident in HBM, K replays of the whole-step graph
    eng._load_batch(host_batches[0])
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks.mark()
    try:
        l0 = eng.ops.launches
        e0.record()
        for _ in range(K):
            eng._run_step_kernels(optimizer=True)
        e1.record()
        barrier()
        ms_dev = e0.elapsed_time(e1)
        # C-ABI launches inside the timed region: counted directly when eager, per captured step when replayed
        launches_timed = (eng.ops.launches - l0) or (eng.kernel_launches_per_step or 0) * K
        # ---- end to end through the public API with pinned host batches
        barrier()
        # (a) the pipelined loop (`train_steps`: two steps in flight; every step copies its batch in and its results
        # out, and every step's loss is read on the host), (b) one synchronous `train_step` call per batch
        t0 = time.perf_counter()
        losses = [r.loss for r in eng.train_steps(host_batches[i % n_batches] for i in range(K))]
        torch.cuda.synchronize()
        ms_e2e = (time.perf_counter() - t0) * 1e3
        assert len(losses) == K and all(math.isfinite(x) for x in losses)
        barrier()
        t0 = time.perf_counter()
        for i in range(K):
            eng.train_step(host_batches[i % n_batches])
        torch.cuda.synchronize()
        ms_e2e_sync = (time.perf_counter() - t0) * 1e3
        if dist is not None:
            t = torch.tensor([ms_dev, ms_e2e, ms_e2e_sync], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_dev, ms_e2e, ms_e2e_sync = float(t[0]), float(t[1]), float(t[2])
        # The two timed loops may be shorter than nvidia-smi's sampling period: keep the same step running (untimed)
        # for about half a second so that a few clock samples under this load exist (same count on every rank).
        for i in range(max(1, min(400, int(500.0 / max(ms_e2e / K, 0.1))))):
            eng.train_step(host_batches[i % n_batches])
        torch.cuda.synchronize()
    finally:
        clocks.__exit__(None, None, None)
    eng.ops.check_status()

    # ---- roofline of the dominant kernel (the tcgen05 GEMM): CUDA-event nodes around every launch of a captured step
    roof = None
    if rank == 0 and not args.no_roofline:
        roof = eng.gemm_roofline(repeats=max(3, min(K, 10)))
    peaks, which = measured_peaks()

    if rank == 0:
        tokens = B * S * world
        value = tokens * K / (ms_dev / 1e3)
        line = {
            "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_dev / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "audit": "1 audited sample per rank-batch (p = 1/128), gradient-corrected, with distillation terms",
                       "global_batch": B * world, "seq_len": S, "parallelism": f"dp{world}",
                       "l2": "per-step working set (~1 GB of activations) exceeds the 126 MB L2; no explicit flush",
                       "timing": "CUDA events around K graph replays, max over ranks"},
            "e2e": {"value": tokens * K / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * S * 8 + (4 + B * 4 if eng.audit is not None else 0),
                    "d2h_bytes_per_step": eng._results.numel() * 4 + 4,
                    "api": "TrainEngine.train_steps(batches): two steps in flight, each step's loss read on the host",
                    "synchronous_train_step": tokens * K / (ms_e2e_sync / 1e3)},
            "gpu_launches": launches_timed,
            "clocks": clocks.summary(),
            "step_roofline": {"flops_per_token": step_flops_per_token(C3_MODEL),
                              "achieved_tflops": step_flops_per_token(C3_MODEL) * value / world / 1e12,
                              "peak_tflops": peaks["bf16_tflops_sustained"], "of": which},
        }
        if roof is not None:
            peak = peaks["bf16_tflops_sustained"]
            line["roofline"] = {"bound": "tensor", "achieved": roof["tflops"], "peak": peak, "unit": "TFLOP/s",
                                "frac": roof["tflops"] / peak,
                                # DRAM bytes per launch (read + write), launch-weighted mean over the nine hot-pass shapes of the
                                # ncu capture summarised in profiles/gemm_tcgen05_c3_shapes_ncu_full.md
                                "traffic": 38.0e6, "traffic_unit": "bytes per launch (ncu dram__bytes_read+write, 9 shapes)",
                                "of": which + " (sustained)",
                                "kernel": "gemm_tcgen05_kernel", "launches_per_step": roof["launches"],
                                "gemm_ms_per_step": roof["gemm_ms_per_step"],
                                "timing": "event-record nodes around each launch inside a captured step",
                                "scope": "hot-pass launches (main stream + its weight-gradient stream); the audit replay's "
                                         "few-row launches overlap them on their own streams and are listed under side_stream",
                                "per_shape": roof["per_shape"], "side_stream": roof.get("side_stream")}
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v, sample = cpu_port_tokens_per_sec(sample_batch=128, steps=32, threads=threads)     # the full step; ~12 s on 16 host cores
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
        _emit(json.dumps(line))
    eng.close()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
        # NCCL's teardown after graph-captured collectives has hung on this pool: the result is out, leave at once
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
