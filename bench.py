"""Benchmark of the `recursive_macro` training step (BASELINE metric: train tokens/sec).

    python bench.py --gpus 1 --steps 20 --warmup 5 [--config c3]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the reference's own CPU implementation of the same step on the host cores

One JSON line on stdout (rank 0).  `value` = device-timed whole-job tokens/sec with the batch already in HBM
(CUDA-graph replays between CUDA events, max over ranks; the median of `--repeats` timed regions of K steps);
`e2e` = the same through `TrainEngine.train_steps` with pinned HOST batches (H2D copy and loss read-back inside
the timed region); `roofline` = the tcgen05 GEMM (the dominant kernel) against the measured bf16 peak;
`cpu_baseline` = the reference (or its CPU restatement) on the host cores; `gpu_torch_baseline` = the reference's
own PyTorch step on this GPU (cuBLAS / SDPA, bf16 autocast), the number the kernels have to beat.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


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


def zipf_batches(vocab: int, B: int, S: int, n: int, seed: int, pin: bool):
    """Synthetic Zipf(1.1) token stream from a seeded CPU generator, cut into windows of S+1 with stride S
    (the reference's `batch_iterator`, utils.py:84-99)."""
    import torch

    ranks_ = torch.arange(1, vocab + 1, dtype=torch.float64)
    probs = (ranks_.pow(-1.1) / ranks_.pow(-1.1).sum()).float()
    gen = torch.Generator().manual_seed(seed)
    stream = torch.multinomial(probs, B * S * n + 1, replacement=True, generator=gen)
    out = []
    for i in range(n):
        win = stream[i * B * S: (i + 1) * B * S + 1]
        x, y = win[:-1].view(B, S).clone(), win[1:].view(B, S).clone()
        out.append((x.pin_memory(), y.pin_memory()) if pin else (x, y))
    return out


# --------------------------------------------------------------------------- the reference's own step
def reference_src() -> str | None:
    """Where the unmodified reference package can be imported from: $RTE_REFERENCE_SRC, the in-tree install
    (`baseline/_ref`, git-ignored) or a checkout beside the repository."""
    for cand in (os.environ.get("RTE_REFERENCE_SRC"), str(ROOT / "baseline" / "_ref"), str(ROOT.parent / "reference" / "src")):
        if cand and Path(cand, "recursive_training_engine", "training.py").exists():
            return cand
    return None


def reference_engine(raw: dict, device: str, precision: str):
    """The reference's `TrainEngine` (training.py:1628-1654) for a workload, with the benchmark's seeded N(0, 0.02)
    weights loaded in registration order.  Returns the engine; its `train_step((tokens, targets))` is the step."""
    import torch

    src = reference_src()
    if src is None:
        raise ImportError("reference package not found")
    if src not in sys.path:
        sys.path.insert(0, src)
    from recursive_training_engine import config as RC
    from recursive_training_engine.training import TrainEngine as RefEngine

    from speedup_thingy_b200.config import ModelConfig
    from speedup_thingy_b200.engine import init_parameters

    m = dict(raw["model"])
    full = ModelConfig(**m)                      # fills the fields the workload leaves at their defaults
    ref_model = {f: getattr(full, f) for f in ("topology", "vocab_size", "d_model", "n_heads", "d_ff", "n_dense_layers", "n_prelude",
                                              "n_coda", "t_max", "attn_banks", "ffn_banks", "head_groups", "ffn_groups",
                                              "active_head_groups", "active_ffn_groups", "recipe_count", "macro_rank")}
    ref_model["depth_choices"] = list(full.depth_choices)
    t = raw["train"]
    k = t.get("audit_fixed_count_per_batch")
    p = (k / t["batch_size"]) if k else 0.0
    tr = RC.TrainingConfig(
        mode=t["mode"], lr=t["lr"], weight_decay=t["weight_decay"], batch_size=t["batch_size"], seq_len=t["seq_len"],
        seed=t["seed"], precision=precision, fixed_depth=t.get("fixed_depth"), audit_p_min=p, audit_p_max=p, audit_alpha=0.0,
        audit_beta=0.0, audit_gamma=0.0, audit_fixed_count_per_batch=k, audit_mode="gradient_corrected" if k else "metric_only",
        audit_gradient_correction=bool(k), lambda_cons=0.0, fused_optimizer=False, foreach_optimizer=True,
        allow_tf32=False, log_every=10 ** 9)
    out = RC.OutputConfig(**raw["output"]) if raw.get("output") else RC.OutputConfig()
    import tempfile
    cfg = RC.ExperimentConfig(model=RC.ModelConfig(**ref_model), training=tr, output=out, run_name="bench",
                              output_dir=tempfile.mkdtemp(prefix="rte_bench_"))
    eng = RefEngine(cfg, device=torch.device(device))
    model = eng.recursive_model if eng.recursive_model is not None else eng.dense_model
    init = init_parameters(full, seed=t["seed"], num_clusters=out.num_clusters)
    with torch.no_grad():
        for name, param in model.named_parameters():
            if name in init and tuple(init[name].shape) == tuple(param.shape):
                param.copy_(init[name])
    return eng


def cpu_reference_tokens_per_sec(raw: dict, steps: int, threads: int, budget_s: float) -> dict:
    """The reference's CPU implementation of the step on the host cores: the unmodified `TrainEngine` when the
    package is importable (kind "reference"), else the CPU restatement under oracle/ (kind "port").  fp32 (the
    reference's CPU path; bf16 autocast on CPU is slower), `threads` torch threads, the full batch per step, one
    warm-up step, at most `steps` timed steps or `budget_s` seconds."""
    import torch

    torch.set_num_threads(threads)
    t = raw["train"]
    B, S, V = t["batch_size"], t["seq_len"], raw["model"]["vocab_size"]
    batches = zipf_batches(V, B, S, 4, seed=0, pin=False)
    kind = "reference"
    try:
        eng = reference_engine(raw, "cpu", "fp32")
        step = lambda b: float(eng.train_step(b).loss)          # noqa: E731
    except Exception as exc:                                      # reference not importable here: the restatement
        kind = f"port ({type(exc).__name__}: reference not importable)"
        from oracle import rte_oracle as O
        model = dict(raw["model"])
        oc = None
        if raw.get("output"):
            model["shortlist_clusters"] = raw["output"]["num_clusters"]
            oc = O.OutputCfg(**raw["output"])
        ocfg = O.ModelCfg(**model)
        trainer = O.OracleTrainer(ocfg, O.TrainCfg(**t), O.init_params(ocfg, seed=t["seed"]), oc=oc)
        step = lambda b: trainer.train_step(*b)                  # noqa: E731
    step(batches[0])
    times = []
    t_start = time.perf_counter()
    for i in range(max(steps, 1)):
        t0 = time.perf_counter()
        step(batches[(i + 1) % len(batches)])
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    med = statistics.median(times)
    return {"value": B * S / med, "unit": "tokens/s", "cores": threads, "kind": kind.split(" ")[0],
            "sample": f"{len(times)} steps of the full batch {B}x{S}, fp32, {threads} threads, median step {med * 1e3:.0f} ms"
                      + ("" if kind == "reference" else f"; {kind}")}


def gpu_torch_tokens_per_sec(raw: dict, dev, steps: int) -> dict:
    """The reference's own PyTorch step on this GPU (its `cuda_torch_fallback` path: cuBLAS GEMMs, SDPA attention,
    bf16 autocast over fp32 parameters, foreach AdamW): what the reference itself would do on this box."""
    import torch

    t = raw["train"]
    B, S, V = t["batch_size"], t["seq_len"], raw["model"]["vocab_size"]
    try:
        eng = reference_engine(raw, str(dev), "bf16")
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    batches = zipf_batches(V, B, S, 4, seed=0, pin=True)
    try:
        for i in range(3):
            eng.train_step(batches[i % 4])
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for i in range(steps):
            eng.train_step(batches[i % 4])
        torch.cuda.synchronize(dev)
        dt = (time.perf_counter() - t0) / steps
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    return {"value": B * S / dt, "unit": "tokens/s", "ms_per_step": dt * 1e3, "steps": steps,
            "what": "reference TrainEngine.train_step on cuda (PyTorch eager: cuBLAS + SDPA, bf16 autocast, host batches)"}


def run_reference(args, raw: dict) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    t = raw["train"]
    base = cpu_reference_tokens_per_sec(raw, steps=max(args.steps, 1), threads=threads, budget_s=150.0)
    value = base["value"]
    line = {"impl": "reference", "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": 1, "ms_per_step": 1000.0 * t["batch_size"] * t["seq_len"] / value,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": raw["title"], "note": "the reference's CPU implementation of the step on all host cores, the full "
                       "batch per step (median step time)"},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# --------------------------------------------------------------------------- stand-alone kernel probes (profiling)
def probe_gemm(iters: int, warmup: int, cublas: bool) -> None:
    """Stand-alone launches of the hot pass's GEMM shapes (one JSON line per shape): the small, fixed case the
    `ncu --set full` capture of the tcgen05 kernel is taken on.  Operands rotate over sets larger than L2; each shape
    is timed over a CUDA graph of `iters` launches, so host launch latency does not enter.  `cublas`: also time
    torch.matmul (cuBLAS) on the plain bf16 shapes, the vendor library's figure for the same product."""
    import torch

    from speedup_thingy_b200 import _abi as A
    from speedup_thingy_b200.ops import CudaOps
    from speedup_thingy_b200.workloads import WORKLOADS

    ops, dev = CudaOps("cuda:0"), "cuda:0"
    w = WORKLOADS["c3"]
    M, d, F, V = w["train"]["batch_size"] * w["train"]["seq_len"], w["model"]["d_model"], w["model"]["d_ff"], w["model"]["vocab_size"]
    bf, f32 = torch.bfloat16, torch.float32
    shapes = [  # name, M, N, K, a_mn, b_mn, epilogue, residual, splits
        ("qkv", M, 3 * d, d, 0, 0, A.EPI_BF16, False, 1), ("wo+residual", M, d, d, 0, 0, A.EPI_F32, True, 1),
        ("w_ug", M, 2 * F, d, 0, 0, A.EPI_BF16, False, 1), ("w_ug+swiglu", M, 2 * F, d, 0, 0, A.EPI_SWIGLU_FWD, False, 1),
        ("w_d+residual", M, d, F, 0, 0, A.EPI_F32, True, 1), ("logits", M, V, d, 0, 0, A.EPI_BF16, False, 1),
        ("dz=dy.w_d", M, F, d, 0, 1, A.EPI_BF16, False, 1), ("dz=dy.w_d+swiglu_bwd", M, F, d, 0, 1, A.EPI_SWIGLU_BWD, False, 1),
        ("dn=dug.w_ug", M, d, 2 * F, 0, 1, A.EPI_BF16, False, 1), ("dn=dqkv.w_qkv", M, d, 3 * d, 0, 1, A.EPI_BF16, False, 1),
        ("dy=du.w_o", M, d, d, 0, 1, A.EPI_BF16, False, 1), ("dw_ug", 2 * F, d, M, 1, 1, A.EPI_F32, False, 2),
        ("dw_d", d, F, M, 1, 1, A.EPI_F32, False, 4), ("dw_qkv", 3 * d, d, M, 1, 1, A.EPI_F32, False, 6),
        ("dw_o", d, d, M, 1, 1, A.EPI_F32, False, 16)]
    sets = 4

    def timed(fn) -> float:
        for i in range(max(warmup, 1)):
            fn(i % sets)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i % sets)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / iters

    for name, m, n, k, a_mn, b_mn, epi, res, splits in shapes:
        a = [torch.randn((k, m) if a_mn else (m, k), device=dev).to(bf) for _ in range(sets)]
        b = [(torch.randn((k, n) if b_mn else (n, k), device=dev) * 0.02).to(bf) for _ in range(sets)]
        kw = dict(M=m, N=n, K=k, a_mn=bool(a_mn), b_mn=bool(b_mn), epilogue=epi)
        extra = [dict() for _ in range(sets)]
        if epi == A.EPI_SWIGLU_FWD:
            out = [torch.empty(m, n // 2, device=dev, dtype=bf) for _ in range(sets)]
            extra = [dict(out2=torch.empty(m, n, device=dev, dtype=bf)) for _ in range(sets)]
            kw.update(pair=n // 2)
        elif epi == A.EPI_SWIGLU_BWD:
            out = [torch.empty(m, 2 * n, device=dev, dtype=bf) for _ in range(sets)]
            extra = [dict(residual=torch.randn(m, 2 * n, device=dev).to(bf)) for _ in range(sets)]
            kw.update(pair=n)
        else:
            out = [torch.empty(splits * m * n, device=dev, dtype=f32 if epi == A.EPI_F32 else bf) for _ in range(sets)]
            kw.update(ldc=n)
            if res:
                extra = [dict(residual=torch.randn(m, n, device=dev)) for _ in range(sets)]
        if splits > 1:
            kw.update(splits=splits, split_stride=m * n)
        us = timed(lambda i: ops.gemm(a[i], b[i], out[i], **extra[i], **kw))
        line = {"gemm": name, "M": m, "N": n, "K": k, "splits": splits, "us": round(us, 2), "tflops": round(2.0 * m * n * k / us / 1e6, 1)}
        if cublas and epi == A.EPI_BF16 and not a_mn:
            outs = [torch.empty(m, n, device=dev, dtype=bf) for _ in range(sets)]
            usc = timed(lambda i: torch.matmul(a[i], b[i] if b_mn else b[i].t(), out=outs[i]))
            line.update(cublas_us=round(usc, 2), cublas_tflops=round(2.0 * m * n * k / usc / 1e6, 1))
        print(json.dumps(line), flush=True)
    ops.check_status()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="c3", choices=["c1", "c2", "c3", "c4", "c5"],
                    help="BASELINE workload (default: c3 = configs[2], the configuration the metric is quoted on)")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each (median and spread reported)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-torch-baseline", action="store_true")
    ap.add_argument("--eager", action="store_true", help="launch kernels one by one instead of replaying the CUDA graph (profiling)")
    ap.add_argument("--no-roofline", action="store_true", help="skip the per-launch GEMM timing pass (profiling)")
    ap.add_argument("--probe-gemm", action="store_true", help="time the hot pass's GEMM shapes stand-alone and exit (profiling)")
    ap.add_argument("--probe-kernels", action="store_true",
                    help="time the memory-bound kernels of the step stand-alone against their algorithmic bytes and exit (profiling)")
    ap.add_argument("--dp-timeline", action="store_true",
                    help="data parallel: add the start / end of every gradient bucket's all-reduce inside a step (profiling)")
    ap.add_argument("--step-timeline", metavar="FILE", default=None,
                    help="write start and duration of every C-ABI call of one captured step, per stream, as JSON lines (profiling; 1 GPU)")
    ap.add_argument("--join-waits", action="store_true",
                    help="also report how long the hot pass idles where it waits for the audit replay (event nodes at those waits only)")
    ap.add_argument("--probe-cublas", action="store_true", help="with --probe-gemm: also time torch.matmul (cuBLAS) on the same shapes")
    ap.add_argument("--probe-iters", type=int, default=20)
    ap.add_argument("--probe-warmup", type=int, default=3)
    args = ap.parse_args()
    if args.probe_gemm:
        probe_gemm(args.probe_iters, args.probe_warmup, args.probe_cublas)
        return
    if args.probe_kernels:
        from speedup_thingy_b200.kernel_probe import probe_kernels
        probe_kernels(args.probe_iters, args.probe_warmup, measured_peaks()[0]["hbm_gbs"])
        return

    from speedup_thingy_b200.workloads import train_flops_per_token, workload

    cfg, raw = workload(args.config)
    if args.impl == "reference":
        run_reference(args, raw)
        return

    import torch

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
        # plain ring / tree collectives: a rank that leaves while its buffers are bound to an NVLink multicast object
        # can fault its peers, and the buckets here are far from the sizes where in-switch reduction pays
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    B, S = cfg.training.batch_size, cfg.training.seq_len
    params = init_parameters(cfg.model, seed=0, num_clusters=cfg.output.num_clusters)
    kw = {"process_group": dist.group.WORLD} if world > 1 else {}
    eng = TrainEngine(cfg, params, device=dev, use_cuda_graph=not args.eager, **kw)
    n_batches = 8
    host_batches = zipf_batches(cfg.model.vocab_size, B, S, n_batches, seed=rank, pin=True)     # per-rank stream

    W, K, R = max(args.warmup, 3), args.steps, max(args.repeats, 1)
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

    def reduce_max(vals: list[float]) -> list[float]:
        if dist is None:
            return vals
        t = torch.tensor(vals, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t]

    # ---- device-timed: batch resident in HBM, R regions of K replays of the whole-step graph
    eng._load_batch(host_batches[0])
    clocks.mark()
    try:
        ms_regions = []
        launches_timed = 0
        for _ in range(R):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0 = eng.ops.launches
            e0.record()
            for _ in range(K):
                eng._run_step_kernels(optimizer=True)
            e1.record()
            barrier()
            ms_regions.append(e0.elapsed_time(e1))
            # C-ABI launches inside one timed region: counted directly when eager, per captured step when replayed
            launches_timed = (eng.ops.launches - l0) or (eng.kernel_launches_per_step or 0) * K
        ms_regions = reduce_max(ms_regions)                       # per region: the slowest rank
        ms_dev = statistics.median(ms_regions)
        # ---- end to end through the public API with pinned host batches
        # (a) the pipelined loop (`train_steps`: two steps in flight; every step copies its batch in and its results
        # out, and every step's loss is read on the host), (b) one synchronous `train_step` call per batch
        e2e_regions = []
        for _ in range(R):
            barrier()
            t0 = time.perf_counter()
            losses = [r.loss for r in eng.train_steps(host_batches[i % n_batches] for i in range(K))]
            torch.cuda.synchronize()
            e2e_regions.append((time.perf_counter() - t0) * 1e3)
            assert len(losses) == K and all(math.isfinite(x) for x in losses)
        barrier()
        t0 = time.perf_counter()
        for i in range(K):
            eng.train_step(host_batches[i % n_batches])
        torch.cuda.synchronize()
        ms_e2e_sync = (time.perf_counter() - t0) * 1e3
        e2e_regions = reduce_max(e2e_regions)
        ms_e2e_sync = reduce_max([ms_e2e_sync])[0]
        ms_e2e = statistics.median(e2e_regions)
        # The timed loops may be shorter than nvidia-smi's sampling period: keep the same step running (untimed)
        # for about half a second so that a few clock samples under this load exist (same count on every rank).
        for i in range(max(1, min(400, int(500.0 / max(ms_e2e / K, 0.1))))):
            eng.train_step(host_batches[i % n_batches])
        torch.cuda.synchronize()
    finally:
        clocks.__exit__(None, None, None)
    eng.ops.check_status()

    timeline = eng.dp_timeline() if (args.dp_timeline and world > 1) else None     # every rank takes part
    if args.step_timeline and world == 1:
        prof = eng.profile_step(repeats=3)
        with open(args.step_timeline, "w") as fh:
            for (name, us), start, where in zip(prof, eng.last_profile_starts, eng.last_profile_streams):
                fh.write(json.dumps({"call": name.split("@")[0], "stream": where, "start_us": round(start, 1), "us": round(us, 2)}) + "\n")

    join_waits = eng.join_waits() if (args.join_waits and world == 1) else None

    # ---- roofline of the dominant kernel (the tcgen05 GEMM): CUDA-event nodes around every launch of a captured step
    roof = None
    if rank == 0 and not args.no_roofline:
        roof = eng.gemm_roofline(repeats=max(3, min(K, 10)))
    peaks, which = measured_peaks()

    if rank == 0:
        tokens = B * S * world
        value = tokens * K / (ms_dev / 1e3)
        fpt = train_flops_per_token(cfg)
        audit_note = (f"{eng.audit_k} audited sample(s) per rank-batch (p = {eng.audit_k}/{B}), gradient-corrected, with distillation terms"
                      if eng.audit_k else "no audit")
        line = {
            "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_dev / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": raw["title"], "audit": audit_note,
                       "global_batch": B * world, "seq_len": S, "parallelism": f"dp{world}",
                       "l2": "per-step working set (~1 GB of activations) exceeds the 126 MB L2; no explicit flush",
                       "timing": f"CUDA events around K graph replays, max over ranks; median of {R} regions"},
            "timed_regions_ms_per_step": {"median": ms_dev / K, "min": min(ms_regions) / K, "max": max(ms_regions) / K,
                                          "all": [m / K for m in ms_regions]},
            "e2e": {"value": tokens * K / (ms_e2e / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": 2 * B * S * 8 + (4 * eng.audit_k + B * 4 if eng.audit is not None else 0),
                    "d2h_bytes_per_step": eng._results.numel() * 4 + 4,
                    "api": "TrainEngine.train_steps(batches): two steps in flight, each step's loss read on the host",
                    "regions_ms_per_step": [m / K for m in e2e_regions],
                    "synchronous_train_step": tokens * K / (ms_e2e_sync / 1e3)},
            "gpu_launches": launches_timed,
            "clocks": clocks.summary(),
            "step_roofline": {"flops_per_token": fpt, "achieved_tflops": fpt * value / world / 1e12,
                              "peak_tflops": peaks["bf16_tflops"], "frac": fpt * value / world / 1e12 / peaks["bf16_tflops"],
                              "of": which + " (burst)"},
        }
        if roof is not None:
            peak = peaks["bf16_tflops"]            # the timed region is tens of milliseconds at full clock: burst figure
            line["roofline"] = {"bound": "tensor", "achieved": roof["tflops"], "peak": peak, "unit": "TFLOP/s",
                                "frac": roof["tflops"] / peak,
                                "frac_of_sustained": roof["tflops"] / peaks["bf16_tflops_sustained"],
                                "peak_sustained": peaks["bf16_tflops_sustained"],
                                # DRAM bytes per launch (read + write), mean over the hot-pass shapes of the ncu capture
                                # summarised in profiles/gemm_tcgen05_c3_shapes_ncu_full.md (cold operand reads; outputs that
                                # fit the L2 do not reach DRAM inside the launch); only meaningful for workload c3
                                "traffic": 41.0e6 if args.config == "c3" else None,
                                "traffic_unit": "bytes per launch (ncu dram__bytes_read+write, c3 shapes)",
                                "of": which + " (burst)",
                                "kernel": "gemm_tcgen05_kernel", "launches_per_step": roof["launches"],
                                "gemm_ms_per_step": roof["gemm_ms_per_step"],
                                "timing": "event-record nodes around each launch inside a captured step",
                                "scope": "hot-pass launches (main stream + its weight-gradient stream); the audit replay's "
                                         "few-row launches overlap them on their own streams and are listed under side_stream",
                                "per_shape": roof["per_shape"], "side_stream": roof.get("side_stream")}
        if timeline is not None:
            line["dp_timeline"] = timeline
        if join_waits is not None:
            line["replay_join_waits"] = join_waits
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            line["cpu_baseline"] = cpu_reference_tokens_per_sec(raw, steps=6, threads=threads, budget_s=40.0)
        if world == 1 and not args.no_torch_baseline:
            line["gpu_torch_baseline"] = gpu_torch_tokens_per_sec(raw, dev, steps=10)
        _emit(json.dumps(line))

    # ---- orderly teardown (graphs that captured collectives must be gone before the communicator is destroyed)
    if dist is not None:
        from speedup_thingy_b200.engine import teardown_data_parallel
        teardown_data_parallel(eng)
    else:
        eng.close()

if __name__ == "__main__":
    main()
