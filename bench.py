#!/usr/bin/env python
"""Benchmark of the decay-rule (LFW) hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload train|decode|long|dfw|gpt2|seqsplit]
                    [--gates raw_f1|raw|sigmoid] [--impl ours|reference] [--ckpt-every C]

Workloads: train (default, below), decode (T=1, B*H=4096), long (B*H=16, T=16384, D=K=128), dfw (the delta
rule at the default shape), gpt2 (GPT-2-small with every attention replaced, whole training step),
seqsplit (16 rows of 65 536 steps with the TIME axis split over the GPUs; strong scaling).

Default workload ("train"): one LFW layer at GPT-2-small shape, fp16, B*H=96, T=1024,
D=K=64, x,q,k,f_key ~ N(0,1) with q,k scaled by 1/8, forget gate f = 1, zero initial state;
a step is one forward + backward over the whole batch.  Prints ONE JSON line on stdout
(rank 0):

  value ..... tokens/s with the inputs resident in HBM, kernels called through the C ABI,
              timed with CUDA events over exactly K steps, max over ranks
  e2e ....... the same metric through LFWFunction.apply with HOST (pinned) inputs: every step
              copies the six inputs to the device, runs forward + backward through autograd and
              copies outputs, next state and the six gradients back (three steps in flight on
              three streams; the region is timed several times and the median is reported)
  roofline .. algorithmic bytes of the slower of the two calls (forward / backward) over its
              measured duration, against the measured HBM copy bandwidth
  value_api . the same step through LFWFunction.apply + autograd with device-resident tensors,
              eager and replayed from a CUDA graph
  extra.decode  the T=1 decode step (B*H=4096) measured in the same run: us/step over 1000 chained
              steps through the allocation-free decode loop (graph replay), GB/s and fraction
  cpu_baseline  the reference's own TorchScript CPU path (oracle/_ref, placed there by
              oracle/make_ref.py; kind "reference") or, where that is absent, its restatement
              oracle/torch_port.py (kind "port"), on this machine's host cores, on a bounded sample
  strong .... (N > 1) the same workload with its batch*head rows split over the ranks

`--impl reference` times that CPU path alone on the whole workload (all rows; the row count is
reduced, and said so, only if K+W calls would not finish within a few minutes) and prints the
same line with "impl": "reference".  Under torchrun each rank runs the full workload on its own
GPU (weak scaling, no collective on the data path); rank 0 reports the aggregate.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, T, D, K)
    "train": (96, 1024, 64, 64),     # single layer, GPT-2-small shape, fwd + bwd
    "decode": (4096, 1, 64, 64),     # T=1 decode step, GPT-2-medium heads x batch 256
    "long": (16, 16384, 128, 128),   # long-sequence prefill + backward
    "dfw": (96, 1024, 64, 64),       # delta rule (DFWFunction), GPT-2-small shape, fwd + bwd
    "gpt2": (96, 1024, 64, 64),      # GPT-2-small, every attention replaced by a fast-weight layer:
                                     # batch 8 x 12 heads per GPU, whole training step (run_gpt2)
    "seqsplit": (16, 65536, 64, 64), # one long sequence per row, its TIME axis split over the GPUs
                                     # (t2fw_b200/seq_parallel.py; strong scaling, run_seqsplit)
}
CPU_SAMPLE_ROWS = {"train": 16, "decode": 4096, "long": 1, "dfw": 16}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--workload", default="train", choices=sorted(WORKLOADS))
    p.add_argument("--gates", default="raw_f1", choices=["raw_f1", "raw", "sigmoid"])
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--e2e-slots", type=int, default=3,
                   help="steps in flight in the end-to-end loop (sets of device tensors and pinned result buffers)")
    p.add_argument("--e2e-blocks", type=int, default=9, help="timed repetitions of the end-to-end region; the median is reported")
    p.add_argument("--e2e-separate-inputs", action="store_true",
                   help="end-to-end loop: one host->device copy per input tensor instead of one copy of the pinned arena "
                        "that holds them all")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--ckpt-every", type=int, default=0,
                   help="checkpoint interval of the C-ABI calls (0: the library's default, 64; "
                        "BASELINE config 4 names 128)")
    p.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                   help="weak: every GPU runs the workload's batch rows; strong: the rows are split over the GPUs")
    p.add_argument("--rule", default="dfw", choices=["dfw", "lfw"],
                   help="recurrence inside the gpt2 workload's attention replacement")
    p.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                   help="replay the K timed steps as one CUDA graph (auto: on)")
    return p.parse_args()


def make_inputs(torch, B, T, D, K, gates, seed, workload):
    g = torch.Generator().manual_seed(seed)
    if workload == "dfw":      # q, k, v, zero state, upstream gradients
        q = torch.randn(B, T, K, generator=g) / math.sqrt(K)
        k = torch.randn(B, T, K, generator=g) / math.sqrt(K)
        v = torch.randn(B, T, D, generator=g)
        return [q, k, v, torch.zeros(B, D, K), torch.randn(B, T, D, generator=g),
                torch.randn(B, D, K, generator=g)]
    x = torch.randn(B, T, D, generator=g)
    q = torch.randn(B, T, K, generator=g) / math.sqrt(K)
    k = torch.randn(B, T, K, generator=g) / math.sqrt(K)
    fk = torch.randn(B, T, K, generator=g)
    if gates == "sigmoid":
        fk = torch.sigmoid(fk)
    if gates == "raw_f1":
        f = torch.ones(B, T, D)
    else:
        f = torch.sigmoid(torch.randn(B, T, D, generator=g))
    if workload == "train":
        s = torch.zeros(B, D, K)
    else:
        s = torch.randn(B, D, K, generator=g) * 0.1
    go = torch.randn(B, T, D, generator=g)
    gs = torch.randn(B, D, K, generator=g)
    return [x, f, q, k, fk, s, go, gs]


def algorithmic_bytes(B, T, D, K, e=2):
    """Bytes the recurrence must move (fp16 I/O), excluding checkpoints and scratch."""
    n = B * T
    fwd = e * (n * (2 * D + 3 * K) + n * D + 2 * B * D * K)
    bwd = e * (n * D + 2 * n * (2 * D + 3 * K) + 3 * B * D * K)
    return fwd, bwd


def algorithmic_bytes_dfw(B, T, D, M, e=2):
    """Delta rule: q, k [N,M], v [N,D] in, outputs out, state in/out; the saved delta is not counted."""
    n = B * T
    fwd = e * (n * (2 * M + D) + n * D + 2 * B * D * M)
    bwd = e * (n * D + 2 * n * (2 * M + D) + 3 * B * D * M)
    return fwd, bwd


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples taken while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                c = [t.strip() for t in line.split(",")]
                if len(c) < 9:
                    continue
                try:
                    sm.append(float(c[1]))
                    mx.append(float(c[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), c[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def cpu_reference_run(workload, gates, steps, warmup, seed, rows=None, budget_s=None):
    """Times the reference's CPU path (oracle/_ref when present, else oracle/torch_port) on the host
    cores.  rows=None: the workload's bounded sample; budget_s: shrink the row count so that
    warmup + steps calls fit the budget.  Returns (tokens/s, description dict)."""
    import torch
    from oracle import make_ref, torch_port

    ref = make_ref.load()
    B, T, D, K = WORKLOADS[workload]
    rows = min(B, rows if rows is not None else CPU_SAMPLE_ROWS[workload])
    # launchers such as torchrun pin OMP_NUM_THREADS=1; the CPU baseline uses every host core
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    full = make_inputs(torch, B, T, D, K, gates, seed, workload)

    def one_call(ins):
        if workload == "dfw":
            if ref is None:
                return torch_port.dfw_fwd_bwd(*ins)
            leaves = [t.detach().clone().requires_grad_(True) for t in ins[:4]]
            out, fin = ref.t2dfw_torch(*leaves)
            return torch.autograd.grad([out, fin], leaves, [ins[4], ins[5]])
        x, f, q, k, fk, s, go, gs = ins
        if workload == "decode":
            with torch.no_grad():
                return (ref.t2fw_torch if ref is not None else torch_port.lfw_loop)(x, f, q, k, fk, s)
        if ref is None:
            return torch_port.lfw_fwd_bwd(x, f, q, k, fk, s, go, gs)
        leaves = [t.detach().clone().requires_grad_(True) for t in (x, f, q, k, fk, s)]
        out, fin = ref.t2fw_torch(*leaves)
        return torch.autograd.grad([out, fin], leaves, [go, gs])

    shrunk = None
    while True:
        ins = [t[:rows].contiguous() for t in full]
        times = []
        restart = False
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            one_call(ins)
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt)
            if budget_s is not None and i == 0 and dt * (warmup + steps) > budget_s and rows > 8:
                shrunk = rows
                rows = max(8, int(rows * budget_s / (dt * (warmup + steps))))
                restart = True
                break
        if not restart:
            break
    med = statistics.median(times)
    value = rows * T / med
    desc = {
        "value": value, "unit": "tokens/s", "cores": torch.get_num_threads(),
        "host_cpus": os.cpu_count(), "kind": "reference" if ref is not None else "port",
        "sample": "%d of %d batch rows%s, T=%d, D=K=%d, fp32, %s; median of %d calls after %d warm-up; %s"
                  % (rows, B, "" if shrunk is None else " (reduced from %d to fit the time budget)" % shrunk,
                     T, D, "forward only" if workload == "decode" else "forward+backward", len(times), warmup,
                     "the reference's TorchScript functions (t2fw/torch.py) + autograd" if ref is not None
                     else "oracle/torch_port.py (the reference module is not present)"),
        "s_per_call": med, "rows": rows,
    }
    return value, desc


def run_gpt2(args):
    """The end-to-end configuration: GPT-2-small (12 layers, d_model 768, 12 heads, 124 M parameters, random
    init), every attention replaced by a fast-weight layer, fp16, sequence 1024, batch 8 per GPU,
    random token ids; one step = forward + backward + DDP gradient all-reduce + AdamW update."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from t2fw_b200 import _lib
    from t2fw_b200.gpt2_fw import GPT2FW, GPT2FWConfig
    from t2fw_b200.parallel import job_throughput, max_over_ranks

    lib = _lib.load_core()
    torch.manual_seed(args.seed)                       # same initial weights on every rank
    cfg = GPT2FWConfig(rule=args.rule)
    model = GPT2FW(cfg).half().to(dev)
    n_params = model.n_params()
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], gradient_as_bucket_view=True)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, eps=1e-4, fused=True)
    bsz, T = 8, cfg.n_positions
    g = torch.Generator().manual_seed(args.seed + 1 + rank)
    host_ids = [torch.randint(0, cfg.vocab_size, (bsz, T + 1), generator=g).pin_memory() for _ in range(4)]
    dev_ids = [h.to(dev) for h in host_ids]

    def step(ids):
        loss = net(ids[:, :-1], targets=ids[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ev = lambda: torch.cuda.Event(enable_timing=True)
    first = None
    for i in range(args.warmup):
        loss = step(dev_ids[i % 4])
        first = float(loss.detach()) if first is None else first
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = lib.t2fw_launch_count()
    t0, t1 = ev(), ev()
    t0.record()
    for i in range(args.steps):
        loss = step(dev_ids[(args.warmup + i) % 4])
    t1.record()
    barrier()
    launches = lib.t2fw_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    total_ms = max_over_ranks(t0.elapsed_time(t1), dev)
    value = job_throughput(bsz * T * args.steps, world, total_ms)
    last = float(loss.detach())

    # end to end: token ids come from pinned host memory and the loss is read back every step
    e2e_steps = max(3, min(args.steps, 10))
    e0, e1 = ev(), ev()
    barrier()
    e0.record()
    for i in range(e2e_steps):
        ids = host_ids[i % 4].to(dev, non_blocking=True)
        loss_host = step(ids).item()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), dev)
    e2e = {"value": bsz * T * e2e_steps * world / (e2e_ms * 1e-3), "unit": "tokens/s",
           "h2d_bytes_per_step": host_ids[0].numel() * 8, "d2h_bytes_per_step": 4, "steps": e2e_steps,
           "ms_per_step": e2e_ms / e2e_steps, "api": "GPT2FW forward + loss.backward() + AdamW step"}
    if rank != 0:
        dist.destroy_process_group()
        return
    flops = 6.0 * n_params * bsz * T                      # matrix-multiply work of the dense layers
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            peak, peak_kind = float(json.load(fh)["bf16_tflops_sustained"]), "measured sustained cuBLAS bf16"
    except Exception:
        peak, peak_kind = 1400.0, "fallback sustained cuBLAS bf16"
    ms = total_ms / args.steps
    achieved = flops / (ms * 1e-3) / 1e12
    line = {
        "metric": "gpt2_small_fw_train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 parameters and activations, f32 recurrence state",
        "data": "synthetic",
        "config": {"workload": "gpt2: GPT-2-small (12 layers, d_model 768, 12 heads, %.1f M parameters, random init), "
                               "every attention replaced by a %s layer, seq 1024, batch 8 per GPU, uniform random "
                               "token ids; forward + backward + AdamW" % (n_params / 1e6, args.rule.upper()),
                   "parallelism": "dp%d (DistributedDataParallel, NCCL all-reduce of gradients)" % world,
                   "l2": "activations of a step (several GB) are larger than L2",
                   "loss_first": first, "loss_last": last},
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "traffic": None, "peak_kind": peak_kind,
                     "kernel": "whole training step, counted as 6 x parameters x tokens dense FLOPs"},
        "cpu_baseline": None,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_seqsplit(args):
    """B*H = 16 rows of 65 536 steps (D = K = 64, fp16), forward + backward through
    LFWSeqParallelFunction: every GPU holds T / N steps of every row and the ranks exchange one segment
    summary per direction (two all-gathers of 16 x 4 224 floats per rank and one all-reduce).  Strong
    scaling: the job is the same at every N; at N = 1 the exchange degenerates to the rank itself."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world == 1:      # the function needs a process group even for one rank
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
    import datetime
    # a short collective timeout: a rank that fails leaves the others with an error, not a long wait
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=180))
    from t2fw_b200 import _lib
    from t2fw_b200.parallel import max_over_ranks
    from t2fw_b200.seq_parallel import LFWSeqParallelFunction

    lib = _lib.load_core()
    B, T, D, K = WORKLOADS["seqsplit"]
    Tr = T // world
    g = torch.Generator().manual_seed(args.seed + 7 * rank)
    def rnd(*shape):
        return torch.randn(*shape, generator=g)
    # two input sets (each rank's segment: 5 x 16 x T/N x 64 x 2 bytes), sigmoid gates on both sides
    sets = []
    for _ in range(2):
        x, q, k = rnd(B, Tr, D), rnd(B, Tr, K) / 8, rnd(B, Tr, K) / 8
        f, fk = torch.sigmoid(rnd(B, Tr, D) + 2), torch.sigmoid(rnd(B, Tr, K) + 2)
        go = rnd(B, Tr, D)
        sets.append([t.half().to(dev) for t in (x, f, q, k, fk, go)])
    state = torch.zeros(B, D, K, dtype=torch.float16, device=dev)
    gfin = (torch.randn(B, D, K, generator=g) / world).half().to(dev)

    def step(i):
        x, f, q, k, fk, go = sets[i & 1]
        leaves = [t.requires_grad_(True) for t in (x, f, q, k, fk)] + [state.clone().requires_grad_(True)]
        out, fin = LFWSeqParallelFunction.apply(*leaves)
        return torch.autograd.grad([out, fin], leaves, [go, gfin])

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()

    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    clk = ClockSampler(local)
    clk.start()
    l0 = lib.t2fw_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    launches = lib.t2fw_launch_count() - l0
    clocks = clk.stop()
    ms = max_over_ranks(e0.elapsed_time(e1), dev) / args.steps
    if rank == 0:
        esz = 2
        algo = esz * (B * T * (2 * D + 3 * K) + B * T * D + 2 * B * D * K) + esz * (B * T * D + 2 * B * T * (2 * D + 3 * K) + 3 * B * D * K)
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
                peak, peak_kind = float(json.load(fh)["hbm_gbs"]), "measured copy bandwidth"
        except Exception:
            peak, peak_kind = 6650.0, "fallback copy bandwidth"
        achieved = algo / world / (ms * 1e-3) / 1e9        # per GPU
        print(json.dumps({
            "metric": "lfw_fwd_bwd_tokens_per_s", "value": B * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 state arithmetic, f16 I/O", "data": "synthetic",
            "config": {"workload": "seqsplit: LFW forward+backward, B*H=%d rows of T=%d steps, D=K=64, fp16; the time axis "
                                   "split over the GPUs (%d steps per GPU), sigmoid gates on both sides" % (B, T, Tr),
                       "api": "t2fw_b200.seq_parallel.LFWSeqParallelFunction.apply + torch.autograd.grad (eager)",
                       "exchange": "per step and rank: 2 all-gathers of %d bytes, 1 all-reduce of %d bytes (NCCL)"
                                   % (B * (D * K + D + K) * 4, B * D * K * 4),
                       "l2": "two alternating input sets; one segment set is %.0f MB" % (6 * B * Tr * 64 * 2 / 1e6)},
            "clocks": clocks, "e2e": None, "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind,
                         "kernel": "whole step per GPU (summaries, exchange, forward and backward kernels)"},
            "cpu_baseline": None}))
    dist.destroy_process_group()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload == "seqsplit":
        print(json.dumps({"impl": "reference", "unavailable": "the reference has no multi-device code; the "
                          "time-split workload is measured against the unsplit run of the same library"}))
        return
    if args.workload == "gpt2":
        print(json.dumps({"impl": "reference", "unavailable": "the reference ships no model: the end-to-end "
                          "GPT-2 configuration has no reference implementation and no CPU baseline"}))
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    B, T, D, K = WORKLOADS[args.workload]
    # the whole workload (all batch rows), the requested number of calls; the row count is reduced
    # only if those calls would not finish within a few minutes on this host
    rows = B if args.workload in ("train", "decode", "dfw") else CPU_SAMPLE_ROWS[args.workload]
    value, desc = cpu_reference_run(args.workload, args.gates, steps, warmup, args.seed, rows=rows, budget_s=300.0)
    line = {
        "impl": "reference", "metric": metric_name(args.workload), "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": desc["s_per_call"] * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, B, T, D, K),
        "cpu_baseline": desc,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(workload):
    return {"train": "lfw_fwd_bwd_tokens_per_s", "decode": "lfw_decode_tokens_per_s",
            "long": "lfw_fwd_bwd_tokens_per_s", "dfw": "dfw_fwd_bwd_tokens_per_s"}[workload]


def workload_config(args, B, T, D, K):
    if args.workload == "dfw":
        return {"workload": "dfw: DFW (delta rule) forward+backward, B*H=%d per GPU, T=%d, D=M=%d, fp16 I/O, "
                            "fp32 state arithmetic" % (B, T, D),
                "inputs": "q, k ~ N(0,1)/sqrt(M), v ~ N(0,1), zero initial state",
                "sharding": "batch*head rows split across GPUs, no collective"}
    return {
        "workload": "%s: LFW %s, B*H=%d per GPU, T=%d, D=K=%d, fp16 I/O, fp32 state arithmetic"
                    % (args.workload, "forward (decode step)" if args.workload == "decode"
                       else "forward+backward", B, T, D),
        "gates": {"raw_f1": "f=1, f_key~N(0,1)", "raw": "f=sigmoid(N(0,1)), f_key~N(0,1)",
                  "sigmoid": "f, f_key = sigmoid(N(0,1))"}[args.gates],
        "sharding": "batch*head rows split across GPUs, no collective",
    }


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from t2fw_b200 import _lib, cabi
    from t2fw_b200.decode import LFWDecodeLoop
    from t2fw_b200.functional_dfw import DFWFunction
    from t2fw_b200.functional_lfw import LFWFunction
    from t2fw_b200.parallel import bind_host_to_gpu_node, max_over_ranks, row_shard

    # several ranks on one box: each rank's pinned host buffers and copy threads on its GPU's own
    # NUMA node (matters for the end-to-end leg only; a no-op where the topology is not visible)
    host_binding = bind_host_to_gpu_node(local) if world > 1 else None

    lib = _lib.load_core()
    B, T, D, K = WORKLOADS[args.workload]
    if args.scaling == "strong":        # contiguous share of the batch x head rows for this rank
        r0, r1 = row_shard(B, world, rank)
        B = r1 - r0
        if B == 0:
            raise SystemExit("bench.py: more GPUs than batch rows")
    rows_all = WORKLOADS[args.workload][0] if args.scaling == "strong" else B * world
    decode = args.workload == "decode"
    dfw = args.workload == "dfw"
    dtype = torch.float16

    # Rotating input sets so that consecutive steps never find their data in the 126 MB L2.
    touched = 2 * (B * T * (3 * D + 3 * K) + 3 * B * D * K) * (1 if decode else 2)
    n_sets = max(2, min(8, int(math.ceil(500e6 / touched))))
    base = [t.to(dtype).to(dev).contiguous() for t in
            make_inputs(torch, B, T, D, K, args.gates, args.seed + 1000 * rank, args.workload)]
    # distinct data per set without regenerating on the host: roll along the batch axis
    sets = [base] + [[t.roll(i, 0).contiguous() for t in base] for i in range(1, n_sets)]

    C = args.ckpt_every if args.ckpt_every > 0 else cabi.ckpt_every_for(T, D, K, dtype)
    code = cabi.dtype_code(base[0])
    if not dfw:
        slots = int(lib.t2fw_lfw_ckpt_slots(T, C))
        outs = [torch.empty(B, T, D, dtype=dtype, device=dev) for _ in range(n_sets)]
        ckpts = [torch.empty(B, slots, D, K, dtype=dtype, device=dev) for _ in range(n_sets)]
        grads = None if decode else [[torch.empty_like(t) for t in s[:6]] for s in sets]
        fsb = lib.t2fw_lfw_forward_scratch_bytes(B, T, D, K, code, C)
        bsb = lib.t2fw_lfw_backward_scratch_bytes(B, T, D, K, code, C)
        fscr = torch.empty(max(fsb, 1), dtype=torch.uint8, device=dev)
        bscr = torch.empty(max(bsb, 1), dtype=torch.uint8, device=dev)
    else:
        bsb = lib.t2fw_dfw_backward_scratch_bytes(B, T, D, K, code)
        bscr = torch.empty(max(bsb, 1), dtype=torch.uint8, device=dev)

    ev = lambda: torch.cuda.Event(enable_timing=True)
    fwd_ms, bwd_ms = [], []

    # fwd_call(i) runs the forward of step i and returns what its backward needs
    if dfw:
        def fwd_call(i):
            q, k, v, s, go, gs = sets[i % n_sets]
            _, fin, delta = cabi.dfw_forward(q, k, v, s)
            return fin, delta

        def bwd_call(i, saved):
            q, k, v, s, go, gs = sets[i % n_sets]
            cabi.dfw_backward(go, gs, q, k, saved[1], saved[0], scratch=bscr)
    elif decode:
        # chained decode: each set's state advances every time the set comes round; the new
        # state is written to the set's other buffer (inputs are never overwritten in place)
        state_a = [s[5] for s in sets]
        state_b = [torch.empty_like(s[5]) for s in sets]

        def fwd_call(i):
            j = i % n_sets
            x, f, q, k, fk = sets[j][:5]
            even = (i // n_sets) % 2 == 0
            src, dst = (state_a[j], state_b[j]) if even else (state_b[j], state_a[j])
            cabi.lfw_forward(x, f, q, k, fk, src, ckpt_every=C, out=outs[j],
                             ckpt=dst.view(B, 1, D, K), scratch=fscr)

        bwd_call = None
    else:
        def fwd_call(i):
            j = i % n_sets
            x, f, q, k, fk, s, go, gs = sets[j]
            cabi.lfw_forward(x, f, q, k, fk, s, ckpt_every=C, out=outs[j], ckpt=ckpts[j], scratch=fscr)

        def bwd_call(i, saved):
            j = i % n_sets
            x, f, q, k, fk, s, go, gs = sets[j]
            cabi.lfw_backward(go, gs, x, f, q, k, fk, s, ckpts[j], ckpt_every=C, grads=grads[j],
                              scratch=bscr)

    def step(i, record=None):
        if record:
            record[0].record()
        saved = fwd_call(i)
        if record:
            record[1].record()
        if bwd_call is not None:
            bwd_call(i, saved)
            if record:
                record[2].record()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = lib.t2fw_launch_count()
    t_start, t_end = ev(), ev()
    graph = None
    if args.graph != "off":
        # the K steps as one CUDA graph: the host's launch cost stays out of the timed region
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(args.steps):
                    step(args.warmup + i)
            graph.replay()
            barrier()
        except Exception as exc:  # capture not possible: time eager launches instead
            sys.stderr.write("bench.py: graph capture failed (%s); timing eager launches\n" % exc)
            graph = None
            torch.cuda.synchronize()
    launches = lib.t2fw_launch_count() - launches0
    if graph is not None:
        t_start.record()
        graph.replay()
        t_end.record()
        barrier()
    else:
        launches0 = lib.t2fw_launch_count()
        t_start.record()
        for i in range(args.steps):
            step(args.warmup + i)
        t_end.record()
        barrier()
        launches = lib.t2fw_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_start.elapsed_time(t_end)
    # per-call split (forward / backward): the forward calls and the backward calls of n_split steps
    # as one CUDA graph each, so that host launch gaps stay out of the durations; an eager pass with
    # events around each call where capture is not possible
    n_split = min(args.steps, 10)
    split_kind = "one CUDA graph per call kind"
    try:
        if args.graph == "off":
            raise RuntimeError("graphs off")
        saved = [fwd_call(args.warmup + i) for i in range(n_split)]
        barrier()

        def timed_graph(fn):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(n_split):
                    fn(i)
            g.replay()
            torch.cuda.synchronize()
            a, b = ev(), ev()
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / n_split

        if decode and graph is not None:
            fwd_ms.append(total_ms / args.steps)      # the timed step is the forward call itself
        else:
            fwd_ms.append(timed_graph(lambda i: fwd_call(args.warmup + i)))
        if bwd_call is not None:
            bwd_ms.append(timed_graph(lambda i: bwd_call(args.warmup + i, saved[i])))
        barrier()
    except Exception:
        split_kind = "eager launches with events (host launch gaps included)"
        torch.cuda.synchronize()
        del fwd_ms[:], bwd_ms[:]
        records = [[ev(), ev(), ev()] for _ in range(n_split)]
        for i in range(n_split):
            step(args.warmup + i, records[i])
        barrier()
        for r in records:
            fwd_ms.append(r[0].elapsed_time(r[1]))
            if not decode:
                bwd_ms.append(r[1].elapsed_time(r[2]))
        if decode and graph is not None:
            fwd_ms[:] = [total_ms / args.steps]
    total_ms = max_over_ranks(total_ms, dev)
    value = rows_all * T * args.steps / (total_ms * 1e-3)     # all ranks' rows over the slowest rank's time

    # ---- batch rows that left the tensor-core path (gate products out of range -> scan kernels) ----
    flagged = None
    if not dfw and not decode and D == 64 and K == 64 and fsb and bsb:
        nc_ = (T + 63) // 64
        off = B * nc_ * 4096 + 2 * B * nc_ * 64 + B * nc_       # rowflag follows M, Ac, Gc, flags
        flagged = {"forward": int(fscr.view(torch.int32)[off:off + B].sum().item()),
                   "backward": int(bscr.view(torch.int32)[off:off + B].sum().item()), "of_rows": B}

    # ---- the same step through the autograd wrapper, tensors resident on the device -------------
    value_api = None
    if not decode:
        Fn, n_in = (DFWFunction, 4) if dfw else (LFWFunction, 6)
        n_api = max(3, min(args.steps, 10))

        def api_step(i):
            t = sets[i % n_sets]
            leaves = [u.detach().requires_grad_(True) for u in t[:n_in]]
            out, nxt = Fn.apply(*leaves)
            return torch.autograd.grad([out, nxt], leaves, [t[n_in], t[n_in + 1]])

        for i in range(3):
            api_step(i)
        barrier()
        a0, a1 = ev(), ev()
        a0.record()
        for i in range(n_api):
            api_step(i)
        a1.record()
        torch.cuda.synchronize()
        eager_ms = a0.elapsed_time(a1) / n_api
        graph_ms = None
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                api_step(0)
            torch.cuda.current_stream(dev).wait_stream(side)
            ga = torch.cuda.CUDAGraph()
            with torch.cuda.graph(ga):
                keep_api = [api_step(i) for i in range(n_api)]
            ga.replay()
            torch.cuda.synchronize()
            a0.record()
            ga.replay()
            a1.record()
            torch.cuda.synchronize()
            graph_ms = a0.elapsed_time(a1) / n_api
            del keep_api, ga
        except Exception as exc:
            sys.stderr.write("bench.py: API graph capture failed (%s)\n" % exc)
            torch.cuda.synchronize()
        best = graph_ms if graph_ms is not None else eager_ms
        value_api = {"value": B * T / (best * 1e-3) * (world if args.scaling == "weak" else 1), "unit": "tokens/s",
                     "eager_ms_per_step": eager_ms, "graph_ms_per_step": graph_ms, "steps": n_api,
                     "api": ("DFWFunction" if dfw else "LFWFunction") + ".apply + torch.autograd.grad, device-resident "
                            "tensors; `value` is this rank's figure times the number of ranks"}

    # ---- the decode step (BASELINE's second metric) in the same run -------------------------------
    extra = None
    if args.workload == "train":
        Bd, Dd, Kd, ring, trips = WORKLOADS["decode"][0], 64, 64, 10, 100
        gd = torch.Generator().manual_seed(args.seed + 7 + 1000 * rank)
        loop = LFWDecodeLoop((torch.randn(Bd, Dd, Kd, generator=gd) * 0.1).to(dtype).to(dev), ring=ring)
        loop.x.copy_(torch.randn(ring, Bd, 1, Dd, generator=gd).to(dtype))
        loop.query.copy_((torch.randn(ring, Bd, 1, Kd, generator=gd) / 8).to(dtype))
        loop.key.copy_((torch.randn(ring, Bd, 1, Kd, generator=gd) / 8).to(dtype))
        # gates in (0, 1): with the literal N(0,1) gate a chained 16-bit state overflows after a few
        # hundred steps (in the reference too); the step's cost does not depend on the values
        loop.f_key.copy_(torch.sigmoid(torch.randn(ring, Bd, 1, Kd, generator=gd)).to(dtype))
        if args.gates != "raw_f1":
            loop.f.copy_(torch.sigmoid(torch.randn(ring, Bd, 1, Dd, generator=gd)).to(dtype))
        loop.run_ring()                 # eager trip, then capture
        loop.run_ring()
        torch.cuda.synchronize()
        d0, d1 = ev(), ev()
        d0.record()
        for _ in range(trips):
            loop.run_ring()
        d1.record()
        torch.cuda.synchronize()
        us = d0.elapsed_time(d1) * 1e3 / (trips * ring)
        dbytes = 2 * (2 * Bd * Dd * Kd) + 2 * Bd * (2 * Dd + 3 * Kd) + 2 * Bd * Dd
        peak_d, kind_d = measured_hbm_peak()
        extra = {"decode": {
            "us_per_step": us, "steps": trips * ring, "tokens_per_s": Bd / (us * 1e-6),
            "achieved_gbs": dbytes / (us * 1e-6) / 1e9, "frac": dbytes / (us * 1e-6) / 1e9 / peak_d,
            "peak": peak_d, "peak_kind": kind_d + " copy bandwidth", "algorithmic_bytes_per_step": dbytes,
            "workload": "decode: B*H=%d, T=1, D=K=64, fp16 I/O, fp32 state arithmetic; %d chained steps, fresh "
                        "inputs from a ring of %d slots (f_key = sigmoid(N(0,1))); the state is chained through two 67 MB "
                        "buffers, so part of a step's output is still in the 126 MB L2 when the next step reads it "
                        "(--workload decode times the step with nothing in L2)"
                        % (Bd, trips * ring, ring),
            "api": "t2fw_b200.decode.LFWDecodeLoop (torch.ops.lfw.decode_step, one CUDA-graph replay per %d steps)" % ring,
            "finite": bool(torch.isfinite(loop.state).all().item())}}
        del loop

    # ---- strong scaling: the same rows split over the ranks (N > 1) -------------------------------
    strong = None
    if world > 1 and args.scaling == "weak" and not dfw and not decode:
        r0, r1 = row_shard(B, world, rank)
        sl = lambda t: t[r0:r1]

        def strong_step(i):
            j = i % n_sets
            x, f, q, k, fk, s0, go, gs = [sl(t) for t in sets[j]]
            cabi.lfw_forward(x, f, q, k, fk, s0, ckpt_every=C, out=sl(outs[j]), ckpt=sl(ckpts[j]), scratch=fscr)
            cabi.lfw_backward(go, gs, x, f, q, k, fk, s0, sl(ckpts[j]), ckpt_every=C,
                              grads=[sl(t) for t in grads[j]], scratch=bscr)

        for i in range(3):
            strong_step(i)
        barrier()
        gs_ = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gs_):
            for i in range(args.steps):
                strong_step(i)
        gs_.replay()
        barrier()
        s0e, s1e = ev(), ev()
        s0e.record()
        gs_.replay()
        s1e.record()
        barrier()
        sms = max_over_ranks(s0e.elapsed_time(s1e), dev)
        strong = {"value": B * T * args.steps / (sms * 1e-3), "unit": "tokens/s", "ms_per_step": sms / args.steps,
                  "rows_total": B, "rows_this_rank": r1 - r0, "steps": args.steps,
                  "note": "the workload's %d batch*head rows split contiguously over %d GPUs, no collective" % (B, world)}

    # ---- end to end through the public API with host buffers -------------------------------
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(3, min(args.steps, 40))
        host = [t.to(dtype) for t in make_inputs(torch, B, T, D, K, args.gates, args.seed + 1000 * rank, args.workload)]
        host = host[:6] if decode else host
        # the step's inputs lie back to back (256-byte aligned) in ONE pinned arena, as a loader that
        # stages a batch would leave them; srcs are the tensors of the step, views into it
        offs, total = [], 0
        for t in host:
            offs.append(total)
            total += (t.numel() * t.element_size() + 255) // 256 * 256
        arena = torch.empty(total, dtype=torch.uint8).pin_memory()
        def views(buf):
            return [buf[o:o + t.numel() * t.element_size()].view(t.dtype).view(t.shape) for o, t in zip(offs, host)]
        srcs = views(arena)
        for v, t in zip(srcs, host):
            v.copy_(t)
        h2d = sum(t.numel() * t.element_size() for t in srcs)
        d2h = 0
        # three streams: inputs in, compute, results out; n_slots sets of pinned result buffers, so
        # that a step's device->host copy overlaps the next steps' host->device copies and compute
        n_slots = max(2, args.e2e_slots)
        s_cmp = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        res_host, out_done, keep = [None] * n_slots, [None] * n_slots, [None] * n_slots

        def e2e_step(i):
            nonlocal d2h
            slot = i % n_slots
            # Tensors are shared between the three streams without record_stream: every tensor of a
            # step stays referenced in keep[slot] until the step n_slots before this one has finished
            # its device->host copies, so the allocator never reuses memory that is still in use.
            if out_done[slot] is not None:
                out_done[slot].synchronize()      # the host is done with this set's previous results
            keep[slot] = None
            with torch.cuda.stream(s_in):
                if args.e2e_separate_inputs:
                    devs = [t.to(dev, non_blocking=True) for t in srcs]
                else:
                    devs = views(arena.to(dev, non_blocking=True))
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            s_cmp.wait_event(ev_in)
            if dfw:
                leaves = [t.requires_grad_(True) for t in devs[:4]]
                out, nxt = DFWFunction.apply(*leaves)
                g = torch.autograd.grad([out, nxt], leaves, [devs[4], devs[5]])
                results = [out, nxt] + list(g)
            elif decode:
                with torch.no_grad():
                    out, nxt = LFWFunction.apply(*devs[:6])
                results = [out, nxt]
            else:
                leaves = [t.requires_grad_(True) for t in devs[:6]]
                out, nxt = LFWFunction.apply(*leaves)
                g = torch.autograd.grad([out, nxt], leaves, [devs[6], devs[7]])
                results = [out, nxt] + list(g)
            ev_c = torch.cuda.Event()
            ev_c.record(s_cmp)
            if res_host[slot] is None:
                res_host[slot] = [torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in results]
                d2h = sum(r.numel() * r.element_size() for r in results)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c)
                for h, r in zip(res_host[slot], results):
                    h.copy_(r, non_blocking=True)
                done = torch.cuda.Event()
                done.record(s_out)
            out_done[slot] = done
            keep[slot] = (devs, results)

        def e2e_drain():
            s_cmp.wait_stream(s_in)
            s_cmp.wait_stream(s_out)

        for i in range(2 * n_slots):
            e2e_step(i)
        e2e_drain()
        torch.cuda.synchronize()
        barrier()
        # The copies cross the host's PCIe and memory system, which other tenants of the machine
        # share: the region of e2e_steps steps is timed --e2e-blocks times and the MEDIAN block is
        # reported; every block's figure is listed beside it.
        blocks = []
        for _ in range(max(1, args.e2e_blocks)):
            barrier()
            t0 = time.perf_counter()
            e0, e1 = ev(), ev()
            e0.record()
            for i in range(e2e_steps):
                e2e_step(i)
            e2e_drain()
            e1.record()
            barrier()
            wall_b = time.perf_counter() - t0
            blocks.append((max_over_ranks(max(e0.elapsed_time(e1), 0.0), dev), wall_b))
        e2e_ms, wall = sorted(blocks)[len(blocks) // 2]
        e2e = {"value": rows_all * T * e2e_steps / (e2e_ms * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "ms_per_step": e2e_ms / e2e_steps,
               "api": ("DFWFunction" if dfw else "LFWFunction") + ".apply + autograd; pinned host buffers (inputs: %s); H2D, compute and D2H on "
                      "three streams with %d steps in flight (a step's D2H overlaps the next steps' H2D and compute)"
                      % ("one copy per tensor" if args.e2e_separate_inputs else "one copy of the arena that holds them", n_slots),
               "wall_ms_per_step": wall * 1e3 / e2e_steps,
               "blocks_ms_per_step": [b[0] / e2e_steps for b in blocks], "reported_block": "median",
               # the least disturbed block, for information: what the loop does when the host is quiet
               "fastest_block_value": rows_all * T * e2e_steps / (min(b[0] for b in blocks) * 1e-3)}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the slower call -------------------------------------------------------
    fb, bb = algorithmic_bytes_dfw(B, T, D, K) if dfw else algorithmic_bytes(B, T, D, K)
    peak, peak_kind = measured_hbm_peak()
    f_ms = statistics.mean(fwd_ms)
    b_ms = statistics.mean(bwd_ms) if bwd_ms else 0.0
    if b_ms >= f_ms and not decode:
        which, alg, dur = "backward call (all kernels of t2fw_%s_backward)" % ("dfw" if dfw else "lfw"), bb, b_ms
    else:
        which, alg, dur = "forward call (all kernels of t2fw_%s_forward)" % ("dfw" if dfw else "lfw"), fb, f_ms
    achieved = alg / (dur * 1e-3) / 1e9
    # DRAM bytes (read + write) per call, summed over the kernels of the call, from the ncu capture
    # recorded beside the kernel versions it was taken on; None where no capture exists
    traffic, traffic_src = None, None
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as fh:
            tj = json.load(fh)
        traffic = tj.get(args.workload, {}).get(which.split()[0])
        traffic_src = {"captured_on_commit": tj.get("captured_on_commit"), "command": tj.get("command")}
    except Exception:
        pass
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_src,
        "peak_kind": peak_kind + " copy bandwidth",
        "kernel": which, "algorithmic_bytes_per_launch": alg, "avg_ms": dur,
        "fwd_ms": f_ms, "bwd_ms": b_ms, "split_timing": split_kind,
        "whole_step_frac": ((fb + (0 if decode else bb)) / ((f_ms + b_ms) * 1e-3) / 1e9) / peak,
    }

    cpu = None
    if not args.no_cpu_baseline:
        _, cpu = cpu_reference_run(args.workload, args.gates, 3, 2, args.seed)

    line = {
        "metric": metric_name(args.workload), "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32 state arithmetic, f16 I/O", "data": "synthetic",
        "config": dict(workload_config(args, B, T, D, K), host_binding=host_binding,
                       l2="inputs larger than L2: %d rotating input/output sets" % n_sets,
                       ckpt_every=C, cuda_graph=graph is not None, flagged_rows=flagged),
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
        "roofline": roofline, "cpu_baseline": cpu, "value_api": value_api,
    }
    if extra is not None:
        line["extra"] = extra
    if strong is not None:
        line["strong"] = strong
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "gpt2":
        run_gpt2(args)
    elif args.workload == "seqsplit":
        run_seqsplit(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
