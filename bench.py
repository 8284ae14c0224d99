"""Benchmark of the DA-Transformer custom-op hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scaling weak|strong]
    (N > 1: python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...)

Workload (configuration C4): sentences with graph length L=512 (= output_length), target_length
~ U{32..64} padded to T=64, fp32 links and fp32 match (match has the distribution log-softmax over
V=42000 bf16 N(0,2) logits gives at the target tokens).  One step = dag_best_alignment + dag_loss
forward (alpha+beta) + dag_loss backward over the rank's sentences + the criterion's statistics,
then the SUM all-reduce of those statistics.  No tensor crosses GPUs.

Headline (`value`): weak scaling, every GPU holds 512 sentences (600 MB of inputs per GPU, larger
than L2, so no flush is needed between steps).  The line also carries a `strong` block: the same
step on 512 / N sentences per GPU, i.e. ONE 512-sentence batch split over the N GPUs; `--scaling
strong` makes that the headline instead.

The timed region of K steps is repeated `--repeats` times (barrier + synchronize around each);
`ms_per_step` is the median region divided by K, min and max are reported beside it.

`e2e` is the same step through the public Python API with inputs copied from pinned host memory
and the statistics copied back every step.  `roofline` describes the dominant kernel (the
alpha/beta sweep of the loss forward) from the median of direct launches on preallocated buffers:
algorithmic special-function evaluations per launch (one exp per (t, i->j) term of the log-domain
recursion, the reference's formulation) against the special-function throughput measured on this
device just before; `roofline_shipped` is the work the shipped probability-domain kernel executes
(FFMA and tf32 tensor-core products) against the measured FP32 and nominal TF32 peaks.
`gather` reports logsoftmax_gather forward+backward on all six C2 cases against the measured HBM
copy bandwidth.  `configs` holds the step times of C1 and C3.  `cpu_baseline` is the CPU oracle (a
C port of the reference's arithmetic) and `cpu_baseline_torch` the torch-native twin, both timed on
this host's cores on a bounded sample.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "dag_loss_fwd_bwd_sentences_per_s"
UNIT = "sentences/s"
GLOBAL_SENTENCES = 512
L_GRAPH, T_MAX, VOCAB = 512, 64, 42000


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "sm_max_mhz": 1965.0}, "fallback"


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def exp_counts(ol, tl, K):
    """Algorithmic exp evaluations per sentence of the log-domain formulation:
    P = sum_{j=1}^{ol-1} min(j, K) predecessor terms per target step;
    sweeps (alpha + beta) = 2 (tl-1) P;  whole forward+backward = 3 (tl-1) P + tl*ol."""
    import torch

    j = torch.arange(1, int(ol.max().item()), dtype=torch.float64)
    cum = torch.cat([torch.zeros(1, dtype=torch.float64), torch.cumsum(torch.clamp(j, max=K), 0)])
    P = cum[(ol - 1).clamp(min=0).long()]
    tlf = tl.to(torch.float64)
    sweeps = 2.0 * (tlf - 1) * P
    total = 3.0 * (tlf - 1) * P + tlf * ol.to(torch.float64)
    return float(sweeps.sum()), float(total.sum())


def shipped_work(ol, tl):
    """What dag_strip_sweep_kernel executes per launch (both directions): vertices are taken in groups
    of 128 (four 32-vertex sub-strips); the 10 blocks of 32 x 32 inside a group run as FFMAs once per
    target step, every block outside runs on the tensor cores as three tf32 products (3xTF32)."""
    ffma = mma = 0.0
    for o, t in zip(ol.tolist(), tl.tolist()):
        nsub = (o + 31) // 32
        groups = (nsub + 3) // 4
        in_group_blocks = 0
        for g in range(groups):
            gs = min(4, nsub - 4 * g)
            in_group_blocks += gs * (gs + 1) // 2
        all_blocks = nsub * (nsub + 1) // 2
        ffma += 2.0 * (t - 1) * in_group_blocks * 1024
        mma += 2.0 * (t - 1) * (all_blocks - in_group_blocks) * 1024 * 3
    return ffma, mma


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi (query only).  Started well before the
    timed regions (its start-up talks to the driver for tens of milliseconds and would stall kernel
    launches if it overlapped them); the samples whose timestamps fall inside the regions are the ones
    reported."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id):
        self.gpu = gpu_id
        self.proc = None
        self.lines = []
        self.t_begin = self.t_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            deadline = time.time() + 3.0
            while not self.lines and time.time() < deadline:   # start-up is over once it prints
                time.sleep(0.01)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def begin(self):
        self.t_begin = time.time()

    def end(self):
        self.t_end = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime

        rows = []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[1]), float(parts[2]), float(parts[3]),
                             [n for n, v in zip(names, parts[5:9]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if self.t_begin is not None and self.t_begin - 0.02 <= r[0] <= self.t_end + 0.02]
        where = "timed regions"
        if not inside:   # clock skew between nvidia-smi's timestamps and this process: use all samples
            inside, where = rows, "whole run (no sample carried a timestamp inside the regions)"
        sm = [r[1] for r in inside]
        reasons = sorted({x for r in inside for x in r[4]})
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": max(r[2] for r in inside) if inside else None,
                "power_w_max": max(r[3] for r in inside) if inside else None,
                "samples": len(sm), "window": where, "reasons": reasons}


# --------------------------------------------------------------------------------------
# CPU arm: the oracle (a C port of the reference's arithmetic) and the torch-native twin
# --------------------------------------------------------------------------------------
def cpu_step(batch_np):
    from oracle import oracle
    import numpy as np

    match, links, ol, tl = batch_np
    oracle.dag_best_alignment(match, links, ol, tl, dtype=np.float32)
    loss, alpha, beta = oracle.dag_loss(match, links, ol, tl, dtype=np.float32)
    oracle.dag_loss_backward(np.ones_like(loss), alpha, beta, match, links, ol, tl, dtype=np.float32)
    return loss


def cpu_sample(n):
    from da_transformer_b200 import workloads

    b = workloads.config4(B=n)
    return (b.match_all.numpy(), b.links.numpy(), b.output_length.numpy(), b.target_length.numpy())


def cpu_threads_setup():
    """All host threads for the oracle's OpenMP loops, whatever OMP_NUM_THREADS the launcher exported
    (torchrun sets it to 1 for N > 1).  Returns the number of threads the loops will really use."""
    from oracle import oracle

    return oracle.set_threads(host_threads())


def cpu_baseline(budget_s=12.0):
    cores = cpu_threads_setup()
    sample = cpu_sample(cores)
    t0 = time.perf_counter()
    cpu_step(sample)                       # also warms the thread pool
    one = time.perf_counter() - t0
    reps = max(1, min(8, int(budget_s / max(one, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        cpu_step(sample)
    dt = (time.perf_counter() - t0) / reps
    return {"value": cores / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{cores} C4 sentences (L=512, T=64) per pass, {reps} passes, fp32 oracle "
                      f"(oracle/dag_oracle.c, OpenMP over sentences, omp_get_max_threads() = {cores}): "
                      f"best alignment + alpha + beta + backward"}


def cpu_baseline_torch(n=8, budget_s=10.0):
    """The torch-native twin (this package's torch_dag_loss / torch_dag_best_alignment, which follow
    the reference's torch path, fs_plugins/custom_ops/dag_loss.py:259-353, and are checked against
    fixtures made by it) on the same kind of sample, all host threads."""
    import torch

    from da_transformer_b200 import torch_twins, workloads

    cores = host_threads()
    torch.set_num_threads(cores)
    b = workloads.config4(B=n)
    sq = workloads.band_to_square(b.links)

    def step():
        m = b.match_all.clone().requires_grad_()
        l = sq.clone().requires_grad_()
        torch_twins.torch_dag_best_alignment(m.detach(), l.detach(), b.output_length, b.target_length)
        loss = torch_twins.torch_dag_loss(m, l, b.output_length, b.target_length)
        torch.autograd.grad(loss.sum(), [m, l])

    t0 = time.perf_counter()
    step()
    one = time.perf_counter() - t0
    reps = max(1, min(5, int(budget_s / max(one, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        step()
    dt = (time.perf_counter() - t0) / reps
    return {"value": n / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n} C4 sentences per pass, {reps} passes, fp32 torch-native twin "
                      f"(da_transformer_b200/torch_twins.py): best alignment + loss + autograd backward"}


def reference_cuda_baseline(match, links, ol, tl, gout, iters=5):
    """GPU baseline leg: the same step on the REFERENCE's own CUDA kernels (compiled unmodified
    by oracle/build_ref.py, default launch configs), when that build is present.  A baseline
    printed next to our numbers, never part of the measured path."""
    import torch

    from oracle import ref_cuda

    if not ref_cuda.available():
        return {"unavailable": "oracle/_ref/dag_loss_fn.so not built"}
    B = match.shape[0]
    m, l = match.detach(), links.detach()
    g = gout.contiguous()

    def step():
        ref_cuda.dag_best_alignment(m, l, ol, tl)
        ref_cuda.dag_loss_fwd_bwd(m, l, ol, tl, g)

    def timed(fn, n):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    ms = timed(step, iters)
    ms_align = timed(lambda: ref_cuda.dag_best_alignment(m, l, ol, tl), iters)
    return {"value": B / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "best_alignment_ms": ms_align,
            "dag_loss_fwd_bwd_ms": ms - ms_align,
            "what": "reference CUDA extension (dag_loss.cu, dag_best_alignment.cu) built for sm_100, "
                    "default configs, same 512-sentence shard, same step"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = cpu_threads_setup()
    n = cores
    sample = cpu_sample(n)
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_step(sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(sample)
    dt = time.perf_counter() - t0
    value = n * args.steps / dt
    desc = (f"{n} C4 sentences per step on {cores} host threads (omp_get_max_threads(), set explicitly), fp32 CPU "
            f"oracle port of the reference arithmetic (the reference's own CPU path is PyTorch code that cannot "
            f"travel to this box)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "C4 sample: L=512, T=64, tl~U{32..64}, dag_best_alignment + dag_loss fwd+bwd",
                   "sentences_per_step": n},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=10, help="how many times the K-step timed region is repeated")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: 512 sentences per GPU; strong: one 512-sentence batch split over the GPUs")
    ap.add_argument("--sentences", type=int, default=None, help="sentences per GPU (overrides --scaling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gather", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the C1 / C3 / peaky-workload legs")
    ap.add_argument("--eager", action="store_true", help="launch the step kernel by kernel instead of replaying a CUDA graph")
    ap.add_argument("--gather-only", action="store_true",
                    help="only the logsoftmax_gather leg (bf16, V=32000) on --gather-batch sentences: the small case "
                         "the profiler captures")
    ap.add_argument("--gather-batch", type=int, default=32)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from da_transformer_b200 import (DagLossFunc, _native, dag_best_alignment, dag_logsoftmax_gather_inplace,
                                     dag_loss, workloads)
    from da_transformer_b200 import dist as ddist
    from da_transformer_b200.build import PROBE_LIB

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _native.lib()
    probe = ctypes.CDLL(PROBE_LIB)     # measurement probes: their own library, not the operator path
    for fn in (probe.dat_probe_mufu, probe.dat_probe_ffma):
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    peaks, peak_kind = measured_peaks()
    ptr, sptr = _native.ptr, _native.stream_ptr

    if args.gather_only:
        Bg, Lg, Vg, Sg = args.gather_batch, 1024, 32000, 128
        g2 = torch.Generator(device=dev)
        g2.manual_seed(workloads.BASE_SEED + 2)
        base = (torch.randn(Bg, Lg, Vg, device=dev, generator=g2) * 2.0).to(torch.bfloat16)
        idx = torch.randint(0, Vg, (Bg, Lg, Sg), device=dev, generator=g2)
        gsel = torch.randn(Bg, Lg, Sg, device=dev, generator=g2)
        times = []
        for it in range(args.warmup + args.steps):
            x = base.clone().requires_grad_()
            work = x.clone()
            a, b_, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            a.record()
            _, sel = dag_logsoftmax_gather_inplace(work, idx)
            b_.record()
            sel.backward(gsel)
            c.record()
            torch.cuda.synchronize()
            if it >= args.warmup:
                times.append((a.elapsed_time(b_), b_.elapsed_time(c)))
        print(json.dumps({"gather_only": {"shape": [Bg, Lg, Vg], "dtype": "bfloat16",
                                          "fwd_ms": statistics.median(t[0] for t in times),
                                          "bwd_ms": statistics.median(t[1] for t in times)}}))
        return

    # ---- data: every rank owns one shard of 512 sentences
    # (shard r is drawn from its own generator, seed 20225 + 1000 r, so it is the same data whatever
    # the number of GPUs and no rank has to generate the other shards).  Weak scaling uses the whole
    # shard; the strong split uses its first 512 / N sentences.
    B_strong = max(1, GLOBAL_SENTENCES // world)
    B_weak = GLOBAL_SENTENCES
    if args.sentences is not None:
        B_head = args.sentences
    else:
        B_head = B_strong if args.scaling == "strong" else B_weak
    B_gen = args.sentences if args.sentences is not None else B_weak
    gen = workloads.generator(4 + 1000 * rank)
    shard = workloads.config4(gen=gen, B=B_gen, L=L_GRAPH, V=VOCAB)
    host_all = [shard.match_all, shard.links, shard.output_length, shard.target_length]
    dev_all = [t.to(dev) for t in host_all]
    K = dev_all[1].shape[2]

    ev = lambda: torch.cuda.Event(enable_timing=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world > 1:
            t = torch.tensor([x], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return x

    class Step:
        """The benchmark step on the first B sentences of the shard: captured once as a CUDA graph
        (the alignment, independent of the loss, is a parallel branch) and replayed, followed by the
        NCCL all-reduce of the statistics."""

        def __init__(self, B, eager=False):
            self.B = B
            self.match = dev_all[0][:B].clone().requires_grad_()
            self.links = dev_all[1][:B].clone().requires_grad_()
            self.ol, self.tl = dev_all[2][:B].clone(), dev_all[3][:B].clone()
            self.gout = (-1.0 / (self.tl.double() * (B * world))).float()   # d(-(loss/tl).mean())/d loss
            self.align_stream = torch.cuda.Stream(device=dev)
            self.reducer = ddist.OverlappedStatsReducer(dev)
            self.graph, self.out, self.mode = None, None, "eager"
            if not (args.eager or eager):
                try:
                    side = torch.cuda.Stream(device=dev)
                    side.wait_stream(torch.cuda.current_stream(dev))
                    with torch.cuda.stream(side):
                        for _ in range(3):
                            self.local()
                    torch.cuda.current_stream(dev).wait_stream(side)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        self.out = self.local(fork=True)
                    self.graph, self.mode = g, "cuda_graph"
                except Exception as exc:   # capture not possible here: kernel-by-kernel launches
                    print(f"[bench] CUDA graph capture failed, running eagerly: {exc}", file=sys.stderr)
                    self.graph, self.out = None, None
                    torch.cuda.synchronize()

        def local(self, fork=False):
            cur = torch.cuda.current_stream(dev)
            if fork:
                self.align_stream.wait_stream(cur)
                with torch.cuda.stream(self.align_stream):
                    path = dag_best_alignment(self.match.detach(), self.links.detach(), self.ol, self.tl)
            else:
                path = dag_best_alignment(self.match.detach(), self.links.detach(), self.ol, self.tl)
            loss = dag_loss(self.match, self.links, self.ol, self.tl)
            gm, gl = torch.autograd.grad(loss, [self.match, self.links], grad_outputs=self.gout)
            stats = ddist.sentence_stats(loss.detach(), self.tl)
            if fork:
                cur.wait_stream(self.align_stream)
            return stats, path, gm, gl

        def run(self):
            if self.graph is None:
                out = self.local()
            else:
                self.graph.replay()
                out = self.out
            # the 32-byte all-reduce runs on a side stream behind this step only; the next step does not wait for it
            return self.reducer.submit(out[0])

        def regions(self, steps, repeats, warmup):
            """`repeats` timed regions of `steps` steps; each bracketed by barrier + synchronize, timed
            with CUDA events on the launching stream, max over ranks."""
            for _ in range(warmup):
                self.run()
            out = []
            stats = None
            for _ in range(repeats):
                barrier()
                t0, t1 = ev(), ev()
                t0.record()
                for _ in range(steps):
                    stats = self.run()
                self.reducer.wait()          # every all-reduce of the region ends inside it
                t1.record()
                barrier()
                out.append(max_over_ranks(t0.elapsed_time(t1)))
            return out, stats

    def summarise(regions_ms, steps, B):
        med = statistics.median(regions_ms)
        return {"ms_per_step": med / steps, "ms_per_step_min": min(regions_ms) / steps,
                "ms_per_step_max": max(regions_ms) / steps, "regions": len(regions_ms),
                "value": B * world / (med / steps * 1e-3), "sentences_per_gpu": B,
                "global_sentences": B * world}

    # ---- special-function and fp32-FMA roofline denominators, measured now
    sink = torch.zeros(1, device=dev)
    sm_count = torch.cuda.get_device_properties(dev).multi_processor_count

    def probe_rate(fn, per_thread):
        blocks, iters = sm_count * 2, 4096
        for _ in range(2):
            fn(iters, blocks, ptr(sink), sptr(dev))
        e0, e1 = ev(), ev()
        e0.record()
        rc = fn(iters, blocks, ptr(sink), sptr(dev))
        e1.record()
        torch.cuda.synchronize()
        if rc != 0:
            raise RuntimeError("measurement probe failed to launch")
        return blocks * 1024 * per_thread * iters / (e0.elapsed_time(e1) * 1e-3)

    mufu_peak = probe_rate(probe.dat_probe_mufu, 8)     # ex2 / s
    ffma_peak = probe_rate(probe.dat_probe_ffma, 16)    # fp32 FMA / s

    # ---- timed regions: device-resident inputs
    uuid = str(torch.cuda.get_device_properties(dev).uuid)
    sampler = ClockSampler(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
    if rank == 0:
        sampler.start()
    head = Step(B_head)
    other_B = B_strong if B_head != B_strong else B_weak
    other = Step(other_B) if (args.sentences is None and other_B != B_head) else None
    head.regions(1, 1, args.warmup)          # warm-up outside the sampled window
    barrier()
    sampler.begin()
    head_regions, stats = head.regions(args.steps, args.repeats, 0)
    sampler.end()
    clocks = sampler.stop() if rank == 0 else None
    head_sum = summarise(head_regions, args.steps, B_head)
    final_stats = stats.cpu().tolist()
    other_sum = None
    if other is not None:
        other_regions, _ = other.regions(args.steps, args.repeats, args.warmup)
        other_sum = summarise(other_regions, args.steps, other_B)
    # the same step launched kernel by kernel through the Python front end (what a criterion that does not
    # capture graphs gets): host time of the ctypes calls and allocations included
    eager_sum = None
    if not args.eager and args.sentences is None:
        eg = Step(B_head, eager=True)
        eg_regions, _ = eg.regions(args.steps, 3, args.warmup)
        eager_sum = summarise(eg_regions, args.steps, B_head)
        del eg
    weak_sum = head_sum if B_head == B_weak else other_sum
    strong_sum = head_sum if B_head == B_strong else other_sum
    if world == 1 and args.sentences is None:
        weak_sum = strong_sum = head_sum

    match, links, ol, tl, gout = head.match, head.links, head.ol, head.tl, head.gout
    B = B_head
    sweep_exps, total_exps = exp_counts(shard.output_length[:B], shard.target_length[:B], K)
    ffma_exec, mma_exec = shipped_work(shard.output_length[:B], shard.target_length[:B])

    # ---- the dominant kernel alone: dat_dag_loss_fast launched directly on preallocated buffers,
    # median of 30 CUDA-event times (nothing is allocated inside the bracket)
    def time_median(fn, n=30, warm=3):
        for _ in range(warm):
            fn()
        marks = [(ev(), ev()) for _ in range(n)]
        torch.cuda.synchronize()
        for a, b in marks:
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        ts = [a.elapsed_time(b) for a, b in marks]
        return statistics.median(ts), min(ts), max(ts)

    md, ld = match.detach(), links.detach()
    alpha = torch.empty(B, T_MAX, L_GRAPH, device=dev)
    beta = torch.empty_like(alpha)
    offsets = torch.empty(B, 2 * T_MAX + 2, dtype=torch.float64, device=dev)
    res = torch.empty(B, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    scratch = torch.empty(lib.dat_dag_loss_fast_scratch_bytes(B, T_MAX, L_GRAPH), dtype=torch.uint8, device=dev)
    flagged = torch.zeros(2, dtype=torch.int32, device=dev)

    def fwd_direct():
        _native.check(lib.dat_dag_loss_fast(ptr(md), ptr(ld), ptr(ol), ptr(tl), ptr(alpha), ptr(beta), ptr(offsets),
                                            ptr(res), ptr(status), ptr(scratch), B, T_MAX, L_GRAPH, K, sptr(dev)),
                      "dag_loss_fast")

    sweep_ms, sweep_ms_min, sweep_ms_max = time_median(fwd_direct)
    _native.check(lib.dat_dag_loss_fast_flagged(ptr(scratch), ptr(flagged), B, T_MAX, L_GRAPH, sptr(dev)), "flagged")
    n_flagged, n_exact_bwd = (int(v) for v in flagged.tolist())

    # ---- per-op breakdown (medians, outside the headline regions)
    breakdown = {}
    if rank == 0:
        breakdown["best_alignment_ms"] = time_median(lambda: dag_best_alignment(md, ld, ol, tl), 15)[0]
        breakdown["loss_fwd_alpha_beta_ms"] = time_median(lambda: dag_loss(match, links, ol, tl), 15)[0]
        breakdown["loss_fwd_no_grad_ms"] = time_median(lambda: dag_loss(md, ld, ol, tl), 15)[0]
        loss_keep = dag_loss(match, links, ol, tl)
        breakdown["loss_bwd_ms"] = time_median(
            lambda: torch.autograd.grad(loss_keep, [match, links], grad_outputs=gout, retain_graph=True), 15)[0]
        fb = breakdown["loss_fwd_alpha_beta_ms"] + breakdown["loss_bwd_ms"]
        breakdown["dag_loss_fwd_bwd_only_sentences_per_s"] = B / (fb * 1e-3)
        breakdown["flagged_sentences"] = n_flagged
        breakdown["exact_backward_only_sentences"] = n_exact_bwd
        del loss_keep

    # ---- end to end through the public API: host inputs in, statistics out, every step
    from da_transformer_b200 import host_io

    host = [t[:B].contiguous().pin_memory() for t in host_all]
    max_ol = int(host[2].max().item())
    h2d_full = sum(t.numel() * t.element_size() for t in host)
    # the links go over PCIe without their padding (host_io.upload_links): row i of the band has only
    # output_length - 1 - i real entries, nothing reads the rest
    links_bytes = host_io.upload_links_bytes(B, L_GRAPH, K, max_ol, pinned=True)
    h2d = h2d_full - host[1].numel() * 4 + links_bytes
    d2h = 4 * 8
    stats_host = torch.empty(4, dtype=torch.float64).pin_memory()

    # The copies of step i+1 run on a second stream while step i computes (two device buffer sets),
    # the way an input pipeline feeds a training step; every step still pays its own full
    # host-to-device copy and its own device-to-host read of the statistics.
    # (two copy streams: the copy engine moves match and the lengths while the pull kernel of upload_links reads
    # the ragged link rows; the two kinds of PCIe reads together come closer to the link's rate than either alone)
    copy_stream = torch.cuda.Stream(device=dev)
    links_stream = torch.cuda.Stream(device=dev)
    bufs = [[torch.empty_like(h, device=dev) for h in host] for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    links_ready = [torch.cuda.Event() for _ in range(2)]
    freed = [torch.cuda.Event() for _ in range(2)]

    full_copy = [False]

    def e2e_upload(slot):
        with torch.cuda.stream(links_stream):
            links_stream.wait_event(freed[slot])         # the step that used this slot is done
            if full_copy[0]:
                bufs[slot][1].copy_(host[1], non_blocking=True)
            else:
                host_io.upload_links(host[1], bufs[slot][1], max_ol)
            links_ready[slot].record(links_stream)
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(freed[slot])
            for k, (d, h) in enumerate(zip(bufs[slot], host)):
                if k != 1:
                    d.copy_(h, non_blocking=True)
            copy_stream.wait_event(links_ready[slot])
            ready[slot].record(copy_stream)

    def e2e_compute(slot):
        cur = torch.cuda.current_stream()
        cur.wait_event(ready[slot])
        m = bufs[slot][0].requires_grad_()
        l = bufs[slot][1].requires_grad_()
        o, t = bufs[slot][2], bufs[slot][3]
        dag_best_alignment(m.detach(), l.detach(), o, t)
        loss = dag_loss(m, l, o, t)
        torch.autograd.grad(loss, [m, l], grad_outputs=gout)
        s = ddist.all_reduce_stats(ddist.sentence_stats(loss.detach(), t))
        stats_host.copy_(s, non_blocking=True)
        freed[slot].record(cur)
        m.requires_grad_(False)
        l.requires_grad_(False)

    def e2e_run(n):
        for f in freed:
            f.record(torch.cuda.current_stream())
        e2e_upload(0)
        for i in range(n):
            if i + 1 < n:
                e2e_upload((i + 1) & 1)
            e2e_compute(i & 1)
        torch.cuda.current_stream().synchronize()      # the last statistics have reached the host

    def e2e_measure():
        e2e_run(3)
        regions = []
        for _ in range(min(args.repeats, 5)):
            barrier()
            t0, t1 = ev(), ev()
            t0.record()
            e2e_run(args.steps)
            t1.record()
            barrier()
            regions.append(max_over_ranks(t0.elapsed_time(t1)))
        return regions

    e2e_regions = e2e_measure()
    e2e_ms = statistics.median(e2e_regions)
    e2e_value = B * world / (e2e_ms / args.steps * 1e-3)
    full_copy[0] = True                      # for comparison: every byte of the band copied
    e2e_full_ms = statistics.median(e2e_measure())
    e2e_full_value = B * world / (e2e_full_ms / args.steps * 1e-3)
    del bufs, host

    # ---- logsoftmax_gather on the C2 shapes (rank 0), HBM roofline
    gather = None
    if rank == 0 and not args.no_gather:
        Bg, Lg, Sg = 32, 1024, 128
        cases = []
        for dt in (torch.bfloat16, torch.float16):
            for Vg in (32000, 50000, 64000):
                g2 = torch.Generator(device=dev)
                g2.manual_seed(workloads.BASE_SEED + 2)
                base = torch.empty(Bg, Lg, Vg, dtype=dt, device=dev)
                for b in range(Bg):
                    base[b] = (torch.randn(Lg, Vg, device=dev, generator=g2) * 2.0).to(dt)
                idx = torch.randint(0, Vg, (Bg, Lg, Sg), device=dev, generator=g2)
                gsel = torch.randn(Bg, Lg, Sg, device=dev, generator=g2)
                fwd_ms, bwd_ms = [], []
                for it in range(8):
                    x = base.clone().requires_grad_()
                    work = x.clone()
                    a, b_, c = ev(), ev(), ev()
                    a.record()
                    _, sel = dag_logsoftmax_gather_inplace(work, idx)
                    b_.record()
                    sel.backward(gsel)
                    c.record()
                    torch.cuda.synchronize()
                    if it >= 3:
                        fwd_ms.append(a.elapsed_time(b_))
                        bwd_ms.append(b_.elapsed_time(c))
                    del x, work, sel
                e = 2
                fwd_bytes = Bg * Lg * Vg * e + 4 * Bg * Lg * Sg + 8 * Bg * Lg * Sg
                bwd_bytes = 2 * Bg * Lg * Vg * e + 4 * Bg * Lg * Sg + 8 * Bg * Lg * Sg
                f, bw = statistics.median(fwd_ms), statistics.median(bwd_ms)
                cases.append({
                    "dtype": str(dt).replace("torch.", ""), "vocab": Vg,
                    "fwd_ms": f, "bwd_ms": bw, "fwd_gbs": fwd_bytes / f / 1e6, "bwd_gbs": bwd_bytes / bw / 1e6,
                    "fwd_bwd_gbs": (fwd_bytes + bwd_bytes) / (f + bw) / 1e6,
                    "frac": (fwd_bytes + bwd_bytes) / (f + bw) / 1e6 / peaks["hbm_gbs"],
                    "frac_of_nominal_8000": (fwd_bytes + bwd_bytes) / (f + bw) / 1e6 / 8000.0,
                    "algorithmic_bytes": fwd_bytes + bwd_bytes,
                })
                del base, idx, gsel
                torch.cuda.empty_cache()
        gather = {"workload": f"C2: logits [{Bg},{Lg},V] N(0,2), select_idx [{Bg},{Lg},{Sg}] int64, fwd+bwd",
                  "peak_gbs": peaks["hbm_gbs"], "peak_kind": peak_kind, "cases": cases}

    # ---- the other configurations' step times and the peaky (trained-like) workload, rank 0
    configs = {}
    if rank == 0 and not args.no_extra:
        configs = extra_legs(torch, dev, ev, workloads, dag_loss, dag_best_alignment, dag_logsoftmax_gather_inplace,
                             DagLossFunc, lib, _native, time_median)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    sweep_rate = sweep_exps / (sweep_ms * 1e-3)
    scaling = "strong" if (args.sentences is None and args.scaling == "strong") else "weak"
    out = {
        "metric": METRIC, "value": head_sum["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head_sum["ms_per_step"],
        "ms_per_step_min": head_sum["ms_per_step_min"], "ms_per_step_max": head_sum["ms_per_step_max"],
        "timed_regions": head_sum["regions"],
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {
            "workload": ("C4: per GPU %d sentences, L=512 (=output_length), target_length~U{32..64}, T=64, "
                         "fp32 links [B,512,511] + fp32 match [B,64,512]; step = dag_best_alignment + dag_loss "
                         "fwd (alpha+beta) + bwd + statistics + scalar all-reduce") % B,
            "sentences_per_gpu": B, "global_sentences": B * world, "parallelism": f"dp{world}",
            "l2": ("inputs (%.0f MB per GPU) exceed L2; no flush between steps" % (h2d_full / 1e6))
                  if h2d_full > 126e6 * 1.5
                  else ("inputs are %.0f MB per GPU, less than L2 holds: the links stay L2-resident between steps, "
                        "as they would after the model's forward pass wrote them" % (h2d_full / 1e6)),
            "launch": head.mode,
            "timing": f"{args.repeats} regions of {args.steps} steps, median region / steps",
        },
        "weak": weak_sum, "strong": strong_sum, "eager": eager_sum,
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "regions": len(e2e_regions),
                "how": "links uploaded without most of their padding (host_io.upload_links: nearly full rows by the copy engine, ragged rows pulled by a kernel, at the same time), match and lengths whole on a second copy stream",
                "with_whole_band_copied": {"value": e2e_full_value, "h2d_bytes_per_step": h2d_full}},
        # per step: alignment (2 with more sentences than SMs: order, persistent strip kernel; else 1), loss forward
        # (3: order, strip sweep with its check, exact fallback), loss backward (3: grad_match + preparation,
        # product-form grad_links, exact fallback), statistics (1)
        "gpu_launches": (8 + (1 if B > torch.cuda.get_device_properties(dev).multi_processor_count else 0))
                        * args.steps * args.repeats,
        "roofline": {
            "kernel": ("dag_loss forward = dag_strip_sweep_kernel (alpha and beta recursions, one CTA each; finished "
                       "vertex groups through tcgen05 3xTF32 products, blocks inside a group as FFMAs on "
                       "exp(links) held in registers) with its order, check and fallback launches"),
            "bound": "mufu", "achieved": sweep_rate / 1e9, "peak": mufu_peak / 1e9, "unit": "Gexp/s",
            "frac": sweep_rate / mufu_peak,
            # dram__bytes_read+write of dag_strip_sweep_kernel from the ncu capture summarised in
            # profiles/dag_strip_sweep_c4_148sent.md (110.4 MB for 148 sentences), scaled by sentences
            "traffic": 110.4e6 / 148 * B,
            "peak_kind": "measured on this device by the ex2 probe just before the timed regions",
            "nominal_peak": 16 * sm_count * peaks.get("sm_max_mhz", 1965.0) * 1e6 / 1e9,
            "algorithmic_exps_per_launch": sweep_exps, "kernel_ms": sweep_ms,
            "kernel_ms_min": sweep_ms_min, "kernel_ms_max": sweep_ms_max,
            "kernel_ms_how": "median of 30 direct dat_dag_loss_fast launches on preallocated buffers",
            "step_frac_all_kernels": (total_exps / (head_sum["ms_per_step"] * 1e-3)) / mufu_peak,
        },
        "roofline_shipped": {
            "what": ("work dag_strip_sweep_kernel executes per launch: 32x32 blocks inside a 128-vertex group as "
                     "fp32 FMAs, all other blocks as 3xTF32 tensor-core products (tcgen05.mma kind::tf32, M=128, accumulator in tensor memory)"),
            "ffma_executed": ffma_exec, "ffma_rate_tfma_s": ffma_exec / (sweep_ms * 1e-3) / 1e12,
            "ffma_peak_tfma_s": ffma_peak / 1e12, "ffma_frac": ffma_exec / (sweep_ms * 1e-3) / ffma_peak,
            "tf32_fma_executed": mma_exec, "tf32_rate_tfma_s": mma_exec / (sweep_ms * 1e-3) / 1e12,
            "tf32_nominal_peak_tfma_s": 550.0, "tf32_frac_of_nominal": mma_exec / (sweep_ms * 1e-3) / 550e12,
            "all_terms_as_fma_frac": (sweep_exps / (sweep_ms * 1e-3)) / ffma_peak,
            "ffma_peak_kind": "measured on this device by the FMA probe",
        },
        "breakdown": breakdown,
        "gather": gather,
        "configs": configs,
        "loss_check": {"mean_nll_per_token": -final_stats[0] / final_stats[2], "invalid": final_stats[3],
                       "flagged_sentences": n_flagged},
    }
    if gather is not None:
        c0 = gather["cases"][0]
        out["roofline_gather"] = {"bound": "hbm", "achieved": c0["fwd_bwd_gbs"], "peak": peaks["hbm_gbs"],
                                  "unit": "GB/s", "frac": c0["frac"],
                                  "case": f"{c0['dtype']} V={c0['vocab']}",
                                  # dram__bytes_read+write of lsg_fwd_kernel + lsg_bwd_kernel from the ncu
                                  # capture summarised in profiles/lsg_c2_bf16_v32000.md
                                  "traffic": GATHER_TRAFFIC_BYTES,
                                  "algorithmic_bytes": c0["algorithmic_bytes"], "peak_kind": peak_kind}
    if world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline()
        out["cpu_baseline_torch"] = cpu_baseline_torch()
        out["reference_cuda"] = reference_cuda_baseline(match, links, ol, tl, gout)
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


# dram bytes (read + write) of one forward + one backward launch of the gather on C2 bf16 V=32000
# (profiles/lsg_c2_bf16_v32000.md: measured on [8,1024,32000], traffic proportional to rows)
GATHER_TRAFFIC_BYTES = 4 * (532.76e6 + 5.34e6 + 536.99e6 + 469.23e6)   # captured on 8 of the 32 sentences


def extra_legs(torch, dev, ev, workloads, dag_loss, dag_best_alignment, dag_logsoftmax_gather_inplace, DagLossFunc,
               lib, _native, time_median):
    """Step times of the configurations that are not the headline: C1 (the translation-shaped step with
    fp16 logits, gather included), C3 (long sequences) and a peaky, trained-like C4 variant."""
    from da_transformer_b200 import last_status

    out = {}
    # C0: the reference's own CPU-runnable case (B=8, L=160, T<=20, V=1000, fp32 logits), the same step as C1
    b0 = workloads.config0().to(dev)
    leaf0 = b0.logits.clone().requires_grad_()
    links0 = b0.links.clone().requires_grad_()

    def c0_step():
        with torch.no_grad():
            _, sel = dag_logsoftmax_gather_inplace(leaf0.detach(), b0.select_idx)
            dag_best_alignment(sel.transpose(1, 2), b0.links, b0.output_length, b0.target_length)
        work = leaf0.clone()
        _, sel = dag_logsoftmax_gather_inplace(work, b0.select_idx)
        loss = dag_loss(sel.transpose(1, 2), links0, b0.output_length, b0.target_length)
        torch.autograd.grad(-(loss / b0.target_length).mean(), [leaf0, links0])

    med, lo, hi = time_median(c0_step, 10)
    out["C0"] = {"workload": f"B={b0.logits.shape[0]}, L={b0.logits.shape[1]}, T={b0.targets.shape[1]}, V={b0.logits.shape[2]}, "
                             f"fp32 logits: gather(no grad) + alignment + gather + dag_loss fwd+bwd + gather bwd, launched "
                             f"kernel by kernel through the Python front end (launch-bound at this size)",
                 "ms_per_step": med, "ms_min": lo, "ms_max": hi, "sentences_per_s": b0.logits.shape[0] / (med * 1e-3)}
    del b0, leaf0, links0

    # C1: B=64 ragged, fp16 logits [64, L<=512, 42000]; step = gather (no grad) + alignment + gather + loss
    # forward/backward + gather backward
    b = workloads.config1(with_logits=False)
    Bc, T, L = b.match_all.shape
    g = torch.Generator(device=dev)
    g.manual_seed(workloads.BASE_SEED + 1)
    logits = torch.empty(Bc, L, 42000, dtype=torch.float16, device=dev)
    for i in range(Bc):
        logits[i] = (torch.randn(L, 42000, device=dev, generator=g) * 2.0).to(torch.float16)
    bd = b.to(dev)
    sel_idx = bd.select_idx
    links = bd.links.clone().requires_grad_()
    leaf = logits.requires_grad_()

    def c1_step():
        with torch.no_grad():
            _, sel = dag_logsoftmax_gather_inplace(leaf.detach(), sel_idx)
            dag_best_alignment(sel.transpose(1, 2), bd.links, bd.output_length, bd.target_length)
        work = leaf.clone()       # the op overwrites its input with the gradient; part of the reference's step too
        _, sel = dag_logsoftmax_gather_inplace(work, sel_idx)
        loss = dag_loss(sel.transpose(1, 2), links, bd.output_length, bd.target_length)
        torch.autograd.grad(-(loss / bd.target_length).mean(), [leaf, links])

    def c1_dag_only():
        m = bd_match.requires_grad_()
        dag_best_alignment(m.detach(), bd.links, bd.output_length, bd.target_length)
        loss = dag_loss(m, links, bd.output_length, bd.target_length)
        torch.autograd.grad(loss.sum(), [m, links])

    with torch.no_grad():
        _, sel0 = dag_logsoftmax_gather_inplace(leaf.detach(), sel_idx)
    bd_match = sel0.transpose(1, 2).contiguous()
    med, lo, hi = time_median(c1_step, 10)
    med_d, _, _ = time_median(c1_dag_only, 10)
    out["C1"] = {"workload": f"B={Bc}, L={L}, T={T}, V=42000, fp16 logits: gather(no grad) + alignment + gather + "
                             f"dag_loss fwd+bwd + gather bwd (includes one clone of the logits)",
                 "ms_per_step": med, "ms_min": lo, "ms_max": hi, "sentences_per_s": Bc / (med * 1e-3),
                 "dag_ops_only_ms": med_d}
    del logits, leaf, sel0, bd_match, links
    torch.cuda.empty_cache()

    # C3: B=16, L=1024, T<=256
    b = workloads.config3().to(dev)
    m = b.match_all.clone().requires_grad_()
    l = b.links.clone().requires_grad_()

    def c3_step():
        dag_best_alignment(m.detach(), l.detach(), b.output_length, b.target_length)
        loss = dag_loss(m, l, b.output_length, b.target_length)
        torch.autograd.grad(loss.sum(), [m, l])

    med, lo, hi = time_median(c3_step, 10)

    def flagged_counts(batch, mm, ll):
        """(sentences redone by the exact kernels, sentences with the exact backward only) of one forward"""
        Bq, Tq, Lq = mm.shape
        Kq = ll.shape[2]
        al = torch.empty(Bq, Tq, Lq, device=dev)
        be = torch.empty_like(al)
        of = torch.empty(Bq, 2 * Tq + 2, dtype=torch.float64, device=dev)
        rs = torch.empty(Bq, device=dev)
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        sc = torch.empty(lib.dat_dag_loss_fast_scratch_bytes(Bq, Tq, Lq), dtype=torch.uint8, device=dev)
        fl = torch.zeros(2, dtype=torch.int32, device=dev)
        p, sp = _native.ptr, _native.stream_ptr
        _native.check(lib.dat_dag_loss_fast(p(mm.detach()), p(ll.detach()), p(batch.output_length), p(batch.target_length),
                                            p(al), p(be), p(of), p(rs), p(st), p(sc), Bq, Tq, Lq, Kq, sp(dev)), "fast")
        _native.check(lib.dat_dag_loss_fast_flagged(p(sc), p(fl), Bq, Tq, Lq, sp(dev)), "flagged")
        return int(fl[0].item()), int(fl[1].item()), int(torch.isfinite(rs).sum().item())

    c3_flagged = flagged_counts(b, m, l)
    out["C3"] = {"workload": f"B={b.match_all.shape[0]}, L=1024, T={b.match_all.shape[1]}: alignment + dag_loss fwd+bwd "
                             f"(rows do not fit in one SM's shared memory: sweep by clusters of 16 CTAs)",
                 "ms_per_step": med, "ms_min": lo, "ms_max": hi,
                 "sentences_per_s": b.match_all.shape[0] / (med * 1e-3),
                 "flagged_sentences": c3_flagged[0], "exact_backward_only_sentences": c3_flagged[1]}
    del m, l, b
    torch.cuda.empty_cache()

    # Peaky, trained-like C4 variant: link scores x 8, one dominant vertex per target token
    pk = workloads.config4_peaky().to(dev)
    m = pk.match_all.clone().requires_grad_()
    l = pk.links.clone().requires_grad_()
    Bp = m.shape[0]
    last_status()

    def pk_step():
        dag_best_alignment(m.detach(), l.detach(), pk.output_length, pk.target_length)
        loss = dag_loss(m, l, pk.output_length, pk.target_length)
        torch.autograd.grad(loss.sum(), [m, l])

    med, lo, hi = time_median(pk_step, 10)
    pk_flagged = flagged_counts(pk, m, l)
    out["C4_peaky"] = {"workload": f"B={Bp}, L=512, T=64, link scores x 8 and one dominant vertex per target token "
                                   f"(trained-like): alignment + dag_loss fwd+bwd",
                       "ms_per_step": med, "ms_min": lo, "ms_max": hi, "sentences_per_s": Bp / (med * 1e-3),
                       "flagged_sentences": pk_flagged[0], "exact_backward_only_sentences": pk_flagged[1],
                       "finite_losses": pk_flagged[2]}
    last_status()
    del m, l, pk
    torch.cuda.empty_cache()

    # The callers either side of the path: links from per-head scores (HBM-bound: the scores are read
    # once, the band written once; the backward writes the dense gradient once) and the decode-side DPs.
    from da_transformer_b200 import dag_links_from_heads, dag_node_passing_prob, dag_viterbi_decode

    Bh, Lh, H = 64, 512, 8
    K = Lh - 1
    g = torch.Generator(device=dev)
    g.manual_seed(workloads.BASE_SEED + 2)
    content = torch.randn(Bh, Lh, Lh, H, device=dev, generator=g).requires_grad_()
    gates = torch.log_softmax(torch.randn(Bh, Lh, H, device=dev, generator=g), -1).requires_grad_()
    nonpad = torch.ones(Bh, Lh, dtype=torch.bool, device=dev)
    glinks = torch.randn(Bh, Lh, K, device=dev, generator=g)
    peaks, peak_kind = measured_peaks()
    peak = peaks.get("hbm_gbs", 6650.0)

    def lh_fwd():
        with torch.no_grad():
            dag_links_from_heads(content, gates, nonpad_mask=nonpad, max_transition_length=K)

    lk = dag_links_from_heads(content, gates, nonpad_mask=nonpad, max_transition_length=K)

    def lh_bwd():
        torch.autograd.grad(lk, [content, gates], grad_outputs=glinks, retain_graph=True)

    f_ms, _, _ = time_median(lh_fwd, 10)
    b_ms, _, _ = time_median(lh_bwd, 10)
    tri = Bh * (Lh * (Lh - 1) // 2) * H * 4.0          # the successors' scores of every vertex
    band = Bh * Lh * K * 4.0
    dense = Bh * Lh * Lh * H * 4.0
    f_bytes = tri + band + Bh * Lh * H * 4.0
    b_bytes = tri + band + dense + 2 * Bh * Lh * H * 4.0
    out["links_from_heads"] = {
        "workload": f"log_multi_content [{Bh},{Lh},{Lh},{H}] fp32 -> band links [{Bh},{Lh},{K}], forward; backward "
                    f"writes the dense [B,L,L,H] gradient",
        "fwd_ms": f_ms, "bwd_ms": b_ms, "fwd_algorithmic_bytes": f_bytes, "bwd_algorithmic_bytes": b_bytes,
        "fwd_gbs": f_bytes / (f_ms * 1e-3) / 1e9, "bwd_gbs": b_bytes / (b_ms * 1e-3) / 1e9,
        "fwd_frac": f_bytes / (f_ms * 1e-3) / 1e9 / peak, "bwd_frac": b_bytes / (b_ms * 1e-3) / 1e9 / peak,
        "bound": "hbm", "peak_gbs": peak, "peak_kind": peak_kind}
    del content, gates, lk, glinks
    torch.cuda.empty_cache()

    raw = torch.randn(Bh, Lh, Lh, device=dev, generator=g)
    upper = torch.triu(torch.ones(Lh, Lh, dtype=torch.bool, device=dev), 1)
    sq = torch.log_softmax(raw.masked_fill(~upper, float("-inf")), -1)
    sq = sq.masked_fill(~upper, float("-inf")).contiguous()
    tok_logit = -torch.rand(Bh, Lh, device=dev, generator=g)
    tok = torch.randint(4, 1000, (Bh, Lh), device=dev, generator=g)
    olen = torch.full((Bh,), Lh, dtype=torch.long, device=dev)
    np_ms, _, _ = time_median(lambda: dag_node_passing_prob(sq), 10)
    vt_ms, _, _ = time_median(lambda: dag_viterbi_decode(sq, (tok_logit, tok), olen, Lh // 4), 10)
    out["decode"] = {"workload": f"square links [{Bh},{Lh},{Lh}] fp32: node-passing probabilities; Viterbi "
                                 f"decoding up to {Lh // 4} tokens with back-trace and token collapse",
                     "node_passing_ms": np_ms, "viterbi_ms": vt_ms}
    last_status()
    return out


if __name__ == "__main__":
    main()
