"""Benchmark of the DA-Transformer custom-op hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    (N > 1: python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...)

Workload (configuration C4): every GPU holds 512 sentences with graph length L=512
(= output_length), target_length ~ U{32..64} padded to T=64, fp32 links and fp32 match
(match has the distribution log-softmax over V=42000 bf16 N(0,2) logits gives at the
target tokens).  One step = dag_best_alignment + dag_loss forward (alpha+beta) +
dag_loss backward over the rank's sentences, then the SUM all-reduce of the scalar
statistics.  Per-GPU work is fixed as N grows (weak scaling); no tensor crosses GPUs.
The inputs (600 MB per GPU) are larger than L2, so no flush is needed between steps.

`value` is sentences/s with the inputs resident in HBM; `e2e` is the same step through
the public Python API with inputs copied from pinned host memory and the statistics
copied back every step.  `roofline` describes the dominant kernel (the alpha/beta sweep):
algorithmic special-function evaluations per launch (one exp per (t, i->j) term of the
log-domain recursion, the reference's formulation) over its CUDA-event duration, against
the special-function throughput measured on this device just before.  The shipped forward
runs the recursion in the probability domain and spends one FFMA per term instead, so the
fraction may exceed 1.  `gather` reports
logsoftmax_gather forward+backward on the C2 shape against the measured HBM copy
bandwidth.  `cpu_baseline` is the CPU oracle (a port of the reference's arithmetic) timed
on this host's cores on a bounded sample.
"""
import argparse
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
SENTENCES_PER_GPU = 512
L_GRAPH, T_MAX, VOCAB = 512, 64, 42000


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "sm_max_mhz": 1965.0}, "fallback"


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


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi.  It is started well before the
    timed region (its start-up talks to the driver for tens of milliseconds and would stall
    kernel launches if it overlapped the region); the samples whose timestamps fall inside the
    region are the ones reported."""
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
                rows.append((ts, float(parts[1]), float(parts[2]),
                             [n for n, v in zip(names, parts[5:9]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if self.t_begin is not None and self.t_begin - 0.02 <= r[0] <= self.t_end + 0.02]
        where = "timed region"
        if not inside:   # clock skew between nvidia-smi's timestamps and this process: use all samples
            inside, where = rows, "whole run (no sample carried a timestamp inside the region)"
        sm = [r[1] for r in inside]
        reasons = sorted({x for r in inside for x in r[3]})
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(r[2] for r in inside) if inside else None,
                "samples": len(sm), "window": where, "reasons": reasons}


# --------------------------------------------------------------------------------------
# CPU arm: the oracle (a port of the reference's arithmetic), all host threads
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


def cpu_baseline(budget_s=12.0):
    cores = os.cpu_count() or 1
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
                      f"(oracle/dag_oracle.c, OpenMP over sentences): best alignment + alpha + beta + backward"}


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
    cores = os.cpu_count() or 1
    n = cores
    sample = cpu_sample(n)
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_step(sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(sample)
    dt = time.perf_counter() - t0
    value = n * args.steps / dt
    desc = (f"{n} C4 sentences per step on {cores} host threads, fp32 CPU oracle port of the reference "
            f"arithmetic (the reference's own CPU path is PyTorch code that cannot travel to this box)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
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
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sentences", type=int, default=SENTENCES_PER_GPU, help="sentences per GPU")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gather", action="store_true")
    ap.add_argument("--eager", action="store_true", help="launch the step kernel by kernel instead of replaying a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from da_transformer_b200 import (_native, dag_best_alignment, dag_logsoftmax_gather_inplace,
                                     dag_loss, workloads)
    from da_transformer_b200 import dist as ddist

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
    peaks, peak_kind = measured_peaks()

    # ---- data: every rank owns one shard of the global batch
    # (shard r is drawn from its own generator, seed 20225 + 1000 r, so it is the same
    # data whatever the number of GPUs and no rank has to generate the other shards)
    B = args.sentences
    gen = workloads.generator(4 + 1000 * rank)
    shard = workloads.config4(gen=gen, B=B, L=L_GRAPH, V=VOCAB)
    host = [shard.match_all.pin_memory(), shard.links.pin_memory(),
            shard.output_length.pin_memory(), shard.target_length.pin_memory()]
    match = host[0].to(dev).requires_grad_()
    links = host[1].to(dev).requires_grad_()
    ol, tl = host[2].to(dev), host[3].to(dev)
    K = links.shape[2]
    sweep_exps, total_exps = exp_counts(shard.output_length, shard.target_length, K)
    gout = (-1.0 / (tl.double() * (B * world))).float()      # d(-(loss/tl).mean())/d loss

    ev = lambda: torch.cuda.Event(enable_timing=True)

    # The alignment and the loss only read match and links, so they are independent: inside the
    # captured graph the alignment is a parallel branch (a second stream during capture) and its
    # last, partly filled wave of CTAs overlaps the loss kernels.  Kernel-by-kernel launches keep one
    # stream (cross-stream tensor reuse made them slower, not faster).
    align_stream = torch.cuda.Stream(device=dev)

    def local_step(record=None, fork=False):
        cur = torch.cuda.current_stream(dev)
        if fork:
            align_stream.wait_stream(cur)
            with torch.cuda.stream(align_stream):
                path = dag_best_alignment(match.detach(), links.detach(), ol, tl)
        else:
            path = dag_best_alignment(match.detach(), links.detach(), ol, tl)
        if record is not None:
            record[0].record()
        loss = dag_loss(match, links, ol, tl)
        if record is not None:
            record[1].record()
        gm, gl = torch.autograd.grad(loss, [match, links], grad_outputs=gout)
        stats = ddist.sentence_stats(loss.detach(), tl)
        if fork:
            cur.wait_stream(align_stream)
        return stats, path, gm, gl

    def step(record=None):
        stats, path, gm, gl = local_step(record)
        return ddist.all_reduce_stats(stats), path, gm, gl

    # The ~30 launches of a step (ours and torch's small statistics kernels) cost more host time
    # than the kernels take on the device, so the rank-local part of the step is captured once
    # into a CUDA graph and replayed; the all-reduce stays an ordinary NCCL call after it.
    graph, graph_out, launch_mode = None, None, "eager"
    if not args.eager:
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(3):
                    local_step()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                graph_out = local_step(fork=True)
            graph, launch_mode = g, "cuda_graph"
        except Exception as exc:   # capture not possible here: fall back to kernel-by-kernel launches
            print(f"[bench] CUDA graph capture failed, running eagerly: {exc}", file=sys.stderr)
            graph, graph_out = None, None
            torch.cuda.synchronize()

    def timed_step(record=None):
        if graph is None:
            return step(record)
        graph.replay()
        return ddist.all_reduce_stats(graph_out[0]), graph_out[1], graph_out[2], graph_out[3]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- special-function roofline denominator, measured now
    sink = torch.zeros(1, device=dev)
    sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
    blocks, iters = sm_count * 2, 4096
    for _ in range(2):
        _native.check(lib.dat_probe_mufu(iters, blocks, _native.ptr(sink), _native.stream_ptr(dev)), "probe")
    e0, e1 = ev(), ev()
    e0.record()
    _native.check(lib.dat_probe_mufu(iters, blocks, _native.ptr(sink), _native.stream_ptr(dev)), "probe")
    e1.record()
    torch.cuda.synchronize()
    mufu_peak = blocks * 1024 * 8 * iters / (e0.elapsed_time(e1) * 1e-3)   # ex2 / s

    # ---- timed region: device-resident inputs
    uuid = str(torch.cuda.get_device_properties(dev).uuid)
    sampler = ClockSampler(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        timed_step()
    marks = [(ev(), ev()) for _ in range(args.steps)]
    barrier()
    sampler.begin()
    t0, t1 = ev(), ev()
    t0.record()
    for k in range(args.steps):
        stats, _, _, _ = timed_step(marks[k])
    t1.record()
    barrier()
    sampler.end()
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = t0.elapsed_time(t1)
    if graph is None:
        sweep_ms = sum(a.elapsed_time(b) for a, b in marks) / args.steps
    else:
        # events cannot be timed inside a replayed graph: time the same forward call, same inputs,
        # launched directly, once per timed step
        for a, b in marks:
            a.record()
            dag_loss(match, links, ol, tl)
            b.record()
        torch.cuda.synchronize()
        sweep_ms = sum(a.elapsed_time(b) for a, b in marks) / args.steps
    if world > 1:
        tmax = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        elapsed_ms = float(tmax.item())
    ms_per_step = elapsed_ms / args.steps
    value = B * world / (ms_per_step * 1e-3)
    final_stats = stats.cpu().tolist()

    # ---- per-op breakdown (rank 0, outside the headline region)
    def time_fn(fn, n=10):
        for _ in range(3):
            fn()
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    breakdown = {}
    if rank == 0:
        breakdown["best_alignment_ms"] = time_fn(lambda: dag_best_alignment(match.detach(), links.detach(), ol, tl))
        breakdown["loss_fwd_alpha_beta_ms"] = time_fn(lambda: dag_loss(match, links, ol, tl))
        with torch.no_grad():
            breakdown["loss_fwd_alpha_only_ms"] = time_fn(lambda: dag_loss(match, links, ol, tl))
        loss_keep = dag_loss(match, links, ol, tl)
        breakdown["loss_bwd_ms"] = time_fn(lambda: torch.autograd.grad(loss_keep, [match, links], grad_outputs=gout,
                                                                       retain_graph=True))
        fb = breakdown["loss_fwd_alpha_beta_ms"] + breakdown["loss_bwd_ms"]
        breakdown["dag_loss_fwd_bwd_only_sentences_per_s"] = B / (fb * 1e-3)

    # ---- end to end through the public API: host inputs in, statistics out, every step
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = 4 * 8
    stats_host = torch.empty(4, dtype=torch.float64).pin_memory()

    # The copies of step i+1 run on a second stream while step i computes (two device buffer sets),
    # the way an input pipeline feeds a training step; every step still pays its own full
    # host-to-device copy and its own device-to-host read of the statistics.
    copy_stream = torch.cuda.Stream(device=dev)
    bufs = [[torch.empty_like(h, device=dev) for h in host] for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    freed = [torch.cuda.Event() for _ in range(2)]

    def e2e_upload(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(freed[slot])          # the step that used this slot is done
            for d, h in zip(bufs[slot], host):
                d.copy_(h, non_blocking=True)
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

    e2e_run(3)
    barrier()
    t0, t1 = ev(), ev()
    t0.record()
    e2e_run(args.steps)
    t1.record()
    barrier()
    e2e_ms = t0.elapsed_time(t1)
    if world > 1:
        tmax = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_ms = float(tmax.item())
    e2e_value = B * world / (e2e_ms / args.steps * 1e-3)

    # ---- logsoftmax_gather on the C2 shape (rank-local), HBM roofline
    gather = None
    if rank == 0 and not args.no_gather:
        Bg, Lg, Vg, Sg = 32, 1024, 32000, 128
        g2 = torch.Generator(device=dev)
        g2.manual_seed(workloads.BASE_SEED + 2)
        base = (torch.randn(Bg, Lg, Vg, device=dev, generator=g2) * 2.0).to(torch.bfloat16)
        idx = torch.randint(0, Vg, (Bg, Lg, Sg), device=dev, generator=g2)
        gsel = torch.randn(Bg, Lg, Sg, device=dev, generator=g2)
        fwd_ms, bwd_ms = [], []
        for it in range(8):
            x = base.clone().requires_grad_()
            work = x.clone()
            a, b, c = ev(), ev(), ev()
            a.record()
            _, sel = dag_logsoftmax_gather_inplace(work, idx)
            b.record()
            sel.backward(gsel)
            c.record()
            torch.cuda.synchronize()
            if it >= 3:
                fwd_ms.append(a.elapsed_time(b))
                bwd_ms.append(b.elapsed_time(c))
            del x, work, sel
        e = 2
        fwd_bytes = Bg * Lg * Vg * e + 4 * Bg * Lg * Sg + 8 * Bg * Lg * Sg
        bwd_bytes = 2 * Bg * Lg * Vg * e + 4 * Bg * Lg * Sg + 8 * Bg * Lg * Sg
        f, bw = statistics.median(fwd_ms), statistics.median(bwd_ms)
        gather = {
            "workload": f"C2: logits [{Bg},{Lg},{Vg}] bf16 N(0,2), select_idx [{Bg},{Lg},{Sg}] int64",
            "fwd_ms": f, "bwd_ms": bw,
            "fwd_gbs": fwd_bytes / f / 1e6, "bwd_gbs": bwd_bytes / bw / 1e6,
            "fwd_bwd_gbs": (fwd_bytes + bwd_bytes) / (f + bw) / 1e6,
            "peak_gbs": peaks["hbm_gbs"], "peak_kind": peak_kind,
            "frac": (fwd_bytes + bwd_bytes) / (f + bw) / 1e6 / peaks["hbm_gbs"],
        }
        del base, idx, gsel

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    sweep_rate = sweep_exps / (sweep_ms * 1e-3)
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {
            "workload": ("C4: per GPU %d sentences, L=512 (=output_length), target_length~U{32..64}, T=64, "
                         "fp32 links [B,512,511] + fp32 match [B,64,512]; step = dag_best_alignment + dag_loss "
                         "fwd (alpha+beta) + bwd + scalar all-reduce") % B,
            "sentences_per_gpu": B, "global_sentences": B * world, "parallelism": f"dp{world}",
            "l2": "inputs (600 MB per GPU) exceed L2; no flush between steps",
            "launch": launch_mode,
        },
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        # per step: alignment (1: strip kernel), loss forward (4: order, strip sweep, check, exact
        # fallback), loss backward (3: grad_match, product-form grad_links, exact fallback), statistics (1)
        "gpu_launches": 9 * args.steps,
        "roofline": {
            "kernel": ("dag_loss forward = dag_strip_sweep_kernel (alpha and beta recursions, one CTA each, "
                       "exp(links) blocks held in registers) with its order, check and fallback launches"),
            "bound": "mufu", "achieved": sweep_rate / 1e9, "peak": mufu_peak / 1e9, "unit": "Gexp/s",
            "frac": sweep_rate / mufu_peak,
            # dram__bytes_read+write of dag_strip_sweep_kernel from the ncu capture summarised in
            # profiles/dag_strip_sweep_c4_148sent.md (108.7 MB for 148 sentences), scaled by sentences
            "traffic": 108.7e6 / 148 * B,
            "peak_kind": "measured on this device by dat_probe_mufu just before the timed region",
            "nominal_peak": 16 * sm_count * peaks.get("sm_max_mhz", 1965.0) * 1e6 / 1e9,
            "algorithmic_exps_per_launch": sweep_exps, "kernel_ms": sweep_ms,
            "step_frac_all_kernels": (total_exps / (ms_per_step * 1e-3)) / mufu_peak,
        },
        "breakdown": breakdown,
        "gather": gather,
        "loss_check": {"mean_nll_per_token": -final_stats[0] / final_stats[2], "invalid": final_stats[3]},
    }
    if gather is not None:
        out["roofline_gather"] = {"bound": "hbm", "achieved": gather["fwd_bwd_gbs"], "peak": peaks["hbm_gbs"],
                                  "unit": "GB/s", "frac": gather["frac"], "traffic": None,
                                  "peak_kind": peak_kind}
    if world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline()
        out["reference_cuda"] = reference_cuda_baseline(match, links, ol, tl, gout)
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
