"""Headline benchmark: sentences/s of the full forward bound pass (3-layer encoder, d_model 128,
4 heads, FFN 512, sequence length 32, one perturbed word, L-inf, eps 0.01, 256 sentences).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One process per GPU (torchrun for N > 1); the 256 sentences are split evenly over the ranks and no
collective is on the data path (sentences are independent).  A step is one bound pass over all
sentences.  Rank 0 prints one JSON line.  Besides the headline it carries: the roofline of the dominant
kernel against the roofs measured in the same run (tensor pipe with TF32 operands, CUDA-core fp32, and the
HBM copy bandwidth of MEASURED_PEAKS.json), the same pass at eps = 1e-3, one entry per benchmark configuration
(`per_config`: C1 linear + relu, C2 attention dot product, C3 tanh + linear, C5 CNN), and the dim_in-sharded CNN
pass over all ranks (`cnn`).  `--impl reference` times the reference's own CPU implementation of
the same pass on the host cores instead (its unchanged VerifierForward and Bounds when staged under oracle/_ref,
else the oracle port).
"""
import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "sentences/sec for full-model bound pass"
UNIT = "sentences/s"
CFG = dict(layers=3, d_model=128, heads=4, ffn=512, L=32, sentences=256, eps=0.01, index=1, seed=4)
WORKLOAD = ("forward bound pass, 3-layer encoder d128 h4 ffn512 relu, layer_norm no_var, token-0 pooler + tanh, "
            "2-class head; L=32, 1 perturbed word (dim_in=128), Linf eps=0.01, 256 sentences")
KINDS = ["matmul", "relax", "dot_product", "mul_bounds", "elementwise", "conv"]
MIN_TIMED_SECONDS = 0.5
INF = float("inf")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v == "Active":
                    reasons.add(n)
        # samples taken while the GPU was busy have the highest clocks; use the upper half
        mhz.sort()
        busy = mhz[len(mhz) // 2:] if mhz else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


_REF = {}


def reference_kind():
    """"reference" when the reference's own modules are staged under oracle/_ref (oracle/stage_reference.py),
    else "port" (the restatement in oracle/bounds_oracle.py)."""
    if "kind" not in _REF:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import stage_reference
        _REF["kind"] = "reference" if stage_reference.staged_root() else "port"
    return _REF["kind"]


def cpu_reference_pass(model, emb, n_sentences, threads):
    """The reference's CPU path, one sentence per call (VerifierForward.py:13), PyTorch fp32: the unchanged
    VerifierForward._bound_input ... _bound_classifier (VerifierForward.py:93-125, 289-305) when its modules are
    staged, else the oracle port."""
    torch.set_num_threads(threads)
    if reference_kind() == "reference":
        import reference_loader
        if "ver" not in _REF:
            _REF["ver"] = reference_loader.build_reference_verifier(model, INF)
        t0 = time.perf_counter()
        for s in range(n_sentences):
            reference_loader.reference_encoder_pass(_REF["ver"], emb[s:s + 1], CFG["index"], CFG["eps"])
        return time.perf_counter() - t0
    from oracle import bounds_oracle as O
    t0 = time.perf_counter()
    for s in range(n_sentences):
        O.encoder_forward(model, emb[s:s + 1], [CFG["index"]], INF, CFG["eps"])
    return time.perf_counter() - t0


def cpu_model():
    try:
        with open("/proc/cpuinfo") as f:
            for ln in f:
                if ln.startswith("model name"):
                    return ln.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def reference_on_gpu(model, emb, dev):
    """The reference's own PyTorch Bounds and VerifierForward, unchanged, with its tensors on the GPU (what the
    reference's figures call "pytorch"): one sentence per call, 4 sentences after one warm-up.  A second baseline next
    to the CPU one; reported, not a target."""
    if reference_kind() != "reference":
        return {"unavailable": "reference modules are not staged under oracle/_ref"}
    try:
        import reference_loader
        ver = reference_loader.build_reference_verifier(model, INF, device=str(dev))
        e = emb[:5].to(dev)
        reference_loader.reference_encoder_pass(ver, e[0:1], CFG["index"], CFG["eps"])
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for s in range(1, 5):
            reference_loader.reference_encoder_pass(ver, e[s:s + 1], CFG["index"], CFG["eps"])
        torch.cuda.synchronize(dev)
        return {"value": 4 / (time.perf_counter() - t0), "unit": UNIT,
                "sample": "4 of the 256 sentences, one sentence per call, the reference's torch operators on this GPU"}
    except Exception as ex:   # the reference creates some tensors on the CPU; whatever stops it is reported, not hidden
        return {"unavailable": "%s: %s" % (type(ex).__name__, str(ex)[:200])}


def baseline_sample_text(n):
    if reference_kind() == "reference":
        return ("%d of the 256 sentences, one sentence per call through the reference's unchanged VerifierForward "
                "and Bounds (fp32 PyTorch on CPU)" % n)
    return "%d of the 256 sentences, one sentence per call, fp32 PyTorch on CPU (oracle port of the reference Bounds)" % n


def run_reference(args):
    """--impl reference: the CPU implementation, all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import bounds_oracle as O
    threads = os.cpu_count() or 1
    model = O.make_encoder(CFG["seed"], CFG["layers"], CFG["d_model"], CFG["heads"], CFG["ffn"])
    emb = torch.randn(CFG["sentences"], CFG["L"], CFG["d_model"], generator=torch.Generator().manual_seed(CFG["seed"]))
    sample = 4
    for _ in range(args.warmup):
        cpu_reference_pass(model, emb, 1, threads)
    times = [cpu_reference_pass(model, emb[i * sample:], sample, threads) for i in range(args.steps)]
    per_step = sum(times) / len(times)
    value = sample / per_step
    sample_txt = baseline_sample_text(sample) + ", per step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample_txt},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "cpu_model": cpu_model(), "kind": reference_kind(),
                         "sample": sample_txt},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------------ helpers
class Ctx:
    """Device, ranks and timing helpers shared by the parts of the benchmark."""

    def __init__(self):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import datetime
            # a collective that one rank never joins must end this run in minutes, not after the default ten
            dist.init_process_group("nccl", device_id=self.dev, timeout=datetime.timedelta(seconds=90))

    def smi_index(self):
        """Index nvidia-smi knows this rank's GPU by (CUDA_VISIBLE_DEVICES may renumber)."""
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.local < len(ids) and ids[self.local].isdigit():
                return int(ids[self.local])
        return self.local

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, steps):
        """Device time of `steps` calls of fn in ms (CUDA events on the launching stream), max over the ranks."""
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        self.barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return float(ms.item())

    def local_ms(self, fn, reps, warm=3):
        """Device time of one call in ms on this rank alone: (median, min) over `reps` single calls."""
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts), min(ts)

    def loop_ms(self, fn, n, warm=3):
        """Device time per call in ms when n calls are enqueued back to back (launch latency hidden)."""
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n


def measure_pipes(lib, ctx):
    """CUDA-core fp32 and tensor-pipe TF32 rates of this device, measured now (TFLOP/s)."""
    st = torch.cuda.current_stream().cuda_stream
    scratch = torch.zeros(1, device=ctx.dev)
    fl = ctypes.c_double()
    out = {}
    for name, call, small, big in (("ffma", lambda it: lib.fb_bench_ffma(scratch.data_ptr(), it, ctypes.byref(fl), st), 2000, 20000),
                                   ("tf32", lambda it: lib.fb_bench_tf32(it, ctypes.byref(fl), st), 200, 4000)):
        call(small)
        torch.cuda.synchronize()
        best = 0.0
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            rc = call(big)
            b.record()
            torch.cuda.synchronize()
            if rc == 0:
                best = max(best, fl.value / a.elapsed_time(b) / 1e9)
        out[name] = best
    return out


def roof_entry(name, ms, flops, nbytes, pipe_tflops, pipe_name, hbm_gbs, extra=None):
    """One measured operator against its binding roof: T_roof = max(flops / pipe, bytes / HBM)."""
    t_pipe = flops / (pipe_tflops * 1e9) if pipe_tflops else 0.0      # ms
    t_hbm = nbytes / (hbm_gbs * 1e6)
    bound = "hbm" if t_hbm >= t_pipe else pipe_name
    e = {"op": name, "ms": ms, "tflops": flops / ms / 1e9, "gbs": nbytes / ms / 1e6, "bound": bound,
         "roof_ms": max(t_pipe, t_hbm), "frac": max(t_pipe, t_hbm) / ms}
    if extra:
        e.update(extra)
    return e


# ------------------------------------------------------------------------------------- per-configuration lines
def epsilon_search_line(ver, emb_dev):
    """The reference's search for the largest certified radius (Verifier.py:106-147: per word a probe at max_eps and
    10 bisection steps, each a full bound pass) on 8 of the benchmark's sentences, every perturbable position: the
    probes of all (sentence, position) pairs of a round go through one call of the driver."""
    import faith_b200
    n_sent, iters, max_eps = 8, 10, 0.02
    emb = emb_dev[:n_sent].contiguous()
    labels = torch.zeros(n_sent, dtype=torch.int64, device=emb.device)
    search = faith_b200.EpsilonSearch(ver, INF, max_eps, iters, max_instances=256)
    search.run(emb[:1], labels[:1])        # warm-up (arena of the instance driver)
    search.passes = search.instances = 0
    torch.cuda.synchronize(emb.device)
    t0 = time.perf_counter()
    radii = search.run(emb, labels)
    torch.cuda.synchronize(emb.device)
    secs = time.perf_counter() - t0
    found = [v for d in radii for v in d.values()]
    return {"sentences": n_sent, "positions_per_sentence": len(radii[0]), "bisection_steps": iters, "max_eps": max_eps,
            "seconds": secs, "sentences_per_s": n_sent / secs, "bound_passes": search.instances,
            "bound_passes_per_s": search.instances / secs, "driver_calls": search.passes,
            "mean_certified_radius": sum(found) / len(found),
            "note": "the reference makes one verify_safety call per bound pass (cpu_baseline.value of them per second)"}


def graph_replay_ms(ctx, fn, replays=200):
    """Device time per replay of a CUDA graph that captured one call of `fn` (its launches and output allocations)."""
    fn()
    torch.cuda.synchronize(ctx.dev)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, capture_error_mode="thread_local"):   # other threads (a collective's watchdog) stay free to call CUDA
        keep = fn()   # noqa: F841  (outputs live in the graph's pool)
    for _ in range(5):
        g.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(ctx.dev)
    a.record()
    for _ in range(replays):
        g.replay()
    b.record()
    torch.cuda.synchronize(ctx.dev)
    return a.elapsed_time(b) / replays


def per_config_lines(ctx, lib, pipes, pk):
    """Benchmark configurations 1-3 and 5 on this GPU: device time of one launch sequence on its own (latency:
    the microsecond-sized problems are below a kernel launch) and the steady state over many independent
    instances in one call, each against its roof."""
    from faith_b200 import ops
    from faith_b200._lib import FB_RELU, FB_TANH
    from oracle import bounds_oracle as O
    dev = ctx.dev
    hbm = pk["hbm_gbs"]
    tf32_alg = pipes["tf32"] * 8.0 / 12.0     # algorithmic flops per second of the 3xTF32 centre/radius kernels
    ffma_alg = pipes["ffma"] * 2.0            # the CUDA-core GEMM executes half of the algorithmic flops
    g = torch.Generator().manual_seed(1)
    out = []

    def bounds(B, L, Di, Do, seed):
        gg = torch.Generator().manual_seed(seed)
        lw = (torch.rand(B, L, Di, Do, generator=gg) - 0.5) * 0.2
        uw = lw + torch.rand(B, L, Di, Do, generator=gg) * 0.02
        lb = torch.rand(B, L, Do, generator=gg) - 0.5
        ub = lb + torch.rand(B, L, Do, generator=gg) * 0.1
        return [t.to(dev) for t in (lw, uw, lb, ub)]

    # C1: Linear 64 -> 128 + bias, ReLU on [1, 16, 64, *] (eps 0.01, L-inf)
    W = (torch.randn(128, 64, generator=g) / 8).to(dev)
    bias = (0.1 * torch.randn(128, generator=g)).to(dev)

    def c1(x):
        y = ops.matmul(x[0], x[1], x[2], x[3], W, bias)
        return ops.relax(FB_RELU, y[0], y[1], y[2], y[3], INF, 0.01)

    def c1_work(B):
        M = B * 16 * 65
        return 8.0 * M * 64 * 128, 4.0 * (2 * M * 64 + 2 * M * 128) + 4.0 * (4 * M * 128)
    x1 = bounds(1, 16, 64, 64, 1)
    med, best = ctx.local_ms(lambda: c1(x1), 50)
    fl, by = c1_work(1)
    out.append(roof_entry("C1 linear 64->128 + relu, one instance [1,16,64,*]", best, fl, by, ffma_alg, "ffma", hbm,
                          {"median_ms": med, "mode": "single launch sequence (2 GEMM launches + 1 relaxation): launch latency"}))
    graph_ms = graph_replay_ms(ctx, lambda: c1(x1))
    out.append(roof_entry("C1 one instance, replayed from a CUDA graph", graph_ms, fl, by, ffma_alg, "ffma", hbm,
                          {"mode": "the same 3 launches captured once and replayed back to back: device-side latency without "
                                   "the host's launch cost"}))
    nb = 2048
    xb = bounds(nb, 16, 64, 64, 2)
    per = ctx.loop_ms(lambda: c1(xb), 10)
    fl, by = c1_work(nb)
    out.append(roof_entry("C1 steady state, %d independent instances per call" % nb, per, fl, by, tf32_alg, "tf32x3", hbm,
                          {"instances_per_s": nb / per * 1e3, "us_per_instance": per / nb * 1e3}))
    del xb

    # C2: attention scores Q.K^T, [4, 32, 128, 32] per instance (2 perturbed words, L2, eps 0.05)
    def c2(q, k):
        return ops.dot_product((q[0], q[1], q[2], q[3]), (k[0], k[1], k[2], k[3]), 2.0, 0.05, 2)

    def c2_work(B):
        return 16.0 * B * 32 * 32 * 129 * 32, 4.0 * (4.0 * B * 32 * 129 * 32 + 2.0 * B * 32 * 32 * 129)
    q, k = bounds(4, 32, 128, 32, 3), bounds(4, 32, 128, 32, 4)
    med, best = ctx.local_ms(lambda: c2(q, k), 50)
    fl, by = c2_work(4)
    out.append(roof_entry("C2 dot product Q.K^T, one instance [4,32,128,32]", best, fl, by, tf32_alg, "tf32x3", hbm,
                          {"median_ms": med, "mode": "single call (2 concretisations + bias + weight kernel): launch latency"}))
    graph_ms = graph_replay_ms(ctx, lambda: c2(q, k))
    out.append(roof_entry("C2 one instance, replayed from a CUDA graph", graph_ms, fl, by, tf32_alg, "tf32x3", hbm,
                          {"mode": "the same launches captured once and replayed back to back"}))
    nb = 1024
    qb, kb = bounds(4 * nb, 32, 128, 32, 5), bounds(4 * nb, 32, 128, 32, 6)
    per = ctx.loop_ms(lambda: c2(qb, kb), 10)
    fl, by = c2_work(4 * nb)
    out.append(roof_entry("C2 steady state, %d independent instances per call" % nb, per, fl, by, tf32_alg, "tf32x3", hbm,
                          {"instances_per_s": nb / per * 1e3, "us_per_instance": per / nb * 1e3}))
    del qb, kb

    # C3: tanh relaxation and Linear 256 -> 256 on [8, 64, 256, 256] (4 perturbed words, L1, eps 0.1)
    x3 = bounds(8, 64, 256, 256, 7)
    W3 = (torch.randn(256, 256, generator=g) / 16).to(dev)
    M3 = 8 * 64 * 257
    per = ctx.loop_ms(lambda: ops.relax(FB_TANH, x3[0], x3[1], x3[2], x3[3], 1.0, 0.1, 4), 20)
    out.append(roof_entry("C3 tanh relaxation [8,64,256,256]", per, 6.0 * M3 * 256, 4.0 * 4 * M3 * 256, None, "-", hbm))
    per = ctx.loop_ms(lambda: ops.matmul(x3[0], x3[1], x3[2], x3[3], W3, None), 20)
    out.append(roof_entry("C3 linear 256->256 [8,64,256,256]", per, 8.0 * M3 * 256 * 256, 4.0 * (4.0 * M3 * 256 + 256 * 256),
                          tf32_alg, "tf32x3", hbm))
    del x3

    # C5: CNN pass of one 3x32x32 image with every pixel perturbed (dim_in 3072), one GPU
    from faith_b200.sharded import CnnVerifier
    layers = O.make_cnn(5)
    img = torch.rand(3, 32, 32, generator=torch.Generator().manual_seed(5)).pin_memory()   # 12 KB, copied every pass
    ver = CnnVerifier(layers, dev)
    # Default route: rows kept as their windows only (fb_cw_*): 7 MB of rows instead of 600 MB; what remains is 14 small
    # launches, so the figure is launch- and latency-bound and a roofline fraction says little (bytes: the compact rows
    # written and read by each operator plus the 0.33 MB head weight, 2.3 GFLOP almost all in the head).
    per = ctx.loop_ms(lambda: ver.forward(img, INF, 2.0 / 255), 10)
    out.append(roof_entry("C5 CNN pass, one image (conv3-16, relu, conv16-32 s2, relu, linear 8192-10), 1 GPU; compact rows "
                          "(default route)", per, 2.3e9, 0.06e9, ffma_alg, "ffma", hbm,
                          {"images_per_s": 1e3 / per, "note": "latency-bound: 14 launches of a few microseconds each, replayed from a CUDA graph"}))
    # Dense rows, identity-input structure used (first convolution + relu written from the filter alone, windowed second
    # convolution): 1.41 GB moved.
    ver_rows = CnnVerifier(layers, dev, compact=False)
    per_r = ctx.loop_ms(lambda: ver_rows.forward(img, INF, 2.0 / 255), 10)
    out.append(roof_entry("C5 CNN pass, same image, dense rows with the identity-input structure used", per_r, 2.3e9, 1.41e9,
                          ffma_alg, "ffma", hbm, {"images_per_s": 1e3 / per_r}))
    per_d = ctx.loop_ms(lambda: ver.forward(img, INF, 2.0 / 255, dense=True), 10)
    out.append(roof_entry("C5 CNN pass, same image, identity materialised and every convolution run by the dense kernel",
                          per_d, 41.9e9, 2.3e9, ffma_alg, "ffma", hbm, {"images_per_s": 1e3 / per_d}))
    return out


def gemm_shape_lines(ctx, pipes, pk, S):
    """The three GEMM shapes of the headline pass at this rank's share of the sentences, each against its binding
    roof (tensor pipe with three TF32 products per fp32 product, or HBM)."""
    from faith_b200 import ops
    dev = ctx.dev
    L, D, F = CFG["L"], CFG["d_model"], CFG["ffn"]
    tf32_alg = pipes["tf32"] * 8.0 / 12.0
    rows = S * L
    out = []
    for (K, N, calls, what) in ((D, D, 4 * CFG["layers"], "projections (Q, K, V, attention output)"),
                                (D, F, CFG["layers"], "feed-forward 1"), (F, D, CFG["layers"], "feed-forward 2")):
        lw = torch.randn(rows, D, K, device=dev)
        uw = lw + 0.01
        lb = torch.randn(rows, K, device=dev)
        W = torch.randn(N, K, device=dev) * 0.02
        per = ctx.loop_ms(lambda: ops.matmul(lw, uw, lb, lb, W, None), 6)
        M = rows * (D + 1)
        out.append(roof_entry("K=%d N=%d" % (K, N), per, 8.0 * M * K * N, 4.0 * (2.0 * M * K + 2.0 * M * N + K * N), tf32_alg,
                              "tf32x3", pk["hbm_gbs"], {"calls_per_pass": calls, "what": what}))
        del lw, uw, lb, W
    return out


def cnn_sharded(ctx, lib, steps):
    """Benchmark configuration 5 with dim_in (3072 pixels) sharded over all ranks: the partial norms before each relu
    and before the final concretisation are all-reduced, by NCCL and by the library's one-shot exchange."""
    from faith_b200.comm import ALGO_NCCL, ALGO_ONESHOT, Comm
    from faith_b200.sharded import CnnVerifier
    from oracle import bounds_oracle as O
    layers = O.make_cnn(5)
    img = torch.rand(3, 32, 32, generator=torch.Generator().manual_seed(5)).pin_memory()   # 12 KB, copied every pass
    eps = 2.0 / 255
    res = {"workload": "CNN 3x32x32 (conv3-16 s1, relu, conv16-32 s2, relu, linear 8192-10), Linf eps 2/255, dim_in 3072 "
                       "sharded over the ranks; all-reduce of [2,8192] and [2,10] fp32 partial norms per image (the first relaxation "
                       "needs none); one C call per image, the image copied from pinned host memory inside the timed region",
           "n_gpus": ctx.world, "unit": "images/s"}
    comm = None
    if ctx.world > 1:
        comm = Comm.from_process_group(oneshot_floats=1 << 16)
    algos = [("nccl", ALGO_NCCL), ("oneshot", ALGO_ONESHOT)] if comm is not None else [("single", ALGO_NCCL)]
    # two routes: rows kept as their windows only (the default; so little work per image that sharding it cannot pay),
    # and dense rows (the formulation of the benchmark description: [3072, C, H, W] tensors sharded along dim_in)
    runs = [(a + "_dense_rows", algo, False) for a, algo in algos] + [(a + "_compact_rows", algo, True) for a, algo in algos]
    for name, algo, compact in runs:
        ver = CnnVerifier(layers, ctx.dev, comm=comm, algo=algo, compact=compact)
        for _ in range(3):
            l, u = ver.forward(img, INF, eps, ctx.rank, ctx.world)
        # (a single-GPU pass is replayed from a CUDA graph, which the library's launch counter does not see: the
        # launches of one pass are counted on an uncaptured run)
        counter = CnnVerifier(layers, ctx.dev, comm=comm, algo=algo, compact=compact, graph=False)
        counter.forward(img, INF, eps, ctx.rank, ctx.world)
        n0 = lib.fb_launch_count()
        counter.forward(img, INF, eps, ctx.rank, ctx.world)
        launches = int(lib.fb_launch_count() - n0)
        ms = ctx.timed(lambda: ver.forward(img, INF, eps, ctx.rank, ctx.world), steps)
        res[name] = {"ms_per_image": ms / steps, "images_per_s": 1e3 * steps / ms, "launches_per_image": launches,
                     "cuda_graph": bool(ver.graph and ctx.world == 1)}
        if comm is not None:
            comm.check(sync=True)
        l, u = ver.forward(img, INF, eps, ctx.rank, ctx.world)
        res[name]["bounds_logit0"] = [float(l[0]), float(u[0])]
    if comm is not None:
        comm.destroy()
    return res


# ----------------------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="faith_b200", choices=["faith_b200", "reference"])
    ap.add_argument("--sentences", type=int, default=CFG["sentences"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline only: skips the per-configuration lines, the eps = 1e-3 companion and the sharded CNN pass")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # plain peer loads and stores for everything this benchmark sends
    if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
        os.environ["NCCL_DEBUG"] = "WARN"            # NCCL's version banner goes to stdout, which carries the JSON line
    import faith_b200
    from faith_b200 import _lib
    from oracle import bounds_oracle as O

    ctx = Ctx()
    world, rank, dev, dist = ctx.world, ctx.rank, ctx.dev, ctx.dist
    lib = faith_b200.load()
    warmup = max(args.warmup, 3)

    total = args.sentences
    per = total // world
    lo = rank * per
    S = per if rank < world - 1 else total - lo
    model = O.make_encoder(CFG["seed"], CFG["layers"], CFG["d_model"], CFG["heads"], CFG["ffn"])
    emb_host = torch.randn(total, CFG["L"], CFG["d_model"], generator=torch.Generator().manual_seed(CFG["seed"]))
    emb_pinned = emb_host[lo:lo + S].contiguous().pin_memory()
    emb_dev = emb_pinned.to(dev)
    ver = faith_b200.EncoderVerifier(model, dev)
    out = (torch.empty(S, device=dev), torch.empty(S, device=dev), torch.empty(1, dtype=torch.int32, device=dev))
    lu_dev = torch.empty(S, 2, device=dev)
    gathered = [torch.empty(per if r < world - 1 else total - (world - 1) * per, 2, device=dev) for r in range(world)] \
        if rank == 0 else None
    res_host = torch.empty(total, 2).pin_memory() if rank == 0 else None
    eps_run = [CFG["eps"]]

    def step_resident():
        ver.forward(emb_dev, [CFG["index"]], INF, eps_run[0], out=out)

    def step_e2e():
        # the call a user makes: host embeddings in, (l, u) of all 256 sentences back on the host of rank 0
        e = emb_pinned.to(dev, non_blocking=True)
        ver.forward(e, [CFG["index"]], INF, eps_run[0], out=out)
        torch.stack((out[0], out[1]), dim=1, out=lu_dev)
        if world > 1:
            dist.gather(lu_dev, gathered, dst=0)
            if rank == 0:
                off = 0
                for t in gathered:
                    res_host[off:off + t.shape[0]].copy_(t, non_blocking=True)
                    off += t.shape[0]
        else:
            res_host.copy_(lu_dev, non_blocking=True)

    for _ in range(warmup):
        step_resident()
    ctx.barrier()
    # The timed region is `blocks` consecutive blocks of `steps` passes, sized from one probe block so that it lasts at
    # least half a second on every rank count (at 8 GPUs a pass is a few milliseconds and a 10-pass region would see two
    # clock samples).
    probe_ms = ctx.timed(step_resident, args.steps)
    blocks = max(1, int(math.ceil(MIN_TIMED_SECONDS * 1e3 / max(probe_ms, 1e-3))))
    n_steps = args.steps * blocks
    launches0 = lib.fb_launch_count()
    sampler = ClockSampler(ctx.smi_index()) if rank == 0 else None
    ms_total = ctx.timed(step_resident, n_steps)
    clocks = sampler.stop() if sampler else None
    launches = lib.fb_launch_count() - launches0
    tc_flag = lib.fb_tc_check()          # synchronising read of the tensor-core kernels' give-up flag
    viol = int(out[2].item())
    for _ in range(2):
        step_e2e()
    ms_e2e = ctx.timed(step_e2e, n_steps)

    # per-operator device times of the same step, from CUDA events around every operator call
    lib.fb_profile_enable(1)
    ctx.barrier()
    for _ in range(args.steps):
        step_resident()
    torch.cuda.synchronize()
    per_op = []
    for k, name in enumerate(KINDS):
        ms, calls, fl, by = ctypes.c_double(), ctypes.c_int64(), ctypes.c_double(), ctypes.c_double()
        _lib.check(lib.fb_profile_read(k, ctypes.byref(ms), ctypes.byref(calls), ctypes.byref(fl), ctypes.byref(by)),
                   "fb_profile_read")
        if calls.value:
            per_op.append(dict(op=name, calls=calls.value, ms=ms.value, tflops=fl.value / ms.value / 1e9,
                               gbs=by.value / ms.value / 1e6, flops_per_call=fl.value / calls.value,
                               bytes_per_call=by.value / calls.value))
    lib.fb_profile_enable(0)

    pipes = measure_pipes(lib, ctx)
    pk = peaks()

    extras = {}
    if not args.no_extras:
        # the same pass at eps = 1e-3, where the bounds of the third layer stay finite and tight
        eps_run[0] = 1e-3
        for _ in range(2):
            step_resident()
        ms_small = ctx.timed(step_resident, args.steps)
        l_s, u_s = out[0].clone(), out[1].clone()
        extras["eps_1e-3"] = {"ms_per_step": ms_small / args.steps, "value": total / (ms_small / args.steps / 1e3), "unit": UNIT,
                              "violation_flag": int(out[2].item()),
                              "finite": bool(torch.isfinite(l_s).all() and torch.isfinite(u_s).all()),
                              "mean_width": float((u_s - l_s).mean())}
        eps_run[0] = CFG["eps"]
        # The same pass with the last layer propagated for the first token only (the pooler reads nothing else of it;
        # the reference, and the headline figure above, propagate every position of every layer).  Reported beside
        # the headline, not as the headline: it does less work than the reference does.
        full_l, full_u = None, None
        step_resident()
        full_l, full_u = out[0].clone(), out[1].clone()
        ver_ft = faith_b200.EncoderVerifier(model, dev, first_token_only=True)
        ver_ft._ws = ver._ws            # same arena
        out_ft = (torch.empty(S, device=dev), torch.empty(S, device=dev), torch.empty(1, dtype=torch.int32, device=dev))

        def step_ft():
            ver_ft.forward(emb_dev, [CFG["index"]], INF, CFG["eps"], out=out_ft)
        for _ in range(2):
            step_ft()
        ms_ft = ctx.timed(step_ft, args.steps)
        wid = float((full_u - full_l).abs().max())
        extras["first_token_only_last_layer"] = {
            "ms_per_step": ms_ft / args.steps, "value": total / (ms_ft / args.steps / 1e3), "unit": UNIT,
            "violation_flag": int(out_ft[2].item()),
            "max_abs_difference_to_full_pass": float(max((out_ft[0] - full_l).abs().max(), (out_ft[1] - full_u).abs().max())),
            "bound_width": wid,
            "note": "keys and values of the last layer at every position, its query, attention row, attention output and "
                    "feed-forward block for token 0 alone; same bounds up to rounding"}
        ver_ft._ws = None
        del ver_ft
        ver._ws = None
        torch.cuda.empty_cache()
        extras["gemm_shapes"] = gemm_shape_lines(ctx, pipes, pk, S)
        torch.cuda.empty_cache()
        extras["cnn"] = cnn_sharded(ctx, lib, max(args.steps, 10))
        if rank == 0:
            extras["per_config"] = per_config_lines(ctx, lib, pipes, pk)
            extras["epsilon_search"] = epsilon_search_line(ver, emb_dev)
        ctx.barrier()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_step = ms_total / n_steps
    value = total / (ms_step / 1e3)
    e2e_value = total / (ms_e2e / n_steps / 1e3)
    total_op_ms = sum(o["ms"] for o in per_op) or 1.0
    for o in per_op:
        o["share"] = o["ms"] / total_op_ms
        o["hbm_frac"] = o["gbs"] / pk["hbm_gbs"]
    dom = max(per_op, key=lambda o: o["ms"])
    tf32_alg = pipes["tf32"] * 8.0 / 12.0
    if dom["op"] == "matmul" and os.environ.get("FB_MATMUL_IMPL", "") != "ffma":
        # The roof that binds is the one that alone would take longer: max(flops / tensor peak, bytes / HBM peak), i.e. the
        # larger of the two fractions.  Both are measured figures (TF32 rate in this run, HBM copy bandwidth of this pool).
        frac_t, frac_h = dom["tflops"] / tf32_alg, dom["gbs"] / pk["hbm_gbs"]
        tensor_side = {"achieved": dom["tflops"], "peak": tf32_alg, "unit": "TFLOP/s", "frac": frac_t,
                       "peak_source": "measured in this run: tcgen05 kind::tf32 rate %.0f TFLOP/s x 8/12 (the kernel executes "
                                      "three TF32 products per fp32 product on two GEMMs instead of four: 12 tensor flops per 8 "
                                      "algorithmic ones)" % pipes["tf32"],
                       "frac_of_bf16_sustained": dom["tflops"] / pk["bf16_sustained"]}
        hbm_side = {"achieved": dom["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": frac_h,
                    "peak_source": "%s HBM copy bandwidth" % pk["source"]}
        binding = hbm_side if frac_h >= frac_t else tensor_side
        roofline = {"kernel": "split_sign_gemm_tc (all products of the pass)", "bound": "hbm" if frac_h >= frac_t else "tensor",
                    "achieved": binding["achieved"], "peak": binding["peak"], "unit": binding["unit"], "frac": binding["frac"],
                    "peak_source": binding["peak_source"], "tensor": tensor_side, "hbm": hbm_side,
                    "avg_ms_per_call": dom["ms"] / dom["calls"], "share_of_step": dom["share"],
                    "hbm_frac": frac_h, "hbm_peak": pk["hbm_gbs"], "hbm_source": pk["source"],
                    # DRAM traffic per launch from the ncu capture of the 32-sentence case (profiles/): reads equal the
                    # algorithmic bytes, a third of the writes was still in L2 at kernel end (ratio 0.82 for the plain
                    # instantiation, 0.93 for the one that writes column norms)
                    "traffic": dom["bytes_per_call"] * 0.87,
                    "traffic_note": "bytes per launch; ncu dram read+write of 32-sentence launches scaled by algorithmic bytes"}
        shapes = extras.get("gemm_shapes")
        if shapes:
            w = sum(s["ms"] * s["calls_per_pass"] for s in shapes)
            roofline["frac_binding_roof_time_weighted"] = sum(s["roof_ms"] * s["calls_per_pass"] for s in shapes) / w
            roofline["by_shape"] = shapes
    elif dom["op"] in ("matmul", "dot_product", "conv"):
        ffma_alg = pipes["ffma"] * (2.0 if dom["op"] != "dot_product" else 4.0 / 3.0)
        roofline = {"kernel": dom["op"], "bound": "tensor", "achieved": dom["tflops"], "peak": ffma_alg, "unit": "TFLOP/s",
                    "frac": dom["tflops"] / ffma_alg, "traffic": None,
                    "peak_source": "measured in this run: CUDA-core fp32 FMA rate, scaled to algorithmic flops",
                    "avg_ms_per_call": dom["ms"] / dom["calls"], "share_of_step": dom["share"]}
    else:
        roofline = {"kernel": dom["op"], "bound": "hbm", "achieved": dom["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": dom["gbs"] / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                    "avg_ms_per_call": dom["ms"] / dom["calls"], "share_of_step": dom["share"]}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "sentences": total, "sentences_per_gpu": per, "sharding": "sentences",
                   "l2": "per-step working set is several GB per GPU, far above the 126 MB L2; no flush needed",
                   "timed_region": "%d blocks of %d steps = %d passes (>= %.1f s)" % (blocks, args.steps, n_steps, MIN_TIMED_SECONDS),
                   "violation_flag": viol, "tc_error_flag": tc_flag},
        "timed_steps": n_steps,
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": emb_host.numel() * 4,
                "d2h_bytes_per_step": total * 2 * 4,
                "path": "pinned host embeddings -> device, pass, (l, u) gathered to rank 0 and copied to its host"},
        "gpu_launches": int(launches),
        "launches_per_step": int(launches) // n_steps,
        "roofline": roofline,
        "per_op": per_op,
        "pipe_peaks_tflops": pipes,
    }
    if clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz"):
        # the pass at the clock the run actually had, expressed at the maximum clock: makes a power-capped single GPU and
        # uncapped GPUs of a larger run comparable
        line["ms_per_step_at_max_clock"] = ms_step * clocks["sm_mhz"] / clocks["sm_max_mhz"]
    line.update(extras)
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        cpu_reference_pass(model, emb_host, 1, threads)
        n = 8
        secs = cpu_reference_pass(model, emb_host, n, threads)
        line["cpu_baseline"] = {"value": n / secs, "unit": UNIT, "cores": threads, "cpu_model": cpu_model(),
                                "kind": reference_kind(), "sample": baseline_sample_text(n)}
        line["reference_torch_gpu"] = reference_on_gpu(model, emb_host, dev)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
