"""Headline benchmark: sentences/s of the full forward bound pass (3-layer encoder, d_model 128,
4 heads, FFN 512, sequence length 32, one perturbed word, L-inf, eps 0.01, 256 sentences).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One process per GPU (torchrun for N > 1); the 256 sentences are split evenly over the ranks and no
collective is on the data path (sentences are independent).  A step is one bound pass over all
sentences.  Rank 0 prints one JSON line.  `--impl reference` times the reference's own CPU implementation of
the same pass on the host cores instead (its unchanged VerifierForward and Bounds when staged under oracle/_ref,
else the oracle port).
"""
import argparse
import ctypes
import json
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
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
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
            _REF["ver"] = reference_loader.build_reference_verifier(model, float("inf"))
        t0 = time.perf_counter()
        for s in range(n_sentences):
            reference_loader.reference_encoder_pass(_REF["ver"], emb[s:s + 1], CFG["index"], CFG["eps"])
        return time.perf_counter() - t0
    from oracle import bounds_oracle as O
    t0 = time.perf_counter()
    for s in range(n_sentences):
        O.encoder_forward(model, emb[s:s + 1], [CFG["index"]], float("inf"), CFG["eps"])
    return time.perf_counter() - t0


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
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": reference_kind(), "sample": sample_txt},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_cnn(args):
    """Secondary workload: conv 3->16, relu, conv 16->32 (stride 2), relu, linear 8192->10 on one 3x32x32
    image with every pixel perturbed (dim_in = 3072, Linf eps = 2/255).  The dim_in axis is sharded over the
    ranks; each relu all-reduces the partial norms over NCCL.  A step is one bound pass of the image."""
    import torch.distributed as dist
    import faith_b200
    from faith_b200.sharded import CnnVerifier
    from oracle import bounds_oracle as O
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = faith_b200.load()
    layers = O.make_cnn(5)
    img = torch.rand(3, 32, 32, generator=torch.Generator().manual_seed(5))
    ver = CnnVerifier(layers, dev)
    eps = 2.0 / 255

    def step():
        return ver.forward(img, float("inf"), eps, rank, world)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    n0 = lib.fb_launch_count()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        l, u = step()
    b.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms_step = float(ms.item()) / args.steps
        print(json.dumps({"metric": "images/sec for CNN bound pass (dim_in sharded)", "value": 1e3 / ms_step,
                          "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
                          "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                          "dtype": "f32", "data": "synthetic",
                          "config": {"workload": "CNN 3x32x32, conv3-16 s1, relu, conv16-32 s2, relu, linear 8192-10; "
                                                 "dim_in 3072 sharded over ranks, Linf eps 2/255",
                                     "collective": "NCCL all-reduce of [2, 16384] and [2, 8192] fp32 partial norms"},
                          "gpu_launches": int(lib.fb_launch_count() - n0),
                          "bounds": {"l0": float(l[0]), "u0": float(u[0])}}))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="faith_b200", choices=["faith_b200", "reference"])
    ap.add_argument("--sentences", type=int, default=CFG["sentences"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="encoder", choices=["encoder", "cnn"],
                    help="encoder = the headline metric; cnn = secondary line for the dim_in-sharded CNN pass")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload == "cnn":
        run_cnn(args)
        return

    import torch.distributed as dist
    import faith_b200
    from faith_b200 import _lib
    from oracle import bounds_oracle as O

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
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
    res_host = torch.empty(2, S).pin_memory()
    p_inf = float("inf")

    def step_resident():
        ver.forward(emb_dev, [CFG["index"]], p_inf, CFG["eps"], out=out)

    def step_e2e():
        e = emb_pinned.to(dev, non_blocking=True)
        ver.forward(e, [CFG["index"]], p_inf, CFG["eps"], out=out)
        res_host[0].copy_(out[0], non_blocking=True)
        res_host[1].copy_(out[1], non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(warmup):
        step_resident()
    barrier()
    launches0 = lib.fb_launch_count()
    sampler = ClockSampler(local) if rank == 0 else None
    ms_total = timed(step_resident, args.steps)
    clocks = sampler.stop() if sampler else None
    launches = lib.fb_launch_count() - launches0
    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)

    # per-operator device times of the same step, from CUDA events around every operator call
    lib.fb_profile_enable(1)
    barrier()
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

    # CUDA-core fp32 peak of this device, measured now (roof of the FFMA GEMM)
    scratch = torch.zeros(1, device=dev)
    fl = ctypes.c_double()
    lib.fb_bench_ffma(scratch.data_ptr(), 2000, ctypes.byref(fl), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    lib.fb_bench_ffma(scratch.data_ptr(), 20000, ctypes.byref(fl), torch.cuda.current_stream().cuda_stream)
    b.record()
    torch.cuda.synchronize()
    ffma_tflops = fl.value / a.elapsed_time(b) / 1e9

    viol = int(out[2].item())
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pk = peaks()
    ms_step = ms_total / args.steps
    value = total / (ms_step / 1e3)
    e2e_value = total / (ms_e2e / args.steps / 1e3)
    total_op_ms = sum(o["ms"] for o in per_op) or 1.0
    for o in per_op:
        o["share"] = o["ms"] / total_op_ms
        o["hbm_frac"] = o["gbs"] / pk["hbm_gbs"]
    dom = max(per_op, key=lambda o: o["ms"])
    if dom["op"] in ("matmul", "dot_product", "conv"):
        roofline = {"kernel": dom["op"], "bound": "tensor", "achieved": dom["tflops"], "peak": pk["bf16_sustained"],
                    "unit": "TFLOP/s", "frac": dom["tflops"] / pk["bf16_sustained"], "traffic": None,
                    "peak_source": pk["source"] + " (dense bf16, sustained)",
                    "avg_ms_per_call": dom["ms"] / dom["calls"], "share_of_step": dom["share"]}
        if dom["op"] == "matmul" and os.environ.get("FB_MATMUL_IMPL", "") != "ffma":
            # DRAM traffic per launch from the ncu capture of the 32-sentence case
            # (profiles/split_sign_gemm_tc_32_sentences.md): 134.4 MB read + 86.9 MB written against 268.6 MB
            # algorithmic (reads match; a third of the writes was still in L2 when the kernel ended), scaled to
            # this run's average launch by the bytes it processes
            roofline["traffic"] = dom["bytes_per_call"] * (134.41 + 86.90) / 268.6
            roofline["traffic_note"] = "bytes; ncu dram read+write of a 32-sentence launch scaled by algorithmic bytes"

            # tcgen05 kind::tf32 runs at half the bf16 rate; the 3xTF32 centre/radius kernel executes
            # 12*M*K*N tensor flops for the 8*M*K*N algorithmic ones
            tf32_peak = pk["bf16_tflops"] / 2.0
            roofline.update({"pipe": "tcgen05 kind::tf32 (3xTF32, centre/radius)", "pipe_peak": tf32_peak,
                             "frac_of_pipe": dom["tflops"] * 1.5 / tf32_peak,
                             "note": "achieved counts the algorithmic 8*M*K*N flops; pipe_peak = measured bf16 burst / 2; "
                                     "frac_of_pipe = achieved * 1.5 / pipe_peak (three TF32 products per fp32 product, "
                                     "two GEMMs instead of four)",
                             "hbm_frac": dom["gbs"] / pk["hbm_gbs"]})
        else:
            roofline.update({"pipe": "fp32 FFMA (CUDA cores)", "pipe_peak": ffma_tflops,
                             "frac_of_pipe": dom["tflops"] * (0.5 if dom["op"] != "dot_product" else 0.75) / ffma_tflops,
                             "note": "achieved counts algorithmic flops; the centre/radius kernels execute 1/2 (matmul, "
                                     "conv) or 3/4 (dot product) of them"})
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
                   "violation_flag": viol},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": emb_pinned.numel() * 4 * world,
                "d2h_bytes_per_step": 2 * S * 4 * world},
        "gpu_launches": int(launches),
        "roofline": roofline,
        "per_op": per_op,
        "ffma_peak_tflops": ffma_tflops,
    }
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        cpu_reference_pass(model, emb_host, 1, threads)
        n = 8
        secs = cpu_reference_pass(model, emb_host, n, threads)
        line["cpu_baseline"] = {"value": n / secs, "unit": UNIT, "cores": threads, "kind": reference_kind(),
                                "sample": baseline_sample_text(n)}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
