"""Benchmark of the hot path: YOLOv3-style post-process (decode + score mask + top-k + class-wise NMS), batch 64
per GPU, synthetic seeded logits.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extra]

A step is one pass of the post-process over one batch of 64 images whose logits are already resident in HBM
(`value`), or, for `e2e`, one call of the public module with HOST (pinned) inputs and a device->host read of the
detections.  With N > 1 every rank processes its own batch (weak scaling) and the ranks all-gather the padded
detection records with NCCL at the end of every step.  `--impl reference` times the CPU oracle (the un-functionalized
TorchScript program the reference's tests use as ground truth) on the host cores instead.
"""
import argparse
import contextlib
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

BATCH = 64
SIZES = (13, 26, 52)
NUM_BOXES = 3 * sum(s * s for s in SIZES)           # 10647
IMG_BYTES = NUM_BOXES * 85 * 4                        # 3 619 980 B of logits per image (algorithmic read)
OUT_BYTES_PER_IMG = 1000 * (5 * 4 + 8)                # <= 28 000 B of detections per image
METRIC = "yolov3_postprocess_batches_per_s"
UNIT = "batches/s (1 batch = 64 images)"


def workload_config(world: int) -> dict:
    """The `config` object of both arms (this build and --impl reference): identical keys and values."""
    return {"workload": "YOLOv3-style decode + score>0.5 mask + top-1000 + class-wise NMS 0.45, 3 scales 13/26/52, batch 64 per GPU",
            "batch_per_gpu": BATCH,
            "inputs": "seeded N(0,1) logits, 231.7 MB per step; the GPU arm rotates 3 input sets so that no step finds its logits in the 126 MB L2",
            "throughput_mode": "GPU arm: up to three batches in flight, one stream each, a block of steps replayed from a CUDA graph (latency_us is one batch at a time, call by call); CPU arm: one call after the other on all host threads",
            "collective": "none" if world == 1 else "gather of the 2 MB detection records of every rank to rank 0 over NVLink, on a second stream while the next steps compute (how: the line's gather key)"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU, sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 8 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 8 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 8 for i in range(4) if r[4 + i].lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------------------------------
# CPU oracle timing (reference arm and the cpu_baseline block)
# ------------------------------------------------------------------------------------------------------------------


def cpu_oracle_rate(sample_images: int, steps: int, warmup: int, threads=None):
    """TorchScript CPU oracle on `sample_images` images per step; returns (batches/s, ms per step, threads)."""
    import torch
    from oracle import workloads as W
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    mod = torch.jit.script(W.YOLOV3Post(sizes=SIZES))
    maps = W.make_yolo_inputs(sample_images)
    for _ in range(warmup):
        mod(maps)
    t0 = time.perf_counter()
    for _ in range(steps):
        mod(maps)
    dt = (time.perf_counter() - t0) / steps
    return (sample_images / BATCH) / dt, dt * 1e3, threads


def cpu_time_ms(fn, warmup: int, iters: int) -> float:
    """Median wall time of fn() in ms (time.perf_counter; the reference's harness times wall clock as well,
    functs/utils/evaluate.py:144-169)."""
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        t0 = time.perf_counter()
        fn()
        ts.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(ts)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # the whole 64-image batch per step (about half a second on 16 cores); at most 40 timed steps keep the run bounded
    sample = BATCH
    steps = max(1, min(args.steps, 40))
    rate, ms, threads = cpu_oracle_rate(sample, steps, max(1, min(args.warmup, 5)))
    sample_txt = (f"the whole batch: {sample} images per step (seeded N(0,1) logits), {steps} timed steps, TorchScript CPU "
                  f"oracle on {threads} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(max(1, args.gpus)),
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample_txt},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------------------


def time_events(fn, iters, torch):
    """Average device time of fn() in ms over iters back-to-back calls (CUDA events on the current stream)."""
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def cpu_baselines_other(torch, W):
    """TorchScript CPU oracle of the other four workloads on the host cores (bounded samples: about 15 s in total)."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    out = {}
    a, b, n = W.make_get_started_inputs()
    f = torch.jit.script(W.get_started)
    out["get_started"] = {"latency_us": cpu_time_ms(lambda: f(a, b, n), 16, 50) * 1e3, "cores": threads, "kind": "port",
                          "sample": "the configured call ([64, 1024] fp32, n = 64), median of 50"}
    loc, conf = W.make_ssd_inputs(8)
    m = torch.jit.script(W.SSDPost())
    ms = cpu_time_ms(lambda: m(loc, conf), 1, 3)
    out["ssd"] = {"batches_per_s": (8 / BATCH) / (ms * 1e-3), "ms_per_sample": ms, "cores": threads, "kind": "port",
                  "sample": "8 of the 64 images per call, median of 3, rate scaled to 64-image batches"}
    x, w_ih, w_hh, b_ih, b_hh = W.make_lstm_inputs()
    m = torch.jit.script(W.LSTMSeq(w_ih, w_hh, b_ih, b_hh))
    ms = cpu_time_ms(lambda: m(x), 2, 10)
    out["lstm"] = {"batches_per_s": 1e3 / ms, "latency_us": ms * 1e3, "cores": threads, "kind": "port",
                   "sample": "the configured call (T = 64, B = 64, H = 512), median of 10"}
    proto, coef, boxes = W.make_yolact_inputs(16)
    m = torch.jit.script(W.YolactMasks())
    ms = cpu_time_ms(lambda: m(proto, coef, boxes), 1, 3)
    out["yolact"] = {"batches_per_s": (16 / BATCH) / (ms * 1e-3), "ms_per_sample": ms, "cores": threads, "kind": "port",
                     "sample": "16 of the 64 images per call, median of 3, rate scaled to 64-image batches"}
    return out


def hbm_roofline(kernel: str, alg_bytes: float, kernel_ms: float, hbm_peak: float, peak_kind: str, note: str = "") -> dict:
    achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
    r = {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
         "peak_kind": peak_kind, "algorithmic_bytes_per_launch": alg_bytes}
    if note:
        r["note"] = note
    return r


def tf32_matmul_peak(torch) -> float:
    """Dense TF32 tensor-core throughput of this GPU in TFLOP/s, measured the way the bf16 peak of MEASURED_PEAKS.json was:
    torch.matmul on 8192^3 with TF32 enabled, best of 10 (CUDA events)."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        for _ in range(3):
            a @ b
        best = float("inf")
        for _ in range(10):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            a @ b
            e.record()
            torch.cuda.synchronize()
            best = min(best, s.elapsed_time(e))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def extra_workloads(torch, fb, W, hbm_peak, peak_kind="measured"):
    """Short device-time measurements of the other four configured workloads (not part of `value`)."""
    out = {}
    dev = "cuda"
    # C1 (0.5 MB: lives in L2; launch-latency bound by construction)
    a, b, n = W.make_get_started_inputs()
    bd = b.to(dev)
    res = torch.empty_like(bd)
    from functs_b200._lib import check, lib
    st = torch.cuda.current_stream().cuda_stream
    f1 = lambda: check(lib.functs_b200_rows_select_add_select_rev(bd.data_ptr(), res.data_ptr(), 64, 1024, n, 1.0, st))
    for _ in range(20):
        f1()
    ms = time_events(f1, 200, torch)
    out["get_started"] = {"latency_us": ms * 1e3, "kernels_per_call": 1, "hbm_gbs": 524288 / (ms * 1e-3) / 1e9,
                          "note": "0.5 MB working set (L2-resident); latency-bound",
                          "roofline": hbm_roofline("rows_add_kernel_v4", 524288, ms, hbm_peak, peak_kind,
                                                   "0.5 MB: one launch of about 5 us; 80 ns of HBM time at peak")}
    # C3, batch 64, three input sets rotated (190 MB per set > L2)
    loc, conf = [t.to(dev) for t in W.make_ssd_inputs(BATCH)]
    sets = [(loc, conf)] + [(loc.roll(s_, 0).clone(), conf.roll(s_, 0).clone()) for s_ in (1, 2)]
    ssd = fb.workloads.SSDBBox(W.ssd_priors(), device=dev)
    it = [0]

    def f3():
        loc, conf = sets[it[0] % 3]
        it[0] += 1
        ssd.forward_padded(loc, conf)
    for _ in range(5):
        f3()
    ms = time_events(f3, 30, torch)
    by = BATCH * (8732 * 81 * 4 + 8732 * 4 * 4)
    e0, e1, e2 = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    loc, conf = sets[0]
    _, bx_, sc_, dets_, ids_, cnt_ = ssd._bufs
    e0.record()
    fb.ops.ssd_softmax_decode(loc, conf, ssd.priors, 300.0, out=(bx_, sc_))
    e1.record()
    fb.ops.ssd_class_nms(bx_, sc_, 0.01, 200, 0.45, out=(dets_, ids_, cnt_))
    e2.record()
    torch.cuda.synchronize()
    out["ssd"] = {"batch": BATCH, "latency_us": ms * 1e3, "batches_per_s": 1e3 / ms, "kernels_per_call": 2,
                  "stage_us": {"softmax_decode": e0.elapsed_time(e1) * 1e3, "class_topk_nms": e1.elapsed_time(e2) * 1e3},
                  "algorithmic_gbs": by / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / hbm_peak,
                  "roofline": hbm_roofline("ssd_softmax_decode_kernel", by, e0.elapsed_time(e1), hbm_peak, peak_kind,
                                           "the streaming kernel of the pair; the class kernel works on 2.8 MB of scores per "
                                           "image and is bound by compare / min / max issue, not by HBM")}
    del sets, ssd
    # C5, batch 64 (279 MB per call > L2)
    proto, coef, boxes = [t.to(dev) for t in W.make_yolact_inputs(BATCH)]
    ym = fb.workloads.YolactBBoxMask(device=dev)
    f5 = lambda: ym(proto, coef, boxes)
    for _ in range(5):
        f5()
    ms = time_events(f5, 30, torch)
    by = BATCH * 4356432
    out["yolact"] = {"batch": BATCH, "latency_us": ms * 1e3, "batches_per_s": 1e3 / ms, "kernels_per_call": 1,
                     "algorithmic_gbs": by / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / hbm_peak,
                     "roofline": hbm_roofline("yolact_masks_kernel", by, ms, hbm_peak, peak_kind)}
    del proto, ym
    # C4, T=64 B=64 H=512
    x, w_ih, w_hh, b_ih, b_hh = W.make_lstm_inputs()
    lm = fb.workloads.LSTM(w_ih, w_hh, b_ih, b_hh, device=dev)
    xd = x.to(dev)
    f4 = lambda: lm.forward_device(xd)
    for _ in range(3):
        f4()
    ms = time_events(f4, 10, torch)
    fb.ops.raise_on_status(lm._status, "lstm bench")
    import ctypes
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for e in evs:
        e.record()
    torch.cuda.synchronize()
    lib.functs_b200_set_stage_events((ctypes.c_void_p * 3)(*[e.cuda_event for e in evs]), 3)
    f4()
    lib.functs_b200_set_stage_events(None, 0)
    torch.cuda.synchronize()
    proj_us, rec_us = evs[0].elapsed_time(evs[1]) * 1e3, evs[1].elapsed_time(evs[2]) * 1e3
    # the other recurrence (mode 2 = tcgen05, mode 3 = fp32 CUDA cores; mode 0 is whichever the library defaults to)
    modes = {}
    for mode in (2, 3):
        fm = lambda: lm.forward_device(xd, mode)
        for _ in range(2):
            fm()
        lib.functs_b200_set_stage_events((ctypes.c_void_p * 3)(*[e.cuda_event for e in evs]), 3)
        fm()
        lib.functs_b200_set_stage_events(None, 0)
        torch.cuda.synchronize()
        fb.ops.raise_on_status(lm._status, "lstm bench")
        modes["tcgen05_3xtf32" if mode == 2 else "cuda_core_fp32"] = {
            "latency_us": time_events(fm, 10, torch) * 1e3, "recurrence_us": evs[1].elapsed_time(evs[2]) * 1e3}
    tf32_peak = tf32_matmul_peak(torch)
    gemm_flop = 2.0 * 4096 * 512 * 2048          # one of the two GEMMs (projection; the recurrence has the same count)
    out["lstm"] = {"T": 64, "B": 64, "H": 512, "latency_us": ms * 1e3, "batches_per_s": 1e3 / ms,
                   "kernels_per_call": lm.kernels_last_call,
                   "stage_us": {"input_projection_tcgen05": proj_us, "recurrence": rec_us},
                   "recurrence_variants": modes,
                   "algorithmic_tflops": 17.18e9 / (ms * 1e-3) / 1e12,
                   "roofline": {"bound": "tensor", "kernel": "lstm_tc_gemm_kernel (hoisted input projection)",
                                "achieved": gemm_flop / (proj_us * 1e-6) / 1e12, "peak": tf32_peak, "unit": "TFLOP/s",
                                "frac": gemm_flop / (proj_us * 1e-6) / 1e12 / tf32_peak,
                                "peak_kind": "measured in this run: torch.matmul 8192^3 with TF32, best of 10",
                                "note": "algorithmic flops counted once; the 3xTF32 split issues three times as many on "
                                        "the pipe, and the stage time includes the operand split kernel",
                                "recurrence_tcgen05_tflops": gemm_flop / (modes["tcgen05_3xtf32"]["recurrence_us"] * 1e-6) / 1e12}}
    del lm, xd
    out["simple_programs"] = simple_ops(torch, fb, hbm_peak, peak_kind)
    return out


def simple_ops(torch, fb, hbm_peak, peak_kind):
    """The two single-group programs the reference times beside its models, three ways on the same device inputs: eager
    PyTorch (views and in-place writes), the functionalized program node by node (every Access / Assign operator is one of
    this library's stand-alone kernels), and the whole fusion group as ONE launch of the generic program kernel."""
    from functs_b200 import jit as J, simpleops
    out = {}
    g = torch.Generator().manual_seed(4242)
    n_sets = 12                                   # 12 x 12.8 MB of images: no call finds its input in the 126 MB L2
    imgs = [torch.rand(800, 1333, 3, generator=g).cuda() for _ in range(n_sets)]
    boxes = [torch.randn(3000, 4, generator=g).cuda()]
    offs = [torch.randn(3000, 4, generator=g).cuda()]
    cases = {
        "normalize_800x1333x3": (simpleops.normalize, [(im, 0.45, 4.4) for im in imgs], 2 * 800 * 1333 * 3 * 4),
        "offset2bbox_3000x4": (simpleops.offset2bbox, [(boxes[0], offs[0])], 3 * 3000 * 4 * 4),
    }
    for name, (fn, arg_sets, alg_bytes) in cases.items():
        want = fn(*arg_sets[0])
        node_by_node = J.script(fn)
        fused = J.build(fn, arg_sets[0])
        it = [0]

        def runner(f):
            def run():
                a = arg_sets[it[0] % len(arg_sets)]
                it[0] += 1
                return f(*a)
            return run
        rec = {}
        for label, f in (("eager", fn), ("access_assign_kernels", node_by_node), ("one_launch", fused)):
            it[0] = 0
            got = f(*arg_sets[0])
            if not torch.equal(got, want):
                raise SystemExit(f"bench: {name}/{label} differs from eager by {float((got - want).abs().max())}")
            r = runner(f)
            for _ in range(5):
                r()
            l0 = fb.launch_count()
            r()
            torch.cuda.synchronize()
            launches = fb.launch_count() - l0
            rec[label] = {"latency_us": time_events(r, 50, torch) * 1e3, "launches_of_this_library": launches}
        i0 = J.interpreted_functor_runs()
        fused(*arg_sets[0])
        rec["one_launch"]["interpreted_functors"] = J.interpreted_functor_runs() - i0
        rec["roofline"] = hbm_roofline("generic_group_kernel_param", alg_bytes, rec["one_launch"]["latency_us"] * 1e-3,
                                       hbm_peak, peak_kind,
                                       "time of the whole call on the stream (host-side program flattening included when "
                                       "the device is idle)")
        out[name] = rec
    return out


def bind_to_gpu_numa_node(index: int):
    """Pins this rank's host threads to the CPU cores next to its GPU (NVML's ideal affinity mask; read-only query), before
    any host buffer is allocated: the pinned input buffers are then first touched, and so placed, on the GPU's own NUMA
    node, and the host-to-device copies of the ranks do not all cross the same socket link.  Best effort.  Returns the
    previous affinity set (restored before the CPU baseline runs, which uses every host core)."""
    before = os.sched_getaffinity(0)
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {w * 64 + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        allowed = os.sched_getaffinity(0)
        if cpus & allowed:
            os.sched_setaffinity(0, cpus & allowed)
    except Exception:
        pass
    return before


def run_ours(args):
    import torch
    import torch.distributed as dist
    import functs_b200 as fb
    from functs_b200 import dist as fdist
    from functs_b200._lib import check, launch_count, lib
    from oracle import workloads as W  # input generator + cpu_baseline leg only

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: functs_b200 has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    all_cpus = bind_to_gpu_numa_node(local)
    if world > 1:
        # the gather shares the GPU with the next step's kernels: its (few) CTAs must not queue behind theirs
        opts = None
        if args.comm_priority == "high":
            opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    hbm_peak, peak_kind = measured_peaks()

    # ---- inputs: this rank's 64 images; three sets rotated so that no step finds its logits in L2 ----
    n_sets = 3
    host_maps = W.make_yolo_inputs(BATCH, first=rank * BATCH)
    sets = [[m.to(dev) for m in host_maps]]
    for s_ in range(1, n_sets):
        sets.append([m.roll(s_, 0).clone() for m in sets[0]])  # same images, permuted inside the batch
    pinned = [m.pin_memory() for m in host_maps]
    bytes_in = sum(m.numel() * 4 for m in host_maps)

    topk, cap = 1000, NUM_BOXES * 80
    plan = fb.ops.YoloPostprocessPlan(BATCH, SIZES, topk, cap, device=dev)
    # Throughput mode: several batches in flight, one stream each (each with its own outputs and scratch), so that the decode
    # kernel of one batch (bandwidth-bound, fills the machine) overlaps the top-k / NMS kernels of the other (a few
    # hundred CTAs of dependent integer work).  Latency (one batch, one stream) is measured and reported separately.
    in_flight = max(1, min(4, args.in_flight))
    plans = [plan] + [fb.ops.YoloPostprocessPlan(BATCH, SIZES, topk, cap, device=dev) for _ in range(in_flight - 1)]
    work_streams = [torch.cuda.Stream(dev) for _ in range(in_flight)]
    rec = torch.empty(BATCH, topk, fdist.RECORD_WORDS, dtype=torch.int32, device=dev)
    # only rank 0 holds the gathered detections
    rec_all = (torch.empty(world * BATCH, topk, fdist.RECORD_WORDS, dtype=torch.int32, device=dev)
               if world > 1 and rank == 0 else None)
    # multi-GPU: the gather of step i runs on a second stream while the next steps compute; ten record buffers in rotation,
    # so that no batch waits for the gather of an earlier one
    n_rec = 1
    group = 1                      # steps whose records travel in one gather (N > 1)
    packed_ev = gathered_ev = cap_packed_ev = cap_gathered_ev = None
    pusher, gather_note = None, "NCCL gather (dist.gather)"
    if world > 1:
        group = max(1, int(args.gather_every))
        n_rec = max(2, -(-(int(args.rec_buffers) if args.rec_buffers > 0 else 10) // group), -(-(in_flight + group) // group))
        comm_stream = torch.cuda.Stream(dev, priority=-1 if args.comm_priority == "high" else 0)
        # record buffers: n_rec groups of `group` steps each; a group is gathered in one go when its last step is done
        recs = [torch.empty(group, BATCH, topk, fdist.RECORD_WORDS, dtype=torch.int32, device=dev) for _ in range(n_rec)]
        rec_alls = ([torch.empty(world * group * BATCH, topk, fdist.RECORD_WORDS, dtype=torch.int32, device=dev)
                     for _ in range(n_rec)] if rank == 0 else [None] * n_rec)
        packed_ev = [[torch.cuda.Event() for _ in range(group)] for _ in range(n_rec)]
        gathered_ev = [torch.cuda.Event() for _ in range(n_rec)]
        for e in gathered_ev:
            e.record()
        cap_packed_ev = [[torch.cuda.Event() for _ in range(group)] for _ in range(n_rec)]
        cap_gathered_ev = [torch.cuda.Event() for _ in range(n_rec)]
        # The gather itself: NCCL send / receive pairs (dist.gather), or --gather one-sided: every rank pushes its records
        # into its slot of rank 0's buffers with an asynchronous copy (CUDA IPC mapping, copy engine over NVLink, no
        # kernel on either side).  Measured at N = 2: 98 us per step one-sided against 88 with NCCL, hence the default.
        if args.gather == "one-sided":
            try:
                pusher = fdist.OneSidedGather((group * BATCH, topk, fdist.RECORD_WORDS), n_rec, dev, dst=0)
                gather_note = "one-sided: asynchronous peer copies into rank 0's buffers (CUDA IPC), one small all-reduce per block"
            except RuntimeError as exc:
                pusher, gather_note = None, f"NCCL gather (one-sided set-up failed: {str(exc)[:120]})"
        gather_note += f"; the records of {group} consecutive steps per transfer" if group > 1 else "; one transfer per step"
    # per-step stage events, recorded inside the one-call entry point through its profiling hook
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    for row in ev:
        for e in row:
            e.record()  # materialises the CUDA event handle
    torch.cuda.synchronize()
    import ctypes
    ev_handles = [(ctypes.c_void_p * 4)(*[e.cuda_event for e in row]) for row in ev]

    def step(i, handles=None, pipelined=False, capturing=False, last=False):
        j, slot = (i // group) % n_rec, i % group   # record buffer group and place inside it (N > 1)
        k = i % in_flight                            # plan and stream of this batch
        p = plans[k] if pipelined else plan
        ctx = torch.cuda.stream(work_streams[k]) if pipelined else contextlib.nullcontext()
        with ctx:
            if handles is not None:
                lib.functs_b200_set_stage_events(handles, 4)
            cur = torch.cuda.current_stream()
            # (a capture has events of its own: an event recorded inside a capture cannot be waited for outside it)
            p_ev, g_ev = (cap_packed_ev, cap_gathered_ev) if capturing else (packed_ev, gathered_ev)
            if world > 1 and not (capturing and i < n_rec * group):
                # the gather that used this group of record buffers n_rec groups ago is done (inside a capture the first
                # uses have no earlier gather: a replay starts after the previous one has finished)
                cur.wait_event(g_ev[j])
            # memset + decode/mask/compact + binned top-k + NMS: 3 kernels; with N > 1 the NMS kernel also writes the records
            p.run(sets[i % n_sets], 0.5, 0.45, records=recs[j][slot] if world > 1 else None)
            if handles is not None:
                lib.functs_b200_set_stage_events(None, 0)
            if world > 1:
                p_ev[j][slot].record(cur)
                if not pipelined:
                    # one batch at a time (the latency block): this step's records travel on their own, right away
                    with torch.cuda.stream(comm_stream):
                        comm_stream.wait_event(p_ev[j][slot])
                        if not args.no_gather:
                            fdist.gather_records_to(recs[j][slot], 0, out=rec_all)
                        g_ev[j].record(comm_stream)
                elif slot == group - 1 or last:   # the group is complete (or the block ends): its records travel now
                    with torch.cuda.stream(comm_stream):
                        for q in range(slot + 1):
                            comm_stream.wait_event(p_ev[j][q])
                        whole = recs[j].view(group * BATCH, topk, fdist.RECORD_WORDS)
                        if args.no_gather:
                            pass
                        elif pusher is not None:
                            pusher.push(whole, j)        # copy engine over NVLink into rank 0's buffer: no kernel
                        else:
                            fdist.gather_records_to(whole, 0, out=rec_alls[j])
                        g_ev[j].record(comm_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    n_warm = max(args.warmup, 3)
    for i in range(n_warm):
        step(i, last=i == n_warm - 1)
    barrier()  # the pipelined steps run on other streams and reuse the first plan's outputs and scratch
    for i in range(n_warm):
        step(i, pipelined=True, last=i == n_warm - 1)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # The timed unit is a block of exactly `steps` steps between two barriers (device time, CUDA events).  One block of 20
    # steps is under 3 ms of GPU time, so the block is repeated until about a second of device time has been measured;
    # `value` comes from the median block.  The first block also records the per-stage events.
    def issue_block(main, fork_event, with_stage_events, pipelined, capturing=False):
        """The `steps` steps of one block, forked from / joined into the stream `main`."""
        if pipelined:
            for ws in work_streams:
                ws.wait_event(fork_event)
        if world > 1 and capturing:
            comm_stream.wait_event(fork_event)
        for i in range(args.steps):
            step(i, ev_handles[i] if with_stage_events else None, pipelined, capturing, last=i == args.steps - 1)
        if pipelined:
            for ws in work_streams:
                main.wait_stream(ws)
        if world > 1:
            if pusher is not None and not args.no_gather:
                with torch.cuda.stream(comm_stream):
                    pusher.landed()         # one small all-reduce: every rank's pushes of this block have arrived
            main.wait_stream(comm_stream)   # the block ends when the last gather has landed

    # Throughput blocks are replayed from a CUDA graph (kernels, memsets, events and the NCCL gather of all `steps` steps,
    # captured once): issuing a step from Python costs about as much host time as the step takes on the GPU once a
    # gather call is part of it, and the ranks then run at the speed of rank 0's interpreter.
    graph, graph_note = None, "off"
    if in_flight > 1 and not args.no_graph:
        try:
            cap_stream = torch.cuda.Stream(dev)
            g = torch.cuda.CUDAGraph()
            l_before = launch_count()
            with torch.cuda.graph(g, stream=cap_stream):
                fork = torch.cuda.Event()
                fork.record(cap_stream)
                issue_block(cap_stream, fork, False, True, capturing=True)
            graph, graph_note = g, f"one graph per block of {args.steps} steps"
            graph_launches = launch_count() - l_before
        except Exception as exc:  # noqa: BLE001 - reported in the JSON line, the block is then issued call by call
            graph, graph_note = None, f"capture failed: {str(exc).splitlines()[0][:160]}"
        barrier()

    def timed_block(with_stage_events: bool, pipelined: bool):
        t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        main = torch.cuda.current_stream()
        t_start.record(main)
        if pipelined and graph is not None:
            graph.replay()
        else:
            issue_block(main, t_start, with_stage_events, pipelined)
        t_end.record(main)
        barrier()
        return t_start.elapsed_time(t_end)

    # block 0: one batch at a time on one stream, with the per-stage events -> latency and the kernels' own durations
    seq_ms = timed_block(True, False)
    launches0 = launch_count()
    block_ms = [timed_block(False, in_flight > 1)]
    launches = (launch_count() - launches0) if graph is None else graph_launches
    # every rank must run the same number of blocks: rank 0's first block decides
    want = torch.tensor([max(1.0, min(2000.0, 1000.0 / max(block_ms[0], 1e-3)))], dtype=torch.float64, device=dev)
    if world > 1:
        dist.broadcast(want, 0)
    repeats = int(want.item())
    for _ in range(repeats - 1):
        block_ms.append(timed_block(False, in_flight > 1))
    total_ms = statistics.median(block_ms)
    fb.ops.raise_on_status(plan.status, "bench")
    decode_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    select_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    nms_ms = statistics.mean(e[2].elapsed_time(e[3]) for e in ev)
    kept = int(plan.counts.sum())

    # ---- e2e: public module, pinned host inputs, detections read back ----
    mod = fb.workloads.YOLOV3BBox(sizes=SIZES, device=dev)
    e2e_steps = max(2, min(args.steps, 10))

    def e2e_step():
        dets, labels, flat_ids, cnt = mod.forward_padded(pinned)
        if world > 1:
            fdist.pack_detections(dets, labels, flat_ids, cnt, out=rec)
            r = fdist.gather_records_to(rec, 0, out=rec_all)
            return r.cpu() if rank == 0 else None   # only rank 0 holds (and reads back) the gathered detections
        return dets.cpu(), labels.cpu(), cnt.cpu()
    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    bytes_out = (world * rec.numel() * 4) if world > 1 else (plan.dets.numel() * 4 + plan.labels.numel() * 8 + plan.counts.numel() * 4)
    clocks = sampler.stop() if rank == 0 else None

    # ---- max over ranks ----
    stats = torch.tensor([total_ms, e2e_ms, decode_ms, select_ms, nms_ms, seq_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, decode_ms, select_ms, nms_ms, seq_ms = [float(v) for v in stats.tolist()]

    if rank == 0:
        ms_per_step = total_ms / args.steps
        alg_bytes = BATCH * IMG_BYTES                       # bytes the decode kernel must read per launch
        achieved = alg_bytes / (decode_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": world * 1e3 / ms_per_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(world),
            "repeats": repeats, "timed_region_s": sum(block_ms) / 1e3,
            "ms_per_step_spread": {"min": min(block_ms) / args.steps, "median": ms_per_step, "max": max(block_ms) / args.steps},
            "in_flight": in_flight,
            "cuda_graph": graph_note,
            **({"gather": gather_note} if world > 1 else {}),
            **({"diagnostic": "gather skipped (--no-gather): not a result"} if args.no_gather else {}),
            "latency_us": seq_ms / args.steps * 1e3, "kernels_per_call": launches / args.steps,
            "images_per_s": world * BATCH * 1e3 / ms_per_step,
            "stage_us": {"decode_mask_compact": decode_ms * 1e3, "select_topk": select_ms * 1e3, "nms": nms_ms * 1e3},
            "detections_kept_last_step": kept, "select_fallbacks_last_step": plan.select_fallbacks(),
            "gpu_launches": launches,
            "e2e": {"value": world * 1e3 / e2e_ms, "unit": UNIT, "h2d_bytes_per_step": bytes_in,
                    "d2h_bytes_per_step": bytes_out, "ms_per_step": e2e_ms, "steps": e2e_steps},
            "roofline": {"bound": "hbm", "kernel": "yolo_decode_staged_kernel", "achieved": achieved, "peak": hbm_peak,
                         "unit": "GB/s", "frac": achieved / hbm_peak, "peak_kind": peak_kind, "traffic": None,
                         "algorithmic_bytes_per_launch": alg_bytes, "whole_step_frac": (alg_bytes + BATCH * OUT_BYTES_PER_IMG) / (ms_per_step * 1e-3) / 1e9 / hbm_peak},
            "clocks": clocks,
        }
        traffic_file = os.path.join(ROOT, "profiles", "yolo_decode_traffic.json")
        if os.path.exists(traffic_file):
            with open(traffic_file) as f:
                line["roofline"]["traffic"] = json.load(f).get("dram_bytes_per_launch_b64")
        if not args.no_extra and world == 1:
            os.sched_setaffinity(0, all_cpus)   # the CPU baseline may use every host core again
            cpu_rate, cpu_ms, threads = cpu_oracle_rate(BATCH, 5, 1)
            line["cpu_baseline"] = {"value": cpu_rate, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": "the whole batch (64 images) per step x 5 steps, TorchScript CPU oracle", "ms_per_step": cpu_ms}
            # latency view (BATCH-independent unit: images/s) for batch 1 and 8, and a 1-thread figure on 8 images
            by_batch = {}
            for bsz, it_ in ((1, 20), (8, 8)):
                r_, ms_, _ = cpu_oracle_rate(bsz, it_, 2)
                by_batch[str(bsz)] = {"ms_per_call": ms_, "images_per_s": bsz / (ms_ * 1e-3)}
            by_batch[str(BATCH)] = {"ms_per_call": cpu_ms, "images_per_s": BATCH / (cpu_ms * 1e-3)}
            r1, ms1, _ = cpu_oracle_rate(8, 2, 1, threads=1)
            line["cpu_baseline"]["by_batch"] = by_batch
            line["cpu_baseline"]["one_thread"] = {"value": r1, "unit": UNIT, "sample": "8 images per step x 2 steps, rate scaled to 64-image batches"}
            del sets
            torch.cuda.empty_cache()
            try:
                line["workloads"] = extra_workloads(torch, fb, W, hbm_peak, peak_kind)
                cpu_other = cpu_baselines_other(torch, W)
                for k, v in cpu_other.items():
                    line["workloads"][k]["cpu_baseline"] = v
            except Exception as exc:  # the headline number must still be printed
                line["workloads"] = {"error": repr(exc)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        if graph is not None:
            # A captured graph that holds NCCL kernels keeps the communicator busy: tearing the process group down with
            # it alive did not return (the run was killed by its time limit).  Everything is printed and every rank is
            # past the barrier: leave without the teardown.
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)
        dist.destroy_process_group()


def run_single_workload(args):
    """Runs a few steps of ONE of the other workloads and exits (no JSON line): the command ncu captures wrap."""
    import torch
    import functs_b200 as fb
    from oracle import workloads as W  # seeded input generator only
    dev = "cuda"
    b = args.batch
    if args.only == "ssd":
        loc, conf = [t.to(dev) for t in W.make_ssd_inputs(b)]
        mod = fb.workloads.SSDBBox(W.ssd_priors(), device=dev)
        fn = lambda: mod.forward_padded(loc, conf)
    elif args.only == "yolact":
        proto, coef, boxes = [t.to(dev) for t in W.make_yolact_inputs(b)]
        mod = fb.workloads.YolactBBoxMask(device=dev)
        fn = lambda: mod(proto, coef, boxes)
    elif args.only == "lstm":
        x, w_ih, w_hh, b_ih, b_hh = W.make_lstm_inputs(64, b, 512)
        mod = fb.workloads.LSTM(w_ih, w_hh, b_ih, b_hh, device=dev)
        xd = x.to(dev)
        fn = lambda: mod.forward_device(xd, args.lstm_mode)
    elif args.only == "normalize":
        from functs_b200 import jit as J, simpleops
        img = torch.rand(800, 1333, 3, device=dev)
        built = J.build(simpleops.normalize, (img, 0.45, 4.4))
        fn = lambda: built(img, 0.45, 4.4)
    elif args.only == "get_started":
        a, bb, n = W.make_get_started_inputs()
        fn = lambda: fb.workloads.get_started(a, bb.to(dev), n)
    else:
        maps = [m.to(dev) for m in W.make_yolo_inputs(b)]
        mod = fb.workloads.YOLOV3BBox(device=dev)
        fn = lambda: mod.forward_padded(maps)
    for _ in range(args.warmup + args.steps):
        fn()
    torch.cuda.synchronize()
    print(f"ran {args.only} batch {b}: {args.warmup + args.steps} calls")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--comm-priority", default="high", choices=["high", "normal"],
                    help="stream priority of the multi-GPU gather (N > 1)")
    ap.add_argument("--in-flight", type=int, default=3, choices=[1, 2, 3, 4],
                    help="batches in flight in the throughput measurement (one stream each; 1 = strictly one after the other; measured on one B200: 129 / 98 / 92 / 91 us per step for 1 / 2 / 3 / 4)")
    ap.add_argument("--rec-buffers", type=int, default=0, help="N > 1: record buffers in rotation (default 10: with four, a step now and then waited for the gather of the fourth step before it)")
    ap.add_argument("--gather-every", type=int, default=4,
                    help="N > 1: the records of this many consecutive steps travel in one gather")
    ap.add_argument("--gather", default="nccl", choices=["nccl", "one-sided"],
                    help="N > 1: NCCL send / receive pairs, or asynchronous peer copies into rank 0's buffers")
    ap.add_argument("--no-gather", action="store_true",
                    help="diagnostic (N > 1): write the detection records but skip the gather (the number is then not a result)")
    ap.add_argument("--no-graph", action="store_true", help="issue the throughput blocks call by call instead of replaying a CUDA graph")
    ap.add_argument("--no-extra", action="store_true", help="skip the cpu_baseline leg and the other workloads")
    ap.add_argument("--only", default=None, choices=["yolo", "ssd", "yolact", "lstm", "get_started", "normalize"],
                    help="run a few calls of one workload and exit (for profiler captures)")
    ap.add_argument("--batch", type=int, default=8, help="batch size for --only")
    ap.add_argument("--lstm-mode", type=int, default=0, choices=[0, 1, 2, 3],
                    help="--only lstm: 0 library default, 1 CUDA cores, 2 tcgen05 projection and recurrence, 3 tcgen05 projection")
    args = ap.parse_args()
    if args.only is not None:
        run_single_workload(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
