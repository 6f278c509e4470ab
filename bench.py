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


def cpu_oracle_rate(sample_images: int, steps: int, warmup: int):
    """TorchScript CPU oracle on `sample_images` images per step; returns (batches/s, ms per step, threads)."""
    import torch
    from oracle import workloads as W
    threads = os.cpu_count() or 1
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


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 8
    rate, ms, threads = cpu_oracle_rate(sample, max(args.steps, 1), max(args.warmup, 1))
    sample_txt = f"{sample} of the 64 images per step (seeded N(0,1) logits), TorchScript CPU oracle, rate scaled to 64-image batches"
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "YOLOv3-style decode + score>0.5 mask + top-1000 + class-wise NMS 0.45, 3 scales 13/26/52, batch 64",
                   "sample_images_per_step": sample},
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


def extra_workloads(torch, fb, W, hbm_peak):
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
                          "note": "0.5 MB working set (L2-resident); latency-bound"}
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
                  "algorithmic_gbs": by / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / hbm_peak}
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
                     "algorithmic_gbs": by / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / hbm_peak}
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
    out["lstm"] = {"T": 64, "B": 64, "H": 512, "latency_us": ms * 1e3, "batches_per_s": 1e3 / ms,
                   "kernels_per_call": lm.kernels_last_call,
                   "stage_us": {"input_projection_tcgen05": evs[0].elapsed_time(evs[1]) * 1e3,
                                "recurrence": evs[1].elapsed_time(evs[2]) * 1e3},
                   "algorithmic_tflops": 17.18e9 / (ms * 1e-3) / 1e12}
    return out


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
    rec = torch.empty(BATCH, topk, fdist.RECORD_WORDS, dtype=torch.int32, device=dev)
    rec_all = torch.empty(world * BATCH, topk, fdist.RECORD_WORDS, dtype=torch.int32, device=dev) if world > 1 else None
    # multi-GPU: the gather of step i runs on a second stream while step i + 1 computes (two record buffers)
    if world > 1:
        comm_stream = torch.cuda.Stream(dev, priority=-1 if args.comm_priority == "high" else 0)
        recs = [rec, torch.empty_like(rec)]
        rec_alls = [rec_all, torch.empty_like(rec_all)]
        packed_ev = [torch.cuda.Event(), torch.cuda.Event()]
        gathered_ev = [torch.cuda.Event(), torch.cuda.Event()]
        for e in gathered_ev:
            e.record()
    # per-step stage events, recorded inside the one-call entry point through its profiling hook
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    for row in ev:
        for e in row:
            e.record()  # materialises the CUDA event handle
    torch.cuda.synchronize()
    import ctypes
    ev_handles = [(ctypes.c_void_p * 4)(*[e.cuda_event for e in row]) for row in ev]

    def step(i, handles=None):
        if handles is not None:
            lib.functs_b200_set_stage_events(handles, 4)
        plan.run(sets[i % n_sets], 0.5, 0.45)   # memset + decode/mask/compact + binned top-k + NMS: 3 kernels
        if handles is not None:
            lib.functs_b200_set_stage_events(None, 0)
        if world > 1:
            j = i & 1
            main = torch.cuda.current_stream()
            main.wait_event(gathered_ev[j])     # the gather that used this buffer pair two steps ago is done
            fdist.pack_detections(plan.dets, plan.labels, plan.flat_ids, plan.counts, out=recs[j])   # 1 kernel
            packed_ev[j].record(main)
            with torch.cuda.stream(comm_stream):
                comm_stream.wait_event(packed_ev[j])
                fdist.gather_records(recs[j], out=rec_alls[j])
                gathered_ev[j].record(comm_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = launch_count()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record()
    for i in range(args.steps):
        step(i, ev_handles[i])
    if world > 1:
        torch.cuda.current_stream().wait_stream(comm_stream)   # the timed region ends when the last gather has landed
    t_end.record()
    barrier()
    launches = launch_count() - launches0
    total_ms = t_start.elapsed_time(t_end)
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
            r = fdist.gather_records(rec, out=rec_all)
            return r.cpu()
        return dets.cpu(), labels.cpu(), cnt.cpu()
    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    bytes_out = (rec_all.numel() * 4) if world > 1 else (plan.dets.numel() * 4 + plan.labels.numel() * 8 + plan.counts.numel() * 4)
    clocks = sampler.stop() if rank == 0 else None

    # ---- max over ranks ----
    stats = torch.tensor([total_ms, e2e_ms, decode_ms, select_ms, nms_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, decode_ms, select_ms, nms_ms = [float(v) for v in stats.tolist()]

    if rank == 0:
        ms_per_step = total_ms / args.steps
        alg_bytes = BATCH * IMG_BYTES                       # bytes the decode kernel must read per launch
        achieved = alg_bytes / (decode_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": world * 1e3 / ms_per_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "YOLOv3-style decode + score>0.5 mask + top-1000 + class-wise NMS 0.45, 3 scales 13/26/52, batch 64 per GPU",
                       "batch_per_gpu": BATCH, "l2": f"inputs 231.7 MB per step > 126 MB L2, {n_sets} input sets rotated",
                       "collective": "none" if world == 1 else "NCCL all-gather of the 2 MB detection records of every step, on a second stream while the next step computes"},
            "latency_us": ms_per_step * 1e3, "kernels_per_call": launches / args.steps,
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
            cpu_rate, cpu_ms, threads = cpu_oracle_rate(4, 3, 1)
            line["cpu_baseline"] = {"value": cpu_rate, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": "4 of the 64 images per step x 3 steps, TorchScript CPU oracle, rate scaled to 64-image batches"}
            del sets
            torch.cuda.empty_cache()
            try:
                line["workloads"] = extra_workloads(torch, fb, W, hbm_peak)
            except Exception as exc:  # the headline number must still be printed
                line["workloads"] = {"error": repr(exc)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
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
        fn = lambda: mod.forward_device(xd)
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
    ap.add_argument("--no-extra", action="store_true", help="skip the cpu_baseline leg and the other workloads")
    ap.add_argument("--only", default=None, choices=["yolo", "ssd", "yolact", "lstm", "get_started"],
                    help="run a few calls of one workload and exit (for profiler captures)")
    ap.add_argument("--batch", type=int, default=8, help="batch size for --only")
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
