#!/usr/bin/env python
"""Benchmark of the uint8 quantized fully-connected forward path (libltq, sm_100a).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload square_4096|skinny|mlp_mnist|mlp_block]
    python bench.py --impl reference ...      # the reference's own CPU code on the host cores

One JSON line on stdout (rank 0).  A step is one pass of the hot path over one batch: activation quantise
(fp32 -> uint8 + row sums, static calibrated qparams as the reference uses them) followed by the quantized GEMM with
its fused epilogue.  `value` has the inputs resident in HBM; `e2e` is the same work through the FullyConnected_q
mirror with pinned host buffers, host->device and device->host copies inside the timed region.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "light-tensor_b200", "python")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402

NOMINAL_INT8_TOPS = 4500.0  # B200 dense INT8, nominal
NOMINAL_HBM_GBS = 8000.0


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi during the timed region (SM clock, throttle reasons)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own FullyConnected_q::forward on the host cores
# ---------------------------------------------------------------------------------------------------------------------
def _cpu_inputs(workload, rows):
    """uint8 operands of the workload (quantized with numpy restating nothing: plain random bytes of the same shapes
    would time identically, but the real quantized tensors are used so the sample is the same work)."""
    import oracle
    from ltq import workloads
    if workload == "skinny":
        x, w = workloads.skinny(seed=4, M=min(rows, 16))
    else:
        x, w = workloads.square_4096(seed=3)
    x = x[:rows]
    qx = oracle.port.compute_qparams(*oracle.port.get_min_max(x))
    qw = oracle.port.compute_qparams(*oracle.port.get_min_max(w))
    return oracle.port.quantize_u8(x, qx), oracle.port.quantize_u8(w, qw), qx, qw, oracle.qp(0.05, 128)


def cpu_forward_seconds(workload, rows, repeats=1):
    """Seconds for one FullyConnected_q::forward over `rows` rows of the workload on one host thread (the path is
    single-threaded by construction).  Uses oracle/_ref (the unmodified reference) when it was built, else the C
    restatement."""
    import oracle
    xq, wq, qx, qw, qo = _cpu_inputs(workload, rows)
    M, K = xq.shape
    N = wq.shape[0]
    if oracle.ref is not None:
        _, secs = oracle.ref.fc_q_forward(xq, wq, M, N, K, qx, qw, qo, repeats=repeats)
        return secs, "reference", M, N, K
    os.environ["OMP_NUM_THREADS"] = "1"
    best = 1e30
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.port.quantized_matmul(xq, wq, M, N, K, [qx, qw, qo])
        best = min(best, time.perf_counter() - t0)
    return best, "port", M, N, K


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = args.workload
    # size the sample so that warmup + steps finish within a couple of minutes
    t_probe, kind, m0, N, K = cpu_forward_seconds(wl, 8)
    per_row = t_probe / m0
    budget = 150.0 / max(1, args.steps + args.warmup)
    full_rows = 16 if wl == "skinny" else 4096
    rows = int(max(1, min(full_rows, budget / per_row)))
    times = []
    for i in range(args.warmup + args.steps):
        t, kind, M, N, K = cpu_forward_seconds(wl, rows)
        if i >= args.warmup:
            times.append(t)
    sec = float(np.mean(times))
    tops = 2.0 * M * N * K / sec / 1e12
    line = {
        "impl": "reference", "metric": "int8_fc_tops", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": workload_name(wl), "sample_rows": M, "N": N, "K": K},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": 1, "kind": kind,
                         "sample": f"FullyConnected_q::forward on the first {M} of {full_rows} rows, 1 thread "
                                   f"(the path is single-threaded by construction), host has {os.cpu_count()} cores"},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_name(wl):
    return {
        "square_4096": "square_4096 (configs[2]): M=N=K=4096 uint8 x uint8 linear, activations quantized from fp32, "
                       "uint8 requantized output",
        "skinny": "skinny (configs[3]): M=16, K=4096, N=11008, fp32 output",
    }.get(wl, wl)


# ---------------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import ltq

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback (use --impl reference)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    ltq.lib()
    pk = peaks()

    wl = args.workload
    if wl == "skinny":
        M, K, N = args.m, 4096, 11008
        out_mode, out_dtype = ltq.OUT_F32, torch.float32
        sets = 6       # 6 x 45 MB of weights: every step streams weights that are not in L2
    else:
        M = K = N = 4096
        out_mode, out_dtype = ltq.OUT_U8, torch.uint8
        sets = 4       # 4 x (64 MB fp32 activations + 16 MB weights + outputs) = 448 MB > 126 MB L2
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    xs = [torch.randn((M, K), generator=g, device=dev) for _ in range(sets)]
    w32 = [torch.randn((N, K), generator=g, device=dev) * 0.02 for _ in range(sets)]
    layers, qps_x = [], []
    for i in range(sets):
        qw = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(w32[i])))
        wq = ltq.Quantize(w32[i], qw)
        qx = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(xs[i])))
        h = ltq.LayerHandle(local, K, N)
        h.set_weights(wq, None)
        # output qparams calibrated from the fp32 product of a row sample (static, as the reference calibrates)
        ref = xs[i][:256] @ w32[i].t()
        qo = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(ref)))
        h.set_qparams(qx, qw, qo)
        layers.append(h)
        qps_x.append(qx)
    del w32
    xq = [torch.empty((M, K), dtype=torch.uint8, device=dev) for _ in range(sets)]
    asum = [torch.empty(M, dtype=torch.int32, device=dev) for _ in range(sets)]
    outs = [torch.empty((M, N), dtype=out_dtype, device=dev) for _ in range(sets)]

    def step(i):
        s = i % sets
        ltq.quantize_rows(xs[s], qp=qps_x[s], q=xq[s], asum=asum[s])
        layers[s].forward(xq[s], out_mode, 0, asum=asum[s], out=outs[s])

    def gemm_only(i):
        s = i % sets
        layers[s].forward(xq[s], out_mode, 0, asum=asum[s], out=outs[s])

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, warmup, graph=True):
        """ms per step over EXACTLY `steps` steps, CUDA events on the launching stream, max over ranks.  The steps are
        captured once into a CUDA graph (the kernels run for tens of microseconds; launching them one by one from
        Python would time the interpreter) and the graph is replayed once untimed before the timed replay."""
        for i in range(warmup):
            fn(i)
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if graph:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for i in range(steps):
                    fn(warmup + i)
            gr.replay()
            sync_all()
            e0.record()
            gr.replay()
            e1.record()
        else:
            e0.record()
            for i in range(steps):
                fn(warmup + i)
            e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    sampler = ClockSampler(local)
    launches0 = ltq.kernel_launches()
    if rank == 0:
        sampler.start()
    ms_step = timed(step, args.steps, args.warmup, graph=not args.no_graph)
    # kernels per timed region: warm-up steps, the capture pass and (with a graph) two replays all launch the same list
    launches = (ltq.kernel_launches() - launches0) // (args.steps + args.warmup) * args.steps
    ms_gemm = timed(gemm_only, args.steps, max(3, args.warmup), graph=not args.no_graph)
    clocks = sampler.stop() if rank == 0 else None
    for h in layers:
        h.check()

    ops = 2.0 * M * N * K
    tops = ops / (ms_step * 1e-3) / 1e12 * world
    gemm_tops = ops / (ms_gemm * 1e-3) / 1e12

    # ---- end to end through the FullyConnected_q mirror with host buffers -----------------------------------------
    fc = ltq.FullyConnected_q(K, N, False)
    fc.init()
    fc.weight_ptr_ = layers[0]._keep[0].view(1, 1, N, K)  # device weights already quantized above
    fc._handle = layers[0]
    fc.set_output(out_mode)
    host_x = [torch.randn((M, K)).pin_memory() for _ in range(2)]
    host_out = torch.empty((M, N), dtype=out_dtype).pin_memory()
    dev_x = torch.empty((M, K), device=dev)

    def e2e_step(i):
        dev_x.copy_(host_x[i % 2], non_blocking=True)
        q, s = ltq.quantize_rows(dev_x, qp=qps_x[0], q=xq[0], asum=asum[0])
        y = fc.forward(q.view(1, M, K), asum=s)
        host_out.copy_(y.view(M, N), non_blocking=True)

    if args.no_e2e:
        ms_e2e = float("nan")
    else:
        ms_e2e = timed(e2e_step, max(3, args.steps // 2), 3, graph=False)
    e2e_tops = ops / (ms_e2e * 1e-3) / 1e12 * world
    fc._handle = None

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    esize = 4 if out_mode == ltq.OUT_F32 else 1
    if wl == "skinny":
        alg_bytes = N * K + M * K + esize * M * N + 4 * N + 4 * M  # weights + acts + out + wsum + asum
        achieved = alg_bytes / (ms_gemm * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "traffic": None, "kernel": "gemv_kernel",
                "peak_source": f"{pk['source']} HBM copy", "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS}
    else:
        int8_peak = 2.0 * pk["bf16_sustained"]  # no INT8 figure is measured on this pool: 2 x measured bf16 (sustained)
        roof = {"bound": "tensor", "achieved": gemm_tops, "peak": int8_peak, "unit": "TOP/s",
                "frac": gemm_tops / int8_peak, "traffic": None, "kernel": "gemm_tc_kernel<256,u8>",
                "peak_source": f"2 x {pk['source']} bf16 sustained ({pk['bf16_sustained']} TFLOP/s); burst would be "
                               f"{2 * pk['bf16']}", "frac_of_nominal_4500": gemm_tops / NOMINAL_INT8_TOPS}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        rows = 16 if wl == "skinny" else 512
        secs, kind, m, n, k = cpu_forward_seconds(wl, rows)
        cpu = {"value": 2.0 * m * n * k / secs / 1e12, "unit": "TOPS", "cores": 1, "kind": kind,
               "seconds": secs, "sample": f"FullyConnected_q::forward on {m} rows of the workload (N={n}, K={k}), "
               f"1 thread of {os.cpu_count()} host cores; the reference path is single-threaded by construction"}

    line = {
        "metric": "int8_fc_tops", "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": workload_name(wl), "M_per_gpu": M, "N": N, "K": K, "sharding": "rows (M) per GPU, "
                   "weights replicated, no collective" if world > 1 else "single GPU",
                   "l2": f"rotating {sets} distinct input/weight/output sets, larger than L2 in total",
                   "step": "quantize_rows (fp32->u8 + row sums) + quantized GEMM with fused epilogue",
                   "timing": "CUDA events around one replay of a CUDA graph holding exactly `steps` steps"
                   if not args.no_graph else "CUDA events around `steps` eager launches"},
        "gemm_only": {"ms": ms_gemm, "tops": gemm_tops},
        "roofline": roof, "cpu_baseline": cpu,
        "e2e": {"value": e2e_tops, "unit": "TOPS", "ms_per_step": ms_e2e, "h2d_bytes_per_step": M * K * 4,
                "d2h_bytes_per_step": M * N * esize},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ltq", choices=["ltq", "reference"])
    ap.add_argument("--workload", default="square_4096", choices=["square_4096", "skinny"])
    ap.add_argument("--m", type=int, default=16, help="rows for the skinny workload (1, 4 or 16)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps one by one instead of from a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
