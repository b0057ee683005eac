#!/usr/bin/env python
"""Benchmark of the uint8 quantized fully-connected forward path (libltq, sm_100a).

    python bench.py [--gpus N] [--steps K] [--warmup W]          # everything the metric names, one JSON line
    python bench.py --workload square_4096|skinny|mlp_block|mlp_mnist|conv|helpers [--shard rows|cols|cols_fused] ...
    python bench.py --impl reference ...                          # the reference's own CPU code on the host cores

One JSON line on stdout (rank 0).  The headline (`value`, `ms_per_step`, `roofline`, `e2e`, `cpu_baseline`) is the
4096^3 quantized linear: a step is one pass of the hot path over one batch, activation quantise (fp32 -> uint8 + row
sums, static calibrated qparams as the reference uses them) followed by the quantized GEMM with its fused epilogue.
`value` has the inputs resident in HBM; `e2e` is the same work through the FullyConnected_q mirror with pinned host
buffers, host->device and device->host copies inside the timed region.  The default run also measures the other parts
of the metric and reports them as sections of the same line: `skinny` (M = 1 / 4 / 16 weight streaming, HBM GB/s),
`helpers` (GetMinMax / Quantize / Dequantize and the dynamic activation step, HBM GB/s), `mlp_mnist` (784-512-512-10,
samples/s, one batch stream and four), `conv2d_q` (the convolution layer), `mlp_block_rows` (8192-32768-8192 over 65536 tokens, row-sharded over the
ranks, strong scaling) and, with more than one rank, `mlp_block_cols` / `mlp_block_cols_fused` (column-sharded with an
NCCL all-gather, and with the exchange fused into the GEMM epilogue).
"""
import argparse
import json
import os
import re
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


def ncu_traffic(profile_md, kernel_launched):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, read from the ncu
    summary committed under profiles/.  Returns (bytes or None, note): None when the summary is missing or was captured
    on another kernel than the one this run launched, so that the figure cannot outlive a kernel change unnoticed."""
    path = os.path.join(ROOT, "profiles", profile_md)
    if not os.path.exists(path):
        return None, f"profiles/{profile_md} not found"
    text = open(path).read()
    title = text.splitlines()[0]
    unit = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    total = 0.0
    for key in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
        m = re.search(r"`" + re.escape(key) + r"`\s*\|\s*([0-9.,]+)\s*([A-Za-z]+)", text)
        if not m:
            return None, f"profiles/{profile_md} has no {key}"
        total += float(m.group(1).replace(",", "")) * unit.get(m.group(2), 1.0)
    base = kernel_launched.split("<")[0]
    if base not in title:
        return None, f"profiles/{profile_md} covers '{title.lstrip('# ')}', this run launched {kernel_launched}"
    return total, f"profiles/{profile_md}"


class ClockSampler:
    """Samples nvidia-smi during the timed region (SM clock, throttle reasons)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
        self.rows = []
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
        self.proc = None
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
    wl = "skinny" if args.workload == "skinny" else "square_4096"
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
def bind_to_gpu_numa_node(local_rank):
    """Keeps this rank's host threads (and so the first touch of its pinned buffers) on the NUMA node its GPU hangs off.
    Returns a short description for the JSON line; does nothing when the node cannot be determined."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = torch.cuda.get_device_properties(local_rank).pci_domain_id
        dev = torch.cuda.get_device_properties(local_rank).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        node = int(open(path).read().strip())
        if node < 0:
            return "numa node unknown (single node or not exposed)"
        cpus = open(f"/sys/devices/system/node/node{node}/cpulist").read().strip()
        ids = set()
        for part in cpus.split(","):
            a, _, b = part.partition("-")
            ids.update(range(int(a), int(b or a) + 1))
        ids &= os.sched_getaffinity(0)
        if ids:
            os.sched_setaffinity(0, ids)
        return f"node {node}, cpus {cpus}"
    except Exception as exc:  # noqa: BLE001 - best effort; the bench runs without it
        return f"not bound ({type(exc).__name__})"


class Harness:
    """Device set-up, barriers, CUDA-graph timing and clock sampling shared by the workloads."""

    def __init__(self, args):
        import torch
        self.torch = torch
        self.args = args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback (use --impl reference)")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.numa = bind_to_gpu_numa_node(self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.sampler = ClockSampler(self.local)

    def sync_all(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, ms):
        if self.dist is not None:
            t = self.torch.tensor([ms], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def timed(self, fn, steps, warmup, graph=True, sample_clocks=False, join=None, capture_stream=None, sustain_s=0.0,
              local_only=False):
        """ms per step over EXACTLY `steps` steps, CUDA events on the launching stream, max over ranks.  The steps are
        captured once into a CUDA graph (the kernels run for tens of microseconds; launching them one by one from
        Python would time the interpreter) and the graph is replayed once untimed before the timed replay.  With
        `sample_clocks` nvidia-smi runs through the warm-up, the timed replay and ~0.4 s of further replays of the same
        graph (the timed region alone is too short to catch more than a sample or two).  With `sustain_s` the same graph
        is then replayed back to back for at least that long, timed with events as one region, and
        `self.sustained` = {ms_per_step, seconds, sm_mhz} describes it.  `local_only`: no barrier / reduction (a
        section that only rank 0 runs)."""
        torch = self.torch
        sync = torch.cuda.synchronize if local_only else self.sync_all
        if sample_clocks and self.rank == 0:
            self.sampler.start()
        for i in range(warmup):
            fn(i)
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        gr = None
        if graph:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=capture_stream):
                for i in range(steps):
                    fn(warmup + i)
            gr.replay()
            sync()
            e0.record()
            gr.replay()
            e1.record()
        else:
            e0.record()
            for i in range(steps):
                fn(warmup + i)
            if join is not None:
                join()  # the timing stream waits for work the steps put on other streams
            e1.record()
        sync()
        ms = e0.elapsed_time(e1)
        if sample_clocks:
            t_end = time.time() + 0.4
            while time.time() < t_end:
                if gr is not None:
                    gr.replay()
                else:
                    fn(0)
                torch.cuda.synchronize()
            self.clocks = self.sampler.stop() if self.rank == 0 else None
        if sustain_s > 0 and gr is not None:
            # back-to-back replays without host synchronisation in between: the GPU stays under load for the whole region
            reps = max(8, int(sustain_s / max(ms * 1e-3, 1e-6)) + 1)
            if self.rank == 0:
                self.sampler.start()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(reps):
                gr.replay()
            s1.record()
            torch.cuda.synchronize()
            clk = self.sampler.stop() if self.rank == 0 else None
            tot = s0.elapsed_time(s1)
            self.sustained = {"ms_per_step": tot / (reps * steps), "seconds": tot * 1e-3,
                              "sm_mhz_median": clk["sm_mhz"] if clk else None,
                              "reasons": clk["reasons"] if clk else None}
        if not local_only:
            ms = self.max_over_ranks(ms)
        return ms / steps

    def finish(self, line):
        if self.rank == 0:
            print(json.dumps(line))
        if self.dist is not None:
            self.dist.destroy_process_group()


def base_line(h, args, value, unit, ms_step, scaling, config, **extra):
    line = {"metric": "int8_fc_tops", "value": value, "unit": unit, "n_gpus": h.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "u8", "data": "synthetic", "config": config}
    line.update(extra)
    return line


def h2d_ceiling_gbs(h, nbytes, d2h_bytes=0, reps=6):
    """Host->device rate (GB/s, this rank) of copies of `nbytes` out of pinned memory, every rank starting together
    after a barrier, so that with N ranks the figure is the rate one rank keeps while the other N - 1 copy too.  Two
    ways of issuing them, the better reading counts (which one wins differs from box to box): one copy at a time on
    the current stream, and `reps` copies back to back on a stream of their own.  With `d2h_bytes` another stream
    copies that many bytes device->host at the same time, once per host->device copy: the traffic pattern of the
    pipelined end-to-end step without any kernel in it."""
    torch = h.torch
    src = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    dst = torch.empty(nbytes, dtype=torch.uint8, device=h.dev)
    up = torch.cuda.Stream()
    if d2h_bytes:
        back_src = torch.empty(d2h_bytes, dtype=torch.uint8, device=h.dev)
        back_dst = torch.empty(d2h_bytes, dtype=torch.uint8).pin_memory()
        down = torch.cuda.Stream()
    best = 0.0
    awake = torch.cuda.Stream() if hasattr(torch.cuda, "_sleep") else None
    for trial in range(5):                                   # the first trial also warms the copy engines up
        single = trial % 2 == 1
        n = 1 if single else reps
        h.sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st = torch.cuda.current_stream() if single else up
        if awake is not None:
            # one CTA spinning for about as long as the copies take: an otherwise idle GPU gave copy rates well below
            # the ones the end-to-end step reaches with kernels running beside its copies
            with torch.cuda.stream(awake):
                torch.cuda._sleep(int(n * nbytes / 20e9 * 1.5e9))
        with torch.cuda.stream(st):
            e0.record(st)
            for _ in range(n):
                dst.copy_(src, non_blocking=True)
            e1.record(st)
        if d2h_bytes:
            with torch.cuda.stream(down):
                for _ in range(n):
                    back_dst.copy_(back_src, non_blocking=True)
        torch.cuda.synchronize()
        if trial:
            best = max(best, n * nbytes / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    return best


# ---- the 4096^3 linear and the skinny linear ---------------------------------------------------------------------------
def measure_linear(h, args, wl, m_rows=16, with_e2e=True, steps=None, sustain_s=0.0, next_hint=True):
    """One quantized linear per step.  Returns a dict of measurements (times are max over ranks)."""
    import ltq
    torch, dev = h.torch, h.dev
    steps = steps or args.steps
    if wl == "skinny":
        M, K, N = m_rows, 4096, 11008
        out_mode, out_dtype = ltq.OUT_F32, torch.float32
        sets = 6       # 6 x 45 MB of weights: every step streams weights that are not in L2
    else:
        M = K = N = 4096
        out_mode, out_dtype = ltq.OUT_U8, torch.uint8
        sets = 4       # 4 x (64 MB fp32 activations + 16 MB weights + outputs) = 448 MB > 126 MB L2
    g = torch.Generator(device=dev).manual_seed(1234 + h.rank)
    xs = [torch.randn((M, K), generator=g, device=dev) for _ in range(sets)]
    w32 = [torch.randn((N, K), generator=g, device=dev) * 0.02 for _ in range(sets)]
    layers, qps_x, qps_w, qps_o, wqs = [], [], [], [], []
    for i in range(sets):
        qw = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(w32[i])))
        wq = ltq.Quantize(w32[i], qw)
        qx = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(xs[i])))
        lh = ltq.LayerHandle(h.local, K, N)
        lh.set_weights(wq, None)
        # output qparams calibrated from the fp32 product of a row sample (static, as the reference calibrates)
        ref = xs[i][:256] @ w32[i].t()
        qo = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(ref)))
        lh.set_qparams(qx, qw, qo)
        layers.append(lh)
        qps_x.append(qx)
        qps_w.append(qw)
        qps_o.append(qo)
        wqs.append(wq)
    del w32
    if wl == "skinny" and next_hint:
        # the steps visit the layers in a fixed order, like the layers of a network: each one names its successor, so
        # that its weight-streaming kernel asks the start of the next weights into L2 (ltq_layer_set_next)
        for i in range(sets):
            layers[i].set_next(layers[(i + 1) % sets])
    xq = [torch.empty((M, K), dtype=torch.uint8, device=dev) for _ in range(sets)]
    asum = [torch.empty(M, dtype=torch.int32, device=dev) for _ in range(sets)]
    outs = [torch.empty((M, N), dtype=out_dtype, device=dev) for _ in range(sets)]

    def step_serial(i):
        s = i % sets
        ltq.quantize_rows(xs[s], qp=qps_x[s], q=xq[s], asum=asum[s])
        layers[s].forward(xq[s], out_mode, 0, asum=asum[s], out=outs[s])

    # Software-pipelined step: while the GEMM of batch i runs (tensor-bound; for the skinny workload, weight streaming),
    # a second stream quantises batch i+1 on the SM resources the persistent GEMM CTAs leave free.  Every step still launches exactly one
    # quantize_rows and one GEMM; batch i's quantised activations come from the step before (or, for the first step of
    # a sequence, are produced up front).
    side = torch.cuda.Stream(priority=0)             # lowest priority: fills what the GEMM leaves free
    state = {"ready": None}

    def step_overlap(i):
        s, nxt = i % sets, (i + 1) % sets
        main = torch.cuda.current_stream()
        if state["ready"] != i:
            ltq.quantize_rows(xs[s], qp=qps_x[s], q=xq[s], asum=asum[s])
        fork = torch.cuda.Event()
        fork.record(main)                            # batch i+1's buffers are free once everything before this is done
        layers[s].forward(xq[s], out_mode, 0, asum=asum[s], out=outs[s])   # enqueued first: its CTAs take the SMs first
        side.wait_event(fork)
        with torch.cuda.stream(side):
            ltq.quantize_rows(xs[nxt], qp=qps_x[nxt], q=xq[nxt], asum=asum[nxt])
        main.wait_stream(side)                       # join
        state["ready"] = i + 1

    step = step_serial if args.no_overlap else step_overlap

    def gemm_only(i):
        s = i % sets
        layers[s].forward(xq[s], out_mode, 0, asum=asum[s], out=outs[s])

    launches0 = ltq.kernel_launches()
    ms_step = h.timed(step, steps, args.warmup, graph=not args.no_graph, sample_clocks=True,
                      capture_stream=torch.cuda.Stream(priority=-1))
    # kernels per timed region: warm-up steps and the capture pass each launch the same list; replays re-run it
    launches = (ltq.kernel_launches() - launches0) // (steps + args.warmup) * steps
    clocks = getattr(h, "clocks", None)
    h.sustained = None
    ms_gemm = h.timed(gemm_only, steps, max(3, args.warmup), graph=not args.no_graph, sustain_s=sustain_s)
    kernel = ltq.last_kernel()
    sustained = h.sustained
    ms_quant = h.timed(lambda i: ltq.quantize_rows(xs[i % sets], qp=qps_x[i % sets], q=xq[i % sets], asum=asum[i % sets]),
                       steps, 3, graph=not args.no_graph)
    for lh in layers:
        lh.check()
        lh.set_next(None)

    res = dict(M=M, N=N, K=K, sets=sets, ms_step=ms_step, ms_gemm=ms_gemm, ms_quant=ms_quant, launches=int(launches),
               kernel=kernel, clocks=clocks, sustained=sustained, step_overlapped=step is step_overlap,
               esize=4 if out_mode == ltq.OUT_F32 else 1, e2e=None)

    # ---- end to end through the FullyConnected_q mirror with host buffers -----------------------------------------
    if with_e2e and not args.no_e2e:
        # The layer is built the way a user of the reference builds it: init(), quantized weights written through
        # get_all_weights() on the host, qparams through the setters, then to("cuda").
        fc = ltq.FullyConnected_q(K, N, False)
        fc.init()
        fc.get_all_weights()[0].copy_(wqs[0].cpu().view(1, 1, N, K))
        fc.set_qparams_in(qps_x[0])
        fc.set_qparams_out(qps_o[0])
        fc.set_qparams_params([qps_w[0]], 1)
        fc.to("cuda", h.local)
        fc.set_output(out_mode)
        ceiling = h2d_ceiling_gbs(h, M * K * 4)
        ceiling_both = h2d_ceiling_gbs(h, M * K * 4, d2h_bytes=M * N * res["esize"])
        # Three streams (upload, compute, download) over two buffer sets: the upload of step i+1 and the download of
        # step i-1 run while step i computes, so a step costs what the slower PCIe direction costs.
        host_x = [torch.randn((M, K)).pin_memory() for _ in range(2)]
        host_out = [torch.empty((M, N), dtype=out_dtype).pin_memory() for _ in range(2)]
        dev_x = [torch.empty((M, K), device=dev) for _ in range(2)]
        dev_q = [torch.empty((M, K), dtype=torch.uint8, device=dev) for _ in range(2)]
        dev_s = [torch.empty(M, dtype=torch.int32, device=dev) for _ in range(2)]
        s_up, s_run, s_down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        ev_up = [torch.cuda.Event() for _ in range(2)]      # upload of set b finished
        ev_run = [torch.cuda.Event() for _ in range(2)]     # compute on set b finished (dev_x[b] free, y[b] ready)
        ev_down = [torch.cuda.Event() for _ in range(2)]    # download of set b finished
        y_keep = [None, None]

        def e2e_step(i):
            b = i % 2
            with torch.cuda.stream(s_up):
                s_up.wait_event(ev_run[b])                  # quantize of the step two back has read dev_x[b]
                dev_x[b].copy_(host_x[b], non_blocking=True)
                ev_up[b].record(s_up)
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_up[b])
                s_run.wait_event(ev_down[b])                # the download two steps back has read y_keep[b]
                q, sm = ltq.quantize_rows(dev_x[b], qp=qps_x[0], q=dev_q[b], asum=dev_s[b])
                y_keep[b] = fc.forward(q.view(1, M, K), asum=sm)
                ev_run[b].record(s_run)
            with torch.cuda.stream(s_down):
                s_down.wait_event(ev_run[b])
                y_keep[b].record_stream(s_down)
                host_out[b].copy_(y_keep[b].view(M, N), non_blocking=True)
                ev_down[b].record(s_down)

        def e2e_join():
            for st in (s_up, s_run, s_down):
                torch.cuda.current_stream().wait_stream(st)

        # The host side of the copies (memory, PCIe switch) is shared with the machine's other tenants and its rate moves
        # on a 100 ms scale: five timed regions of the same K steps, the fastest one is reported and all five are
        # listed; the copy ceilings are taken again after the regions and the larger reading of each is kept.
        k_e2e = max(8, steps // 2)
        regions = [h.timed(e2e_step, k_e2e, 4 if r == 0 else 2, graph=False, join=e2e_join) for r in range(5)]
        ms_e2e = min(regions)
        ceiling = max(ceiling, h2d_ceiling_gbs(h, M * K * 4))
        ceiling_both = max(ceiling_both, h2d_ceiling_gbs(h, M * K * 4, d2h_bytes=M * N * res["esize"]))
        h2d, d2h = M * K * 4, M * N * res["esize"]
        res["e2e"] = {"ms_per_step": ms_e2e, "steps": k_e2e, "ms_per_step_of_each_region": regions,
                      "timing": f"fastest of 5 regions of {k_e2e} steps each (CUDA events, max over ranks per region)",
                      "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                      "pcie_gbs": {"h2d": h2d / (ms_e2e * 1e-3) / 1e9, "d2h": d2h / (ms_e2e * 1e-3) / 1e9},
                      "h2d_ceiling_gbs": max(ceiling, ceiling_both),
                      "frac_of_h2d_ceiling": h2d / (ms_e2e * 1e-3) / 1e9 / max(ceiling, ceiling_both),
                      "h2d_copy_rates_gbs": {"alone": ceiling, "with_d2h_running": ceiling_both},
                      "ceiling_method": "plain copies of the step's upload out of pinned memory, all ranks at once after "
                                        "a barrier, singly and 6 back to back, one CTA kept spinning so that the GPU is "
                                        "not idle, before and after the timed regions; `alone` = nothing else running, "
                                        "`with_d2h_running` = the step's download bytes copied on another stream at the "
                                        "same time; the ceiling is the best reading of all",
                      "bound": "host->device copy of the fp32 activations (PCIe); compute is "
                               f"{ms_step / ms_e2e * 100:.1f} % of the step" +
                               ("; with several ranks the copy rates themselves fall (the ranks share host memory and "
                                "PCIe roots): compare h2d_copy_rates_gbs with the 1-GPU line" if h.world > 1 else ""),
                      "host_numa_binding": h.numa}
        if res["e2e"]["frac_of_h2d_ceiling"] > 1.0:
            res["e2e"]["ceiling_note"] = ("the plain-copy readings came out below the rate the step itself kept: the host "
                                          "side (shared with other tenants) was disturbed while they ran")
    return res


def skinny_roofline(r, pk, traffic, traffic_note):
    M, N, K, esize = r["M"], r["N"], r["K"], r["esize"]
    alg_bytes = N * K + M * K + esize * M * N + 8 * N + 4 * M  # weights + acts + out + (wsum, bias) + asum
    achieved = alg_bytes / (r["ms_gemm"] * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
            "traffic": traffic, "traffic_source": traffic_note, "kernel": r["kernel"], "algorithmic_bytes": alg_bytes,
            "ms": r["ms_gemm"], "peak_source": f"{pk['source']} HBM copy",
            "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS}


def run_linear(args, h=None, sections=False):
    """square_4096 (default) and skinny: one quantized linear per step.  With `sections` (the default run) the other
    parts of the metric are measured too and attached to the same line."""
    import ltq
    h = h or Harness(args)
    world = h.world
    pk = peaks()
    wl = args.workload if args.workload in ("square_4096", "skinny") else "square_4096"
    r = measure_linear(h, args, wl, m_rows=args.m, sustain_s=1.2 if wl == "square_4096" else 0.0)
    M, N, K = r["M"], r["N"], r["K"]
    ops = 2.0 * M * N * K
    tops = ops / (r["ms_step"] * 1e-3) / 1e12 * world
    gemm_tops = ops / (r["ms_gemm"] * 1e-3) / 1e12

    e2e = None
    if r["e2e"]:
        e2e = dict(r["e2e"])
        e2e.update(value=ops / (e2e["ms_per_step"] * 1e-3) / 1e12 * world, unit="TOPS")

    if wl == "skinny":
        traffic, note = ncu_traffic("gemv_kernel_skinny_m16.md", r["kernel"])
        roof = skinny_roofline(r, pk, traffic, note)
    else:
        traffic, note = ncu_traffic("gemm_tc_pair_kernel_square4096.md", r["kernel"])
        # The kernel is timed in isolation (a graph of `steps` launches, ~1 ms): the denominator is the burst figure.
        # No INT8 GEMM is measured on this pool, so the proxy is 2 x the measured bf16 burst rate.
        int8_peak = 2.0 * pk["bf16"]
        roof = {"bound": "tensor", "achieved": gemm_tops, "peak": int8_peak, "unit": "TOP/s", "frac": gemm_tops / int8_peak,
                "traffic": traffic, "traffic_source": note, "kernel": r["kernel"], "algorithmic_ops": ops, "ms": r["ms_gemm"],
                "peak_source": f"2 x {pk['source']} bf16 burst ({pk['bf16']} TFLOP/s), the rate for a kernel timed alone",
                "frac_of_nominal_4500": gemm_tops / NOMINAL_INT8_TOPS}
        if r["sustained"]:
            s = r["sustained"]
            s_tops = ops / (s["ms_per_step"] * 1e-3) / 1e12
            roof["sustained"] = {"tops": s_tops, "ms": s["ms_per_step"], "seconds": s["seconds"],
                                 "sm_mhz_median": s["sm_mhz_median"], "reasons": s["reasons"],
                                 "frac_of_2x_bf16_sustained": s_tops / (2.0 * pk["bf16_sustained"]),
                                 "frac_of_nominal_4500": s_tops / NOMINAL_INT8_TOPS,
                                 "us_x_mhz": (s["ms_per_step"] * 1e3 * s["sm_mhz_median"]) if s["sm_mhz_median"] else None,
                                 "note": "the same graph of GEMM launches replayed back to back for `seconds`"}

    cpu = None
    if h.rank == 0 and world == 1 and not args.no_cpu_baseline:
        rows = 16 if wl == "skinny" else 512
        secs, kind, m, n, k = cpu_forward_seconds(wl, rows)
        cpu = {"value": 2.0 * m * n * k / secs / 1e12, "unit": "TOPS", "cores": 1, "kind": kind,
               "seconds": secs, "sample": f"FullyConnected_q::forward on {m} rows of the workload (N={n}, K={k}), "
               f"1 thread of {os.cpu_count()} host cores; the reference path is single-threaded by construction"}

    cfg = {"workload": workload_name(wl), "M_per_gpu": M, "N": N, "K": K,
           "sharding": "rows (M) per GPU, weights replicated, no collective" if world > 1 else "single GPU",
           "l2": f"rotating {r['sets']} distinct input/weight/output sets, larger than L2 in total",
           "step": "quantize_rows (fp32->u8 + row sums) + quantized GEMM with fused epilogue" +
                   ("; batch i+1 is quantised on a second stream while batch i's GEMM runs" if r["step_overlapped"] else ""),
           "timing": "CUDA events around one replay of a CUDA graph holding exactly `steps` steps"
           if not args.no_graph else "CUDA events around `steps` eager launches"}
    quant_bytes = 5.0 * M * K + 4.0 * M  # fp32 in, uint8 out, one int32 row sum per row
    extra = {}
    if sections:
        extra = run_sections(h, args, pk)
    h.finish(base_line(h, args, tops, "TOPS", r["ms_step"], "weak", cfg,
                       gemm_only={"ms": r["ms_gemm"], "tops": gemm_tops},
                       quantize_only={"ms": r["ms_quant"], "gbs": quant_bytes / (r["ms_quant"] * 1e-3) / 1e9,
                                      "frac_of_hbm_peak": quant_bytes / (r["ms_quant"] * 1e-3) / 1e9 / pk["hbm_gbs"]},
                       roofline=roof, cpu_baseline=cpu, e2e=e2e, gpu_launches=r["launches"], clocks=r["clocks"], **extra))


def run_sections(h, args, pk, only=None):
    """The parts of the metric beside the headline: skinny M = 1 / 4 / 16 (HBM GB/s), the MNIST-shaped MLP (samples/s)
    and the 8192-32768-8192 block sharded over the ranks.  Each section is timed like the headline (CUDA graph, events,
    max over ranks); a section that fails reports its error instead of taking the line down."""
    out = {}

    def guarded(name, fn):
        try:
            out[name] = fn()
        except Exception as exc:  # noqa: BLE001
            out[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        h.torch.cuda.synchronize()
        import gc
        gc.collect()
        h.torch.cuda.empty_cache()

    def skinny():
        res = {"config": "configs[3]: K=4096, N=11008, fp32 out, 6 rotating 45 MB weight sets (every launch streams its "
                         "weights from HBM), visited in a fixed order with each layer naming the next (ltq_layer_set_next); "
                         "us = weight-streaming kernel alone, step_us = quantize_rows + kernel, per GPU; "
                         "us_without_next_hint = the kernel alone with no layer naming its successor; "
                         "graphs of at least 60 launches"}
        traffic, note = None, None
        for m in (1, 4, 16):
            r = measure_linear(h, args, "skinny", m_rows=m, with_e2e=False, steps=max(args.steps, 60))
            if traffic is None:
                traffic, note = ncu_traffic("gemv_kernel_skinny_m16.md", r["kernel"])
            roof = skinny_roofline(r, pk, traffic, note)
            res[f"m{m}"] = {"us": r["ms_gemm"] * 1e3, "gbs": roof["achieved"], "frac_of_measured": roof["frac"],
                            "frac_of_nominal": roof["frac_of_nominal_8TBs"], "step_us": r["ms_step"] * 1e3,
                            "algorithmic_bytes": roof["algorithmic_bytes"], "kernel": r["kernel"]}
            if m == 16:
                r0 = measure_linear(h, args, "skinny", m_rows=m, with_e2e=False, steps=max(args.steps, 60), next_hint=False)
                res[f"m{m}"]["us_without_next_hint"] = r0["ms_gemm"] * 1e3
        res["traffic"] = traffic
        res["traffic_source"] = note
        return res

    def mnist():
        r = measure_mlp_mnist(h, args)
        return {"config": "configs[0]: 784-512-512-10, batch 64, independent replicas (one batch stream per GPU)",
                "us_per_batch": r["ms_step"] * 1e3, "samples_per_s": 64 * h.world / (r["ms_step"] * 1e-3),
                "gpu_launches_per_batch": r["launches_per_step"], "kernels": r["kernels"],
                "path": "fused chain: Quantize + 3 layers in one launch (ltq_mlp_forward)",
                "layer_by_layer": {"us_per_batch": r["ms_layerwise"] * 1e3, "gpu_launches_per_batch": r["launches_layerwise"],
                                   "kernels": r["kernels_layerwise"]},
                "fused_output_equals_layer_by_layer": r["fused_equals_layerwise"],
                "batch_streams": dict(r["batch_streams"],
                                      samples_per_s=64 * h.world / (r["batch_streams"]["us_per_batch"] * 1e-6),
                                      what="the same chain with four independent batch streams in flight per GPU "
                                           "(four CUDA streams, own buffers each): throughput, not latency")}

    def block(shard):
        def run():
            steps = max(2, min(args.steps, 4))
            r = measure_mlp_block(h, args, shard, 65536, 8192, steps=steps, warmup=3)
            d = {"config": f"configs[4]: 8192->32768->8192, 65536 tokens in total, sharding {shard}; strong scaling",
                 "ms": r["ms_step"], "tops": r["tops"], "samples_per_s": 65536 / (r["ms_step"] * 1e-3),
                 "kernel": r["kernel"], "timing": r["timing"], "clocks": r["clocks"], "steps": steps}
            if shard == "rows" and h.world > 1:
                # the same 65536 tokens on rank 0 alone, in the same run, for the speed-up
                h.sync_all()
                n1 = measure_mlp_block(h, args, "rows", 65536, 8192, steps=2, warmup=2, alone=True) if h.rank == 0 else None
                h.sync_all()
                if n1:
                    d["n1_ms_same_run"] = n1["ms_step"]
                    d["speedup_vs_n1"] = n1["ms_step"] / r["ms_step"]
            if shard != "rows":
                d["nvlink_egress_bytes_per_gpu_per_step"] = r["egress_bytes"]
            if shard == "cols_multicast":
                d["multicast_in_use"] = r["multicast"]
            return d
        return run

    def conv():
        r = measure_conv(h, args)
        return {"config": conv_workload_name(r) + " (Conv2d_q, the next layer type on the path; per GPU)",
                "us_per_batch": r["ms_step"] * 1e3, "tops": r["ops"] / (r["ms_step"] * 1e-3) / 1e12, "kernel": r["kernel"],
                "channels_last_us": r["channels_last"]["ms"] * 1e3,
                "channels_last_equals_nchw_result": r["channels_last"]["equals_nchw_result"],
                "through_patch_buffer_us": r["through_patch_buffer"]["ms"] * 1e3,
                "through_patch_buffer_kernel": r["through_patch_buffer"]["kernel"]}

    def helpers():
        """The per-tensor helpers beside the layers (GetMinMax, Quantize, Dequantize: one streaming pass each) and the
        dynamic activation step built from them, on the 4096 x 4096 activation block; 6 rotating sets (384 MB of fp32)."""
        import ltq
        torch, dev = h.torch, h.dev
        n, sets = 4096 * 4096, 6
        xs = [torch.randn((4096, 4096), device=dev) for _ in range(sets)]
        qs = [torch.empty((4096, 4096), dtype=torch.uint8, device=dev) for _ in range(sets)]
        sums = torch.empty(4096, dtype=torch.int32, device=dev)
        mm = torch.empty(2, device=dev)
        qpd = torch.zeros(8, dtype=torch.uint8, device=dev)
        qp = ltq.QParams(0.04, 128)

        def f_minmax(i):
            ltq.GetMinMax(xs[i % sets], out=mm)

        def f_quant(i):
            ltq.Quantize(xs[i % sets], qp, out=qs[i % sets])

        def f_dequant(i):
            ltq.Dequantize(qs[i % sets], qp, out=xs[i % sets])

        def f_dynamic(i):   # GetMinMax -> ComputeQuantizationParams (device) -> quantize_rows with the device parameters
            ltq.GetMinMax(xs[i % sets], out=mm)
            ltq.compute_qparams_dev(mm, out=qpd)
            ltq.quantize_rows(xs[i % sets], qp_dev=qpd, q=qs[i % sets], asum=sums)

        c_src = [torch.empty(5 * n // 2, dtype=torch.uint8, device=dev) for _ in range(sets)]
        c_dst = [torch.empty(5 * n // 2, dtype=torch.uint8, device=dev) for _ in range(sets)]

        def f_copy(i):      # a plain device copy that moves the same 5 bytes per element: what a job of this size can reach
            c_dst[i % sets].copy_(c_src[i % sets])

        res = {"config": "4096 x 4096 fp32 block (64 MiB), 6 rotating sets; GB/s = algorithmic bytes / time, "
                         "frac_of_measured against the measured copy rate (taken on buffers of gigabytes); "
                         "device_copy_same_bytes = torch's device-to-device copy moving the bytes of quantize_u8 / "
                         "dequantize, timed the same way: the rate a streaming job of this size reaches"}
        for name, fn, nbytes in (("get_min_max", f_minmax, 4 * n), ("quantize_u8", f_quant, 5 * n),
                                 ("dynamic_quantize_rows", f_dynamic, 9 * n + 4 * 4096), ("dequantize", f_dequant, 5 * n),
                                 ("device_copy_same_bytes", f_copy, 5 * n)):
            ms = h.timed(fn, 24, 3, graph=not args.no_graph)
            gbs = nbytes / (ms * 1e-3) / 1e9
            res[name] = {"us": ms * 1e3, "gbs": gbs, "frac_of_measured": gbs / pk["hbm_gbs"], "algorithmic_bytes": nbytes}
        res["dynamic_quantize_rows"]["what"] = ("GetMinMax + ComputeQuantizationParams on the device + quantize_rows "
                                                "reading the parameters from device memory: the fp32 block is read twice")
        return res

    if only == "helpers":
        guarded("helpers", helpers)
        return out
    guarded("skinny", skinny)
    guarded("helpers", helpers)
    guarded("mlp_mnist", mnist)
    guarded("conv2d_q", conv)
    guarded("mlp_block_rows", block("rows"))
    if h.world > 1:
        guarded("mlp_block_cols", block("cols"))
        guarded("mlp_block_cols_fused", block("cols_fused"))
        guarded("mlp_block_cols_multicast", block("cols_multicast"))
    return out


# ---- 8192 -> 32768 -> 8192 block ---------------------------------------------------------------------------------------
def measure_mlp_block(h, args, shard, Mt, d_model, steps, warmup, alone=False):
    """8192 -> 32768 -> 8192 quantized MLP block with ReLU over Mt tokens (configs[4]), sharded over the ranks by
    activation rows (no collective) or by weight columns (all-gather of output slices over NCCL + relayout, or the
    exchange fused into the GEMM epilogue).  Total work is fixed, so scaling is strong.  `alone`: this rank runs all Mt
    tokens by itself, without touching the process group."""
    import ltq
    from ltq import sharded
    torch, dev = h.torch, h.dev
    world, rank = (1, 0) if alone else (h.world, h.rank)
    K1, N1, N2 = d_model, 4 * d_model, d_model
    g = torch.Generator(device=dev).manual_seed(77)          # weights identical on every rank
    w1 = torch.randn((N1, K1), generator=g, device=dev) * 0.01
    w2 = torch.randn((N2, N1), generator=g, device=dev) * 0.01
    qw1 = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(w1)))
    qw2 = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(w2)))
    w1q, w2q = ltq.Quantize(w1, qw1), ltq.Quantize(w2, qw2)
    # static calibration on a row sample, as the reference calibrates offline: input range and hidden (post-ReLU) range
    gs = torch.Generator(device=dev).manual_seed(78)
    sample = torch.randn((256, K1), generator=gs, device=dev)
    qx = ltq.ComputeQuantizationParams(-5.5, 5.5)            # N(0,1) activations: fixed calibrated range
    hid = torch.relu(sample @ w1.t())
    qh = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(hid)))
    del w1, w2, hid, sample
    egress = 0
    if shard == "rows":
        r0, r1 = sharded.shard_range(Mt, rank, world)
        M = r1 - r0
        l1 = ltq.LayerHandle(h.local, K1, N1)
        l1.set_weights(w1q, None)
        l1.set_qparams(qx, qw1, qh)
        l2 = ltq.LayerHandle(h.local, N1, N2)
        l2.set_weights(w2q, None)
        l2.set_qparams(qh, qw2, ltq.QParams(1.0, 0))
    else:
        M = Mt
        fused = shard in ("cols_fused", "cols_multicast")
        mc = shard == "cols_multicast"
        l1 = sharded.ColShardedLinear(w1q, None, N1, qx, qw1, qh, fused=fused, max_rows=M, out_mode=ltq.OUT_U8, multicast=mc)
        l2 = sharded.ColShardedLinear(w2q, None, N2, qh, qw2, ltq.QParams(1.0, 0), fused=fused, max_rows=M,
                                      out_mode=ltq.OUT_F32, multicast=mc)
        del w1q, w2q
        copies = 1 if (mc and l1.multicast) else world - 1     # a multicast store leaves the GPU once
        egress = copies * (M * (N1 // world) * 1 + M * (N2 // world) * 4)
        mc_in_use = bool(mc and l1.multicast)
    gx = torch.Generator(device=dev).manual_seed(1000 + (rank if shard == "rows" else 0))
    x = torch.randn((M, K1), generator=gx, device=dev)
    xq = torch.empty((M, K1), dtype=torch.uint8, device=dev)
    asum = torch.empty(M, dtype=torch.int32, device=dev)
    if shard == "rows":
        hq = torch.empty((M, N1), dtype=torch.uint8, device=dev)
        y = torch.empty((M, N2), dtype=torch.float32, device=dev)
        hsum = torch.zeros(M, dtype=torch.int32, device=dev)   # row sums of hq, left behind by layer 1's epilogue
        l1.set_rowsum_output(hsum)

        def step(i):
            hsum.zero_()
            ltq.quantize_rows(x, qp=qx, q=xq, asum=asum)
            l1.forward(xq, ltq.OUT_U8, ltq.FLAG_RELU, asum=asum, out=hq)
            l2.forward(hq, ltq.OUT_F32, 0, asum=hsum, out=y)
    elif fused:
        def step(i):
            ltq.quantize_rows(x, qp=qx, q=xq, asum=asum)
            hh = l1.forward(xq, ltq.OUT_U8, ltq.FLAG_RELU)      # epilogue stores into every rank's buffer
            l2.forward(hh, ltq.OUT_F32, 0)
    else:
        n1l, n2l = N1 // world, N2 // world
        loc1 = torch.empty((M, n1l), dtype=torch.uint8, device=dev)
        gat1 = torch.empty((world, M, n1l), dtype=torch.uint8, device=dev)
        hq = torch.empty((M, N1), dtype=torch.uint8, device=dev)
        loc2 = torch.empty((M, n2l), dtype=torch.float32, device=dev)
        gat2 = torch.empty((world, M, n2l), dtype=torch.float32, device=dev)
        y = torch.empty((M, N2), dtype=torch.float32, device=dev)

        def step(i):
            ltq.quantize_rows(x, qp=qx, q=xq, asum=asum)
            hh = l1.forward(xq, ltq.OUT_U8, ltq.FLAG_RELU, out=hq, gathered=gat1, local=loc1)
            l2.forward(hh, ltq.OUT_F32, 0, out=y, gathered=gat2, local=loc2)

    launches0 = ltq.kernel_launches()
    # NCCL collectives are not captured here: the column-sharded step is timed over eager launches
    use_graph = (not args.no_graph) and shard == "rows"
    ms_step = h.timed(step, steps, warmup, graph=use_graph, sample_clocks=not alone, local_only=alone)
    launches = (ltq.kernel_launches() - launches0) // (steps + warmup) * steps
    kernel = ltq.last_kernel()
    if shard == "rows":
        l1.check()
    elif hasattr(l1, "close"):
        l1.close()
        l2.close()
    ops = 2.0 * Mt * (K1 * N1 + N1 * N2)
    return dict(ms_step=ms_step, tops=ops / (ms_step * 1e-3) / 1e12, launches=int(launches), M=M, kernel=kernel,
                clocks=None if alone else getattr(h, "clocks", None), egress_bytes=egress,
                multicast=(shard == "cols_multicast" and mc_in_use),
                timing="CUDA graph replay" if use_graph else "eager launches (NCCL inside the step)")


def run_mlp_block(args):
    h = Harness(args)
    Mt, K1 = args.m_total, args.d_model
    N1, N2 = 4 * K1, K1
    r = measure_mlp_block(h, args, args.shard, Mt, K1, steps=args.steps, warmup=args.warmup)
    cfg = {"workload": f"mlp_block (configs[4]): {K1}->{N1}->{N2} with ReLU, {Mt} tokens in total, uint8 hidden "
                       "activations via fused requant, fp32 output",
           "sharding": {"rows": "activation rows split over the ranks, weights replicated, no collective",
                        "cols": "weight columns split over the ranks, all-gather of output slices (NCCL) + relayout "
                                "after each layer",
                        "cols_fused": "weight columns split over the ranks, the GEMM epilogue stores each rank's columns "
                                      "into every rank's output buffer over NVLink (peer stores), one 4-byte all-reduce "
                                      "per layer as the barrier",
                        "cols_multicast": "as cols_fused, the stores going once to an NVLink multicast address that "
                                          "NVSwitch replicates to every rank (multimem.st)"}[args.shard],
           "M_per_gpu": r["M"], "l2": "operands far larger than L2 (x, hidden and output are each >= 0.25 GB per rank)",
           "step": "quantize_rows + layer 1 (uint8, ReLU) + layer 2 (fp32)", "timing": r["timing"]}
    h.finish(base_line(h, args, r["tops"], "TOPS", r["ms_step"], "strong", cfg, samples_per_s=Mt / (r["ms_step"] * 1e-3),
                       gpu_launches=r["launches"], clocks=r["clocks"], kernel=r["kernel"], e2e=None, roofline=None,
                       cpu_baseline=None))


# ---- MNIST-shaped MLP ---------------------------------------------------------------------------------------------------
def measure_mlp_mnist(h, args):
    """MNIST-shaped 784-512-512-10 MLP, batch 64 (configs[0]); every rank is an independent replica with its own batch
    stream."""
    import ltq
    from ltq import workloads
    torch, dev = h.torch, h.dev
    x, layers = workloads.mlp_mnist(seed=0, batch=64)
    xd = torch.from_numpy(x).to(dev)
    acts = [xd]
    for (w, b) in layers:
        acts.append(torch.relu(acts[-1] @ torch.from_numpy(w).to(dev).t() + torch.from_numpy(b).to(dev)))
    qa = [ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(a.contiguous()))) for a in acts]
    hs = []
    for li, (w, b) in enumerate(layers):
        wd = torch.from_numpy(w).to(dev)
        qw = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(wd)))
        wq = ltq.Quantize(wd, qw)
        bq = ltq.QuantizeInt32(torch.from_numpy(b).to(dev), ltq.QParams(np.float32(qa[li].scale) * np.float32(qw.scale), 0))
        lh = ltq.LayerHandle(h.local, w.shape[1], w.shape[0])
        lh.set_weights(wq, bq)
        lh.set_qparams(qa[li], qw, qa[li + 1])
        hs.append(lh)
    xq = torch.empty((64, 784), dtype=torch.uint8, device=dev)
    asum = torch.empty(64, dtype=torch.int32, device=dev)
    h1 = torch.empty((64, 512), dtype=torch.uint8, device=dev)
    h2 = torch.empty((64, 512), dtype=torch.uint8, device=dev)
    y = torch.empty((64, 10), dtype=torch.float32, device=dev)
    # the hidden layers' epilogues leave the row sums the next layer needs, and each array is cleared for the next batch by
    # a layer that runs after its consumer: neither a sum pass nor a clearing launch between the layers
    sums = torch.zeros((2, 64), dtype=torch.int32, device=dev)
    hs[0].set_rowsum_output(sums[0])        # rows of h1, read by layer 2, cleared by layer 3
    hs[1].set_rowsum_output(sums[1])        # rows of h2, read by layer 3, cleared by layer 1 of the next batch
    hs[2].set_clear_on_forward(sums[0])
    hs[0].set_clear_on_forward(sums[1])
    kernels = []

    def step(i):
        ltq.quantize_rows(xd, qp=qa[0], q=xq, asum=asum)
        hs[0].forward(xq, ltq.OUT_U8, ltq.FLAG_RELU, asum=asum, out=h1)
        if i == 0:
            kernels.append(ltq.last_kernel())
        hs[1].forward(h1, ltq.OUT_U8, ltq.FLAG_RELU, asum=sums[0], out=h2)
        if i == 0:
            kernels.append(ltq.last_kernel())
        hs[2].forward(h2, ltq.OUT_F32, 0, asum=sums[1], out=y)
        if i == 0:
            kernels.append(ltq.last_kernel())

    steps = max(args.steps, 20)
    launches0 = ltq.kernel_launches()
    ms_layerwise = h.timed(step, steps, args.warmup, graph=not args.no_graph, sample_clocks=False)
    launches_layerwise = (ltq.kernel_launches() - launches0) // (steps + args.warmup)
    # the same batch through the fused chain: Quantize + the three layers in ONE launch (clusters of 8 CTAs, activations
    # in distributed shared memory)
    for lh in hs:
        lh.set_rowsum_output(None)
        lh.set_clear_on_forward(None)
    mlp = ltq.FusedMLP(hs)
    flags = [ltq.FLAG_RELU, ltq.FLAG_RELU, 0]
    y_ref = y.clone()
    kernels_fused = []

    def step_fused(i):
        mlp.forward(xd, flags, ltq.OUT_F32, out=y)
        if i == 0:
            kernels_fused.append(ltq.last_kernel())

    launches0 = ltq.kernel_launches()
    ms_step = h.timed(step_fused, steps, args.warmup, graph=not args.no_graph, sample_clocks=True)
    launches = (ltq.kernel_launches() - launches0) // (steps + args.warmup)
    same = bool(torch.equal(y, y_ref))

    # Throughput with several batches in flight: a chain launch occupies 4 clusters of 8 SMs, so independent batch
    # streams (a server with several request queues) run side by side on the rest of the device.  Four CUDA streams, each
    # with its own input and output buffers, batches dealt round robin; one graph holds all of them.
    S = 4
    steps_s = (max(steps, 40) + S - 1) // S * S
    side = [torch.cuda.Stream() for _ in range(S)]
    xs = [xd.clone() for _ in range(S)]
    ys = [torch.empty_like(y) for _ in range(S)]
    warm = max(args.warmup, S)

    def step_streams(i):
        k, cur, st = i - warm, torch.cuda.current_stream(), side[i % S]
        if k < S:
            st.wait_stream(cur)                                  # first batch of this stream in the timed region
        with torch.cuda.stream(st):
            mlp.forward(xs[i % S], flags, ltq.OUT_F32, out=ys[i % S])
        if k < 0 or k == steps_s - 1:
            for t in side:
                cur.wait_stream(t)

    ms_streams = h.timed(step_streams, steps_s, warm, graph=not args.no_graph)
    same_streams = all(bool(torch.equal(t, y_ref)) for t in ys)
    hs[0].check()
    return dict(ms_step=ms_step, launches_per_step=int(launches), steps=steps, kernels=kernels_fused,
                batch_streams={"streams": S, "us_per_batch": ms_streams * 1e3, "steps": steps_s,
                               "outputs_equal_single_stream": same_streams},
                ms_layerwise=ms_layerwise, launches_layerwise=int(launches_layerwise), kernels_layerwise=kernels,
                fused_equals_layerwise=same, clocks=getattr(h, "clocks", None))


def run_mlp_mnist(args):
    h = Harness(args)
    r = measure_mlp_mnist(h, args)
    ops = 2.0 * 64 * (784 * 512 + 512 * 512 + 512 * 10)
    cfg = {"workload": "mlp_mnist (configs[0]): 784-512-512-10, batch 64, uint8 hidden activations with fused ReLU, "
                       "fp32 logits", "sharding": "independent replicas, one batch stream per GPU",
           "l2": "the whole model (0.67 MB) is L2-resident by nature; this configuration is launch-latency bound",
           "step": "fused chain (ltq_mlp_forward): Quantize + 3 quantized linears in one launch; the layer-by-layer "
                   f"form (4 kernels) takes {r['ms_layerwise'] * 1e3:.2f} us per batch", "timing": "CUDA graph replay"}
    args.steps = r["steps"]
    h.finish(base_line(h, args, ops / (r["ms_step"] * 1e-3) / 1e12 * h.world, "TOPS", r["ms_step"], "weak", cfg,
                       samples_per_s=64 * h.world / (r["ms_step"] * 1e-3), gpu_launches=r["launches_per_step"] * r["steps"],
                       clocks=r["clocks"], kernels=r["kernels"], batch_streams=r["batch_streams"], e2e=None, roofline=None,
                       cpu_baseline=None))


def measure_conv(h, args, sample_clocks=False):
    """Conv2d_q on a ResNet-like layer: batch 32, 64 -> 64 channels, 56 x 56, 3 x 3, pad 1 (not one of the configs the
    metric is quoted on; it gives the convolution path a measured number).  A step = one Conv2d_q::forward on uint8
    NCHW input; this geometry takes the kernel without a patch buffer.  Timed beside it: the same layer inside a
    channels-last chain, and through the patch buffer."""
    import ltq
    torch, dev = h.torch, h.dev
    B, Cin, H, W, Cout, k = 32, 64, 56, 56, 64, 3
    sets = 4                                          # 4 x (6.4 MB input + 58 MB patches + 6.4 MB output)
    g = torch.Generator(device=dev).manual_seed(4321 + h.rank)
    xs = [torch.randint(0, 256, (B, Cin, H, W), dtype=torch.uint8, device=dev, generator=g) for _ in range(sets)]
    convs, outs = [], []
    for i in range(sets):
        wq = torch.randint(0, 256, (Cout, Cin * k * k), dtype=torch.uint8, device=dev, generator=g)
        c = ltq.ConvHandle(h.local, Cin, Cout, k, k, 1, 1, 1, 1)
        c.set_weights(wq)
        c.set_qparams(ltq.QParams(0.02, 128), ltq.QParams(0.005, 127), ltq.QParams(0.6, 5))
        convs.append(c)
        outs.append(torch.empty((B, Cout, H, W), dtype=torch.uint8, device=dev))

    def step(i):
        convs[i % sets].forward(xs[i % sets], ltq.OUT_U8, ltq.FLAG_RELU, out=outs[i % sets])

    for i in range(sets):      # every handle allocates its buffers on first use, which must not happen in a capture
        step(i)
    launches0 = ltq.kernel_launches()
    ms_step = h.timed(step, args.steps, args.warmup, graph=not args.no_graph, sample_clocks=sample_clocks)
    launches = (ltq.kernel_launches() - launches0) // (args.steps + args.warmup) * args.steps
    kernel = ltq.last_kernel()

    # the same layer inside a channels-last chain (input and output [B, H, W, C]: plain tensor copies, nothing to transpose)
    xs_cl = [x.permute(0, 2, 3, 1).contiguous() for x in xs]
    outs_cl = [torch.empty((B, H, W, Cout), dtype=torch.uint8, device=dev) for _ in range(sets)]
    cl = ltq.FLAG_RELU | ltq.FLAG_NHWC_IN | ltq.FLAG_NHWC_OUT

    def step_cl(i):
        convs[i % sets].forward(xs_cl[i % sets], ltq.OUT_U8, cl, out=outs_cl[i % sets])
    for i in range(sets):
        step_cl(i)
    ms_cl = h.timed(step_cl, args.steps, 3, graph=not args.no_graph)
    same = bool(torch.equal(outs_cl[0].permute(0, 3, 1, 2), convs[0].forward(xs[0], ltq.OUT_U8, ltq.FLAG_RELU)))

    # the same layer through the patch buffer (the form every geometry can take), for comparison
    def step_patches(i):
        convs[i % sets].forward(xs[i % sets], ltq.OUT_U8, ltq.FLAG_RELU | ltq.FLAG_FORCE_TC, out=outs[i % sets])
    for i in range(sets):
        step_patches(i)
    ms_patches = h.timed(step_patches, args.steps, 3, graph=not args.no_graph)
    kernel_patches = ltq.last_kernel()
    return dict(B=B, Cin=Cin, H=H, W=W, Cout=Cout, k=k, sets=sets, ms_step=ms_step, launches=int(launches), kernel=kernel,
                ops=2.0 * B * H * W * Cout * Cin * k * k,
                channels_last={"ms": ms_cl, "equals_nchw_result": same,
                               "step": "the kernel alone: input and output [B, H, W, C] (LTQ_FLAG_NHWC_IN | LTQ_FLAG_NHWC_OUT)"},
                through_patch_buffer={"ms": ms_patches, "kernel": kernel_patches,
                                      "step": "patch gather of the batch + patch sums + one GEMM over all images"})


def conv_workload_name(r):
    return (f"conv2d_q: batch {r['B']}, {r['Cin']}->{r['Cout']} channels, {r['H']}x{r['W']}, {r['k']}x{r['k']} kernel, pad 1, "
            "uint8 NCHW in/out, fused ReLU")


def run_conv(args):
    h = Harness(args)
    r = measure_conv(h, args, sample_clocks=True)
    ms_step, world = r["ms_step"], h.world
    cfg = {"workload": conv_workload_name(r), "sharding": "independent replicas, one batch stream per GPU",
           "l2": f"rotating {r['sets']} distinct input / output sets",
           "step": "one Conv2d_q forward of the batch: one kernel that gathers its NCHW input tile by tile (8-byte asynchronous "
                   "copies + a 4 x 4 byte transposition in registers) and reads every patch slice out of that tile (no NHWC copy, "
                   "no patch buffer)",
           "timing": "CUDA graph replay" if not args.no_graph else "eager launches"}
    h.finish(base_line(h, args, r["ops"] / (ms_step * 1e-3) / 1e12 * world, "TOPS", ms_step, "weak", cfg,
                       samples_per_s=r["B"] * world / (ms_step * 1e-3), gpu_launches=r["launches"], kernel=r["kernel"],
                       channels_last=r["channels_last"], through_patch_buffer=r["through_patch_buffer"],
                       clocks=getattr(h, "clocks", None), e2e=None, roofline=None, cpu_baseline=None))


def run_helpers(args):
    """The per-tensor helpers alone (GetMinMax, Quantize, Dequantize, the dynamic activation step): the `helpers` section
    of the default line as a line of its own, for profiling runs."""
    h = Harness(args)
    pk = peaks()
    r = run_sections(h, args, pk, only="helpers")["helpers"]
    if "error" in r:
        raise RuntimeError(r["error"])
    d = r["dynamic_quantize_rows"]
    cfg = {"workload": "helpers: GetMinMax / Quantize / Dequantize / dynamic quantize_rows on a 4096 x 4096 fp32 block",
           "l2": "6 rotating sets (384 MB of fp32)", "timing": "CUDA graph replay" if not args.no_graph else "eager launches"}
    args.steps = 24
    h.finish(base_line(h, args, d["gbs"] * h.world, "GB/s", d["us"] * 1e-3, "weak", cfg, helpers=r, gpu_launches=24 * 6,
                       e2e=None, roofline=None, cpu_baseline=None))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ltq", choices=["ltq", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "square_4096", "skinny", "mlp_block", "mlp_mnist", "conv", "helpers"],
                    help="all (default): the 4096^3 headline plus the skinny / mlp_mnist / mlp_block sections")
    ap.add_argument("--m", type=int, default=16, help="rows for the skinny workload (1, 4 or 16)")
    ap.add_argument("--m-total", type=int, default=65536, help="tokens of the mlp_block workload (all ranks together)")
    ap.add_argument("--d-model", type=int, default=8192, help="width of the mlp_block workload (hidden = 4x)")
    ap.add_argument("--shard", default="rows", choices=["rows", "cols", "cols_fused", "cols_multicast"], help="mlp_block partitioning")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps one by one instead of from a CUDA graph")
    ap.add_argument("--no-overlap", action="store_true",
                    help="quantise and multiply one after the other instead of overlapping batch i+1's quantisation with batch i's GEMM")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "mlp_block":
        run_mlp_block(args)
    elif args.workload == "mlp_mnist":
        run_mlp_mnist(args)
    elif args.workload == "conv":
        run_conv(args)
    elif args.workload == "helpers":
        run_helpers(args)
    else:
        run_linear(args, sections=args.workload == "all")


if __name__ == "__main__":
    main()
