#!/usr/bin/env python
"""Benchmark of the real-quantized segmented linear path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload layer|mmdit|sweep|kernels]

Headline workload (the same layer at every N): a FLUX-shape W8A8 INT8 SegLinear of the GEMM sweep -- X bf16
[M=16384, K=12288] in 4 equal K-segments whose magnitudes are drawn log-uniform in [0.25, 32], W bf16 [N=3072, K=12288]
~ N(0, 0.02) with per-output-channel int8 scales, bf16 output, seed 5.  Synthetic data, random-init weights.
One step = one layer forward on one batch: activation quantise (per-segment scales) + tcgen05 GEMM + scale / cast
epilogue.  With N > 1 the layer is COLUMN-SHARDED over the ranks (N/g output columns each, activations replicated)
and a step also includes the exchange of the output column blocks over NVLink: strong scaling.

Prints ONE JSON line (rank 0).  `value` is useful TOPS = 2*M*N*K / step time with inputs resident in HBM; `e2e` is the
same through the public layer API with pinned HOST input and a device->host read of the output inside the timed region.
`roofline` describes the dominant kernel (the GEMM) against 2 x the measured bf16 rate, burst and sustained;
`cpu_baseline` is the reference's own CPU path for the same layer on the box's host cores; `configs` (N = 1) carries
one compact entry per BASELINE configuration: the INT8 4-segment layer, the DualScale FP8 layer, the three W4A8
projections and the synthetic MMDiT denoise step.

`--impl reference` times the reference's own fake-quant SegmentLinear forward (imported, unmodified, through
oracle/reference_loader.py; the restatement in oracle/fake_path.py only where the reference package is absent) for the
headline layer on all host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# headline layer: a config[4] sweep point at FLUX shape (MLP down-projection), 4 K-segments
HM, HK, HN, HS, HSEED = 16384, 12288, 3072, 4, 5
HEAD_NAME = f"config[4] point: W8A8 INT8 SegLinear M={HM} K={HK} N={HN}, {HS} K-segments (scales log-uniform in [0.25, 32]), bf16 in/out, seed {HSEED}"
# profiles/seg_gemm2_int8_16384x3072x12288.md: dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline GEMM
HEAD_TRAFFIC_NCU = 543.4e6
HEAD_TRAFFIC_SRC = "profiles/seg_gemm2_int8_16384x3072x12288.md"


def log_uniform_scales(S, gen):
    return torch.exp(torch.empty(S).uniform_(-1.386, 3.466, generator=gen))   # [0.25, 32]


def headline_tensors(rows=HM, n_rows=None):
    """(x bf16 [rows, K], w bf16 [N, K]) from the seeded generator; identical on every rank."""
    g = torch.Generator().manual_seed(HSEED)
    scale = log_uniform_scales(HS, g)
    w = (torch.randn(HN, HK, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(rows, HK, generator=g)
    seg = HK // HS
    for s in range(HS):
        x[:, s * seg:(s + 1) * seg] *= scale[s]
    return x.to(torch.bfloat16), w


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except OSError:
        return {}


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.samples.append((time.perf_counter(), parts))

    def mark(self):
        return time.perf_counter()

    def summary(self, t0=None, t1=None):
        rows = [p for (t, p) in self.samples if (t0 is None or t >= t0) and (t1 is None or t <= t1)]
        sm = sorted(int(s[1]) for s in rows if s[1].isdigit())
        mx = [int(s[2]) for s in rows if s[2].isdigit()]
        pw = [float(s[3]) for s in rows if s[3].replace(".", "", 1).isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in rows:
            for name, v in zip(names, s[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(rows)}

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()   # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()


# ---------------------------------------------------------------------------------------------
# CPU baseline: the reference's own fake-quant path (or its restatement where the package is absent)
# ---------------------------------------------------------------------------------------------
def _import_reference():
    try:
        from oracle.reference_loader import find_reference, import_reference
        if find_reference() is None:
            return None
        import contextlib
        import io
        with contextlib.redirect_stdout(io.StringIO()):      # the reference prints on import; keep stdout one JSON line
            return import_reference("stub")
    except Exception:
        return None


def cpu_headline(runs=5, warmup=2):
    """The reference's SegmentLinear(real_quant=False).forward for the WHOLE headline layer (all rows, fp32 tensors: the
    bf16 values up-cast, which is the reference's fp32 CPU path), all host cores, best of `runs` after `warmup`."""
    torch.set_num_threads(os.cpu_count() or 1)
    x, w = headline_tensors()
    x, w = x.float(), w.float()
    ref = _import_reference()
    if ref is not None:
        lin = ref.SegmentLinear(HK, HN, bias=False, seg_mode="input", chunks=HS, custom_weight_tensor=w,
                                input_quant_type="int8", weight_quant_type="int8",
                                input_quant_args={"real_quant": False, "axis": None}, weight_quant_args={"real_quant": False, "axis": 1},
                                opt_type="default", opt_kwargs={}, calib_type="amax", calib_kwargs={}, device="cpu")
        lin.calibrate(x.clone())
        lin.finish_calibrate()
        kind, what = "reference", "the reference's own segquant.layers.SegmentLinear (unmodified package, stub extension loaders), real_quant=False"

        def fwd(xc):
            return lin(xc)          # writes into xc (optimizer.py:120-121): a fresh copy per run, made outside the timed region
    else:
        from oracle import fake_path as F
        seg = HK // HS
        bounds = [i * seg for i in range(HS + 1)]
        w_fake = F.fake_weight_int(w, 127.0)[0]
        sx = [F.amax_scale(x[:, bounds[s]:bounds[s + 1]], 127.0) for s in range(HS)]
        kind, what = "port", "oracle/fake_path.py restatement of the reference's fake-quant forward (reference package not importable here)"

        def fwd(xc):
            return F.seg_linear_fake(xc, w_fake, None, bounds, act="int8", sx=sx)
    times = []
    with torch.no_grad():
        for i in range(warmup + runs):
            xc = x.clone()
            t0 = time.perf_counter()
            fwd(xc)
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt)
    best = min(times)
    return {"value": 2.0 * HM * HN * HK / best / 1e12, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"the whole headline layer (all {HM} rows), fp32 fake-quant forward (per-segment quantise-dequantise + matmul + segment sum), "
                      f"{what}; best of {runs} runs after {warmup} warm-ups (mean {sum(times) / len(times) * 1e3:.0f} ms)",
            "ms_per_step": best * 1e3}


def cpu_mmdit_block(batch=2):
    """One fake-quant joint block (hidden 1536, 4096 + 333 tokens) on the host cores, best of 2 after 1 warm-up; the step
    baseline is this x 24 blocks (extrapolated, embedders and output head ignored)."""
    from oracle.mmdit_block_cpu import FakeQuantJointBlock
    torch.set_num_threads(os.cpu_count() or 1)
    ref = _import_reference()
    blk = FakeQuantJointBlock(ref=ref)
    g = torch.Generator().manual_seed(3)
    img, txt = torch.randn(batch, 4096, 1536, generator=g), torch.randn(batch, 333, 1536, generator=g)
    c = torch.nn.functional.silu(torch.randn(batch, 1536, generator=g))
    blk.calibrate(img, txt, c)
    times = []
    for i in range(3):
        t0 = time.perf_counter()
        blk(img, txt, c)
        if i >= 1:
            times.append(time.perf_counter() - t0)
    return {"one_block_ms": min(times) * 1e3, "step_ms_extrapolated": min(times) * 1e3 * 24, "kind": blk.kind, "cores": torch.get_num_threads(),
            "sample": f"ONE fake-quant joint block (all 14 linears + joint attention, fp32, batch {batch}) timed on the host cores, x 24 blocks"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb = cpu_headline(runs=max(1, args.steps), warmup=max(1, args.warmup))
    line = {
        "impl": "reference", "metric": "seglinear_gemm_tops", "value": cb["value"], "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": HEAD_NAME, "note": "reference's own CPU path (fake-quant SegmentLinear forward) on host cores; "
                                                  "value from the best timed step"},
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# helpers of our arm
# ---------------------------------------------------------------------------------------------
def _dist_setup():
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this library has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return dist, world, rank, dev


def timed(fn, steps, warmup=3):
    """Mean milliseconds per call of fn over `steps` calls (CUDA events on the current stream), after `warmup` calls."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def split_timed(quant, gemm, steps):
    """(quantise ms, GEMM ms) per launch: CUDA events around each launch on the launch stream, mean over `steps`."""
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    for e in ev:
        e[0].record()
        quant()
        e[1].record()
        gemm()
        e[2].record()
    torch.cuda.synchronize()
    return (sum(e[0].elapsed_time(e[1]) for e in ev) / steps, sum(e[1].elapsed_time(e[2]) for e in ev) / steps)


def graph_timed(fn, n, replays=3):
    """Mean milliseconds per call of fn with `n` calls recorded once into a CUDA graph and the replay timed by CUDA events:
    layers that run tens of microseconds are otherwise bound by the Python / ctypes launch path (15-40 us per call), not by
    the GPU.  fn may rotate over operand sets: the rotation is part of what is recorded."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    cur = torch.cuda.current_stream()
    side = torch.cuda.Stream()
    side.wait_stream(cur)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(n):
                fn()
    cur.wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    del graph
    return e0.elapsed_time(e1) / (n * replays)


def layer_bound(M, N, K, in_bytes, out_bytes, w_bytes_per_el, dual, peaks):
    """Roofline bound of a layer step in ms: max(useful-or-issued ops / tensor peak, algorithmic bytes / HBM bandwidth)."""
    tensor = 2.0 * peaks["tensor"]
    ops = 2.0 * M * N * K * (2 if dual else 1)
    byt = M * K * in_bytes + 2 * M * K * (2 if dual else 1) + N * K * w_bytes_per_el + M * N * out_bytes   # x in, xq out + in, W, y
    t_tensor, t_hbm = ops / (tensor * 1e12) * 1e3, byt / (peaks["hbm"] * 1e9) * 1e3
    return ("tensor" if t_tensor >= t_hbm else "hbm"), max(t_tensor, t_hbm)


# ---------------------------------------------------------------------------------------------
# the other BASELINE configurations, one compact entry each (N = 1)
# ---------------------------------------------------------------------------------------------
def config_entries(dev, peaks, steps=20):
    from segquant_b200 import _lib as L
    from segquant_b200 import ops
    from segquant_b200.layers.SegmentLinear import SegmentLinear
    out = {}
    pk = {"tensor": peaks.get("bf16_tflops") or 1590.0, "hbm": peaks.get("hbm_gbs") or 6650.0}
    peak8 = 2.0 * pk["tensor"]

    def run_layer(lin, x, kernel_type, dual, rotate):
        """rotate: independent (layer, x) pairs cycled so operands come from HBM; returns (step ms, quant ms, gemm ms)."""
        kind, a_kind, _ = ops.KERNELS[kernel_type]
        fs = []
        for ln, xx in rotate:
            ln.optimizer._build_fused()
            f = ln.optimizer._fused
            M_, K_ = xx.shape
            fs.append((f, xx, torch.empty((1, M_, K_), dtype=torch.uint8, device=dev),
                       torch.empty((1, M_, K_), dtype=torch.uint8, device=dev) if dual else None,
                       torch.empty((1, M_, f["N"]), dtype=xx.dtype, device=dev), ln.bias_data if ln.bias else None))
        state = {"i": 0}

        def quant():
            f, xx, xq, xqn, y, b = fs[state["i"] % len(fs)]
            ops.quantize_act(xx, f["bounds"], f["sx"], f["sx_neg"], a_kind, out=xq, out_neg=xqn)

        def gemm():
            f, xx, xq, xqn, y, b = fs[state["i"] % len(fs)]
            ops.gemm(kind, xq, f["wq"], f["N"], f["bounds"], f["sx"], f["sw"], xq_neg=xqn, sx_neg=f["sx_neg"], group_size=f["group"],
                     sw_strides=f["sw_strides"], bias=b, out_dtype=xx.dtype, out=y)
            state["i"] += 1

        def gemm_only():
            gemm()

        def quant_only():
            quant()
            state["i"] += 1

        def step():
            quant()
            gemm()
        n = max(steps, 4 * len(fs))
        ms = graph_timed(step, n)
        g_ms = graph_timed(gemm_only, n)       # every xq buffer of the rotation was filled by the steps above
        q_ms = graph_timed(quant_only, n)
        return ms, q_ms, g_ms

    # ---- config[0]: INT8, 4 K-segments, fp32 in / out, M=4096 K=N=1536, seed 0
    M, K, N, S = 4096, 1536, 1536, 4
    rot = []
    for r in range(4):
        g = torch.Generator().manual_seed(0 + 100 * r)
        x = torch.randn(M, K, generator=g)
        for s, f_ in enumerate([0.5, 1.0, 4.0, 16.0]):
            x[:, s * 384:(s + 1) * 384] *= f_
        x[:, torch.randperm(K, generator=g)[:30]] *= 20.0
        w = torch.randn(N, K, generator=g) * 0.02
        b = torch.randn(N, generator=g) * 0.01
        lin = SegmentLinear(K, N, bias=True, seg_mode="input", chunks=S, custom_weight_tensor=w.to(dev), custom_bias_tensor=b.to(dev),
                            input_quant_type="int8", weight_quant_type="int8", input_quant_args={"real_quant": True, "axis": None},
                            weight_quant_args={"real_quant": True, "axis": 1}, device=dev)
        xd = x.to(dev)
        lin.calibrate(xd)
        lin.finish_calibrate()
        rot.append((lin, xd))
    ms, q_ms, g_ms = run_layer(rot[0][0], rot[0][1], "Wint8Aint8", False, rot)
    bound, t_bound = layer_bound(M, N, K, 4, 4, 1, False, pk)
    out["config0_int8_4seg"] = {"workload": "config[0]: W8A8 INT8, fp32 in/out, M=4096 K=N=1536, 4 K-segments, seed 0", "ms": ms,
                                "tops_useful": 2.0 * M * N * K / ms / 1e9, "act_quant_ms": q_ms,
                                "roofline": {"bound": bound, "frac": t_bound / ms, "bound_ms": t_bound, "kernel": "seg_gemm_kernel<I8>", "kernel_ms": g_ms,
                                             "kernel_frac_of_2x_bf16": 2.0 * M * N * K / g_ms / 1e9 / peak8}}
    del rot
    # ---- config[1]: DualScale FP8 after GELU, bf16, M=4096 K=6144 N=1536, seed 1
    M, K, N = 4096, 6144, 1536
    rot = []
    for r in range(4):
        g = torch.Generator().manual_seed(1 + 100 * r)
        x = torch.nn.functional.gelu(torch.randn(M, K, generator=g).to(torch.bfloat16).float()).to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
        b = (torch.randn(N, generator=g) * 0.01).to(torch.bfloat16)
        lin = SegmentLinear(K, N, bias=True, seg_mode="weight", chunks=1, custom_weight_tensor=w.to(dev), custom_bias_tensor=b.to(dev),
                            input_quant_type="fpe4m3", weight_quant_type="fpe4m3",
                            input_quant_args={"real_quant": True, "axis": None, "dual_scale": True},
                            weight_quant_args={"real_quant": True, "axis": 1}, device=dev)
        xd = x.to(dev)
        lin.calibrate(xd)
        lin.finish_calibrate()
        rot.append((lin, xd))
    ms, q_ms, g_ms = run_layer(rot[0][0], rot[0][1], "Wfpe4m3Afpe4m3", True, rot)
    bound, t_bound = layer_bound(M, N, K, 2, 2, 1, True, pk)
    out["config1_fp8_dual"] = {"workload": "config[1]: DualScale W8A8 FP8-e4m3 down-projection, bf16, M=4096 K=6144 N=1536, seed 1", "ms": ms,
                               "tops_useful": 2.0 * M * N * K / ms / 1e9, "act_quant_ms": q_ms,
                               "act_quant_gbs": M * K * 4 / q_ms / 1e6, "act_quant_frac_of_hbm": M * K * 4 / q_ms / 1e6 / pk["hbm"],
                               "roofline": {"bound": bound, "frac": t_bound / ms, "bound_ms": t_bound, "kernel": "seg_gemm2_kernel<F8, dual>", "kernel_ms": g_ms,
                                            "kernel_frac_issued": 4.0 * M * N * K / g_ms / 1e9 / peak8,
                                            "kernel_frac_useful": 2.0 * M * N * K / g_ms / 1e9 / peak8,
                                            "note": "DualScale issues 4*M*N*K (positive and negative activation tiles against the same weights); "
                                                    "the useful fraction cannot exceed 0.5 by construction"}}
    del rot
    # ---- config[2]: W4A8, int4 weights with bf16 group scales (g=128), M=4608; QKV, MLP up (2 unequal K-segments), MLP down (DualScale after SiLU)
    M, G = 4608, 128
    entries = {}
    for name, N, K, bounds, dual in (("qkv", 9216, 3072, [0, 1024, 3072], False), ("mlp_up", 12288, 3072, [0, 1024, 3072], False),
                                     ("mlp_down", 3072, 12288, [0, 12288], True)):
        g = torch.Generator().manual_seed(2)
        if dual:
            x = torch.nn.functional.silu(torch.randn(M, K, generator=g)).to(torch.bfloat16).to(dev)
        else:
            x = torch.randn(M, K, generator=g)
            x[:, 1024:] *= 3.0
            x = x.to(torch.bfloat16).to(dev)
        w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        sw16 = (7.0 / w.float().view(N, K // G, G).abs().amax(-1)).to(torch.bfloat16).contiguous()
        wq = torch.empty(N * K // 2, dtype=torch.uint8, device=dev)
        ops.quantize_weight(w, wq, sw16.float().contiguous(), L.SQ_Q_INT4, group_size=G)
        sw_strides = (0, 0, 1, K // G)     # (N, K / G): what DualScale layers measure fastest with
        if not dual:
            sw16 = sw16.t().contiguous()   # group-major (K / G, N): a unit's scales are contiguous for the table builders
            sw_strides = (0, 0, N, 1)
        wq3 = wq.view(1, N, K // 2)
        xf = x.float()
        if dual:
            pos, neg = xf.clamp(min=0).max().item(), (-xf).clamp(min=0).max().item()
            sx, sxn = torch.tensor([127.0 / pos], device=dev), torch.tensor([128.0 / neg], device=dev)
        else:
            sx = torch.stack([127.0 / xf[:, bounds[s]:bounds[s + 1]].abs().max() for s in range(len(bounds) - 1)]).contiguous()
            sxn = None
        del xf, w
        xq = torch.empty((1, M, K), dtype=torch.uint8, device=dev)
        xqn = torch.empty((1, M, K), dtype=torch.uint8, device=dev) if dual else None
        y = torch.empty((1, M, N), dtype=torch.bfloat16, device=dev)

        def quant():
            ops.quantize_act(x, bounds, sx, sxn, L.SQ_Q_INT8, out=xq, out_neg=xqn)

        def gemm():
            ops.gemm(L.SQ_GEMM_W4A8, xq, wq3, N, bounds, sx, sw16, xq_neg=xqn, sx_neg=sxn, group_size=G, sw_strides=sw_strides,
                     out_dtype=torch.bfloat16, out=y)

        def step():
            quant()
            gemm()
        ms = graph_timed(step, steps)
        q_ms, g_ms = graph_timed(quant, steps), graph_timed(gemm, steps)
        entries[name] = {"N": N, "K": K, "dual_scale": dual, "ms": ms, "tops_useful": 2.0 * M * N * K / ms / 1e9, "act_quant_ms": q_ms,
                         "kernel_ms": g_ms, "kernel_frac_of_2x_bf16": 2.0 * M * N * K * (2 if dual else 1) / g_ms / 1e9 / peak8}
        del x, wq, wq3, xq, xqn, y
    out["timing"] = ("every entry: `steps` launches recorded once into a CUDA graph, the replay timed by CUDA events (ms = quantise + GEMM per "
                     "forward, kernel_ms / act_quant_ms = the kernel alone, back to back); configs 0 and 1 rotate over four operand sets "
                     "so activations and weights come from HBM")
    out["config2_w4a8_g128"] = {"workload": "config[2]: W4A8, int4 weights + bf16 group scales (g=128), bf16, M=4608, seed 2 "
                                            "(operands 50-170 MB per projection: weights partly L2-resident between steps, activations from HBM)",
                                "kernel": "seg_gemm_kernel<W4A8>", "projections": entries,
                                "note": "kernel_frac counts issued ops (4*M*N*K for the DualScale down-projection) against 2 x measured bf16"}
    return out


def mmdit_entry(dev, steps=5, cpu=True):
    from segquant_b200 import ops
    from segquant_b200.mmdit import GraphedStep, SyntheticMMDiT, synthetic_inputs
    model = SyntheticMMDiT(dev)
    inputs = synthetic_inputs(2, dev, seed=100)
    model.calibrate(*inputs)
    torch.cuda.synchronize()
    step = GraphedStep(model, *inputs)
    l0 = ops.launch_count
    ms = timed(lambda: step(*inputs), steps, warmup=3)
    launches = (ops.launch_count - l0) // (steps + 3)
    lin_ops = model.linear_ops(2)
    entry = {"workload": "config[3]: synthetic MMDiT denoise step, 24 joint blocks, hidden 1536, 4096+333 tokens, batch 2, every linear W8A8 INT8 "
                         "SegLinear, attention / norms bf16; one CUDA graph per step", "ms": ms, "linear_tops_useful": lin_ops / ms / 1e9,
             "library_kernels_per_step": launches}
    del step, model
    torch.cuda.empty_cache()
    if cpu:
        cb = cpu_mmdit_block(2)
        entry["cpu_baseline"] = cb
        entry["speedup_vs_cpu_extrapolated"] = cb["step_ms_extrapolated"] / ms
    return entry


def mmdit_dp_entry(dist, world, rank, dev, steps=3):
    """config[3] at N > 1: the denoise step batch-data-parallel, 16 samples split over the ranks (replicas: no collective
    inside the step, so a rank's time is the one-GPU time at its local batch).  Every rank runs; rank 0 gets the entry."""
    from segquant_b200.mmdit import GraphedStep, SyntheticMMDiT, synthetic_inputs
    batch = max(1, 16 // world)
    model = SyntheticMMDiT(dev)
    inputs = synthetic_inputs(batch, dev, seed=100 + rank)
    model.calibrate(*inputs)
    torch.cuda.synchronize()
    step = GraphedStep(model, *inputs)
    dist.barrier()
    ms = timed(lambda: step(*inputs), steps, warmup=3)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    ts = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(ts, t)
    per_rank = [float(v.item()) for v in ts]
    lin_ops = model.linear_ops(batch) * world
    del step, model
    torch.cuda.empty_cache()
    return {"workload": f"config[3]: synthetic MMDiT denoise step, batch-data-parallel: 16 samples over {world} GPUs ({batch} per GPU), "
                        "one CUDA graph per step and rank, no collective inside the step",
            "batch_per_gpu": batch, "ms": max(per_rank), "ms_per_rank": per_rank, "samples_per_s": batch * world / max(per_rank) * 1e3,
            "linear_tops_useful": lin_ops / max(per_rank) / 1e9}


# ---------------------------------------------------------------------------------------------
# our arm: the headline layer
# ---------------------------------------------------------------------------------------------
def run_ours(args):
    from segquant_b200 import _lib as L
    from segquant_b200 import ops
    dist, world, rank, dev = _dist_setup()
    L.load()
    peaks = load_peaks()
    bf16 = peaks.get("bf16_tflops")
    peak8 = 2.0 * (bf16 or 1590.0)
    peak8_sus = 2.0 * (peaks.get("bf16_tflops_sustained") or 1400.0)
    hbm = peaks.get("hbm_gbs") or 6650.0
    peak_src = "of measured" if bf16 else "of fallback"
    if HN % world:
        raise SystemExit(f"bench.py: N={HN} is not divisible by {world} ranks")
    n_loc = HN // world

    x_cpu, w_cpu = headline_tensors()
    x = x_cpu.to(dev)
    from segquant_b200.sharded import ColumnShardedSegLinear, row_range, shard_range
    cs = ColumnShardedSegLinear.from_full(x, w_cpu.to(dev), None, rank, world, kernel_type="Wint8Aint8", seg_mode="input", chunks=HS)
    lin = cs.layer
    lin.optimizer._build_fused()
    f = lin.optimizer._fused
    kind, a_kind, _ = ops.KERNELS["Wint8Aint8"]
    xq = torch.empty((1, HM, HK), dtype=torch.uint8, device=dev)
    y_loc = torch.empty((1, HM, n_loc), dtype=torch.bfloat16, device=dev)
    torch.cuda.synchronize()

    def quant():
        ops.quantize_act(x, f["bounds"], f["sx"], None, a_kind, out=xq)

    def gemm():
        ops.gemm(kind, xq, f["wq"], n_loc, f["bounds"], f["sx"], f["sw"], sw_strides=f["sw_strides"], out_dtype=torch.bfloat16, out=y_loc)

    exchange = None
    if world > 1:
        cs.enable_symmetric(HM)
        exchange = args.exchange
        fwd = {"auto": cs.forward_auto, "push": cs.forward_push, "fused": cs.forward_fused, "nccl": cs.forward}[exchange]

        def step():
            return fwd(x)
    else:
        def step():
            quant()
            gemm()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(vals):
        t = torch.tensor(vals, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    W = max(args.warmup, 3)
    for _ in range(W):
        step()
    barrier()
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    launches0 = ops.launch_count
    t_mark0 = sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    t_mark1 = sampler.mark()
    launches = ops.launch_count - launches0
    (ms_step,) = max_over_ranks([e0.elapsed_time(e1) / args.steps])

    # ---- the two kernels alone (every rank, max over ranks)
    q_ms, g_ms = split_timed(quant, gemm, args.steps)
    q_ms, g_ms = max_over_ranks([q_ms, g_ms])
    sharded = None
    if world > 1:
        # exchange alone: the same step with the GEMM output already in place (push of the block + barrier), and each method's total
        lo, hi = shard_range(HN, world, rank)
        esz = 2
        out_bytes = HM * n_loc * esz * (world - 1)
        totals = {}
        for name, fn in (("nccl_allgather", cs.forward), ("block_push", cs.forward_push), ("fused_epilogue", cs.forward_fused)):
            barrier()
            (totals[name],) = max_over_ranks([timed(lambda: fn(x), args.steps)])
        full, peers = cs._next_buffer(HM)
        mine = full[:, lo:hi]

        def push_only():
            ops.push_columns(mine, [p + lo * esz for p in peers], HN * esz)
            cs._barrier()
        barrier()
        (push_ms,) = max_over_ranks([timed(push_only, args.steps)])
        # results: every method gives the same [M, N] matrix on every rank
        y_nccl = cs.forward(x)
        same = int(torch.equal(cs.forward_push(x), y_nccl)) & int(torch.equal(cs.forward_fused(x), y_nccl))
        (same,) = max_over_ranks([1 - same])
        nvlink = 770.0     # GB/s per direction per GPU: the measured peer-copy rate on this pool (nominal 900)
        t_link = out_bytes / (nvlink * 1e9) * 1e3
        sharded = {"what": f"N={HN} split into {world} column blocks of {n_loc}; activations replicated and quantised on every rank; "
                           f"exchange method of the headline value: {exchange}",
                   "gemm_only_ms": g_ms, "act_quant_ms": q_ms, "exchange_ms": push_ms, "total_ms": ms_step,
                   "totals_ms_by_method": totals, "methods_agree": same == 0,
                   "exchange_bytes_out_per_gpu": out_bytes, "exchange_gbs_per_gpu": out_bytes / push_ms / 1e6,
                   "nvlink_frac": out_bytes / push_ms / 1e6 / nvlink,
                   "nvlink_peak_gbs": nvlink, "nvlink_note": "measured peer-copy rate per direction per GPU on this pool (nominal 900)",
                   "ceiling": {"exchange_ms_at_nvlink_peak": t_link,
                               "total_ms_if_exchange_fully_overlapped": q_ms + max(g_ms, t_link),
                               "note": "the exchange must move (g-1)/g*M*N*2 bytes out of every GPU; the quantise of the replicated activations does not shrink with g"}}

    # ---- sustained: the same step looped for more than a second (N = 1)
    sustained = None
    if world == 1 and not args.quick:
        n_sus = max(50, int(1300.0 / ms_step))
        ts0 = sampler.mark()
        ms_sus = timed(step, n_sus, warmup=0)
        ts1 = sampler.mark()
        gq, gg = split_timed(quant, gemm, 20)
        time.sleep(0.15)
        clk = sampler.summary(ts0, ts1)
        sustained = {"steps": n_sus, "seconds": ms_sus * n_sus / 1e3, "ms_per_step": ms_sus, "tops_useful": 2.0 * HM * HN * HK / ms_sus / 1e9,
                     "kernel_ms_hot": gg, "sm_mhz_median": clk["sm_mhz"], "power_w_max": clk["power_w_max"], "reasons": clk["reasons"],
                     "peak": peak8_sus, "frac": 2.0 * HM * HN * HK / (ms_sus - gq) / 1e9 / peak8_sus if ms_sus > gq else None,
                     "note": f"frac = 2*M*N*K / (step - quantise) against 2 x the measured sustained bf16 rate ({peak_src}); quantise time "
                             "taken right after the loop, at the same clocks"}

    # ---- end to end through the public layer API with host buffers
    r_lo, r_hi = row_range(HM, world, rank)
    host_x = [x_cpu[r_lo:r_hi].contiguous().pin_memory() for _ in range(2)]
    o_lo, o_hi = row_range(HM, world, rank)
    host_y = torch.empty((o_hi - o_lo, HN), dtype=torch.bfloat16).pin_memory()
    if world == 1:
        s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        x_dev = [torch.empty((HM, HK), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        y_dev = [torch.empty((1, HM, HN), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        ev_in, ev_cmp, ev_out = ([torch.cuda.Event() for _ in range(2)] for _ in range(3))

        def e2e_step(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_cmp[b])              # the forward two steps ago has consumed x_dev[b]
                x_dev[b].copy_(host_x[b], non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in[b])
                s_cmp.wait_event(ev_out[b])             # y_dev[b] has been read back
                lin(x_dev[b].unsqueeze(0), out=y_dev[b])
                ev_cmp[b].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[b])
                host_y.copy_(y_dev[b][0], non_blocking=True)
                ev_out[b].record(s_out)

        def e2e_run(n):
            for st_ in (s_in, s_cmp, s_out):
                st_.wait_stream(torch.cuda.current_stream())
            for i in range(n):
                e2e_step(i)
            for st_ in (s_in, s_cmp, s_out):
                torch.cuda.current_stream().wait_stream(st_)
        e2e_mode = ("SegmentLinear.forward(x, out=) fed from pinned host memory; copy-in, forward and read-back of consecutive steps "
                    "overlap on three streams (double-buffered)")
    else:
        from segquant_b200.sharded import HostRowPipeline
        pipe = HostRowPipeline(cs, HM, HK, torch.bfloat16, torch.bfloat16, exchange=exchange)

        def e2e_run(n):
            pipe.run(n, host_x, host_y)
        e2e_mode = ("sharded.HostRowPipeline: every rank copies its 1/g of the input rows from pinned host memory, the rows are "
                    "all-gathered over NVLink, sharded forward + exchange, every rank reads back its 1/g of the output rows; copy-in, "
                    "compute and read-back of consecutive steps overlap on three streams (double-buffered)")
    e2e_steps = 1 if args.quick else args.steps
    e2e_run(1 if args.quick else 3)
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    e2e_run(e2e_steps)
    e3.record()
    barrier()
    (e2e_ms,) = max_over_ranks([e2.elapsed_time(e3) / e2e_steps])
    clocks = None
    if rank == 0:
        time.sleep(0.15)
        clocks = sampler.summary(t_mark0, t_mark1)
        if not clocks["samples"]:
            clocks = sampler.summary()
        sampler.stop()

    status = ops.device_status()
    configs = None
    if world == 1 and rank == 0 and args.configs != "none" and not args.quick:
        del x, xq, y_loc
        torch.cuda.empty_cache()
        configs = config_entries(dev, peaks)
        configs["config3_mmdit_step"] = mmdit_entry(dev, cpu=args.configs == "all")
        status = status or ops.device_status()
    if world > 1 and args.configs != "none" and not args.quick:
        del x, xq, y_loc, cs
        torch.cuda.empty_cache()
        configs = {"config3_mmdit_step": mmdit_dp_entry(dist, world, rank, dev)}
        status = status or ops.device_status()
    if rank == 0:
        achieved = 2.0 * HM * n_loc * HK / g_ms / 1e9
        line = {
            "metric": "seglinear_gemm_tops", "value": 2.0 * HM * HN * HK / ms_step / 1e9, "unit": "TOPS",
            "n_gpus": world, "steps": args.steps, "warmup": W, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": HEAD_NAME,
                       "step": "activation quantise + GEMM + epilogue" + ("" if world == 1 else f" + exchange of the output column blocks ({exchange})"),
                       "ops_counted": "useful 2*M*N*K of the whole layer",
                       "cache": f"inputs larger than L2: activations {HM * HK * 2 / 1e6:.0f} MB bf16 + {HM * HK / 1e6:.0f} MB quantised per step (L2 126 MB)",
                       "parallelism": "1 GPU" if world == 1 else f"column-sharded over {world} GPUs (N/{world} = {n_loc} columns each)"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak8, "unit": "TFLOP/s", "frac": achieved / peak8,
                         "traffic": HEAD_TRAFFIC_NCU if world == 1 else None,
                         "traffic_source": HEAD_TRAFFIC_SRC + " (one ncu capture of this kernel on this workload; a constant, not re-measured by this run)",
                         "algorithmic_bytes": HM * HK + n_loc * HK + HM * n_loc * 2,
                         "kernel": "seg_gemm2_kernel<I8, KSUB=2> (CTA pair, tcgen05.mma.cta_group::2.kind::i8)", "kernel_ms": g_ms,
                         "frac_useful": achieved / peak8, "frac_issued": achieved / peak8,
                         "sustained": sustained,
                         "note": f"achieved = 2*M*(N/g)*K per launch / mean launch time (CUDA events on the launch stream); peak = 2 x measured bf16 burst ({peak_src}); "
                                 "single-scale layer: issued = useful"},
            "e2e": {"value": 2.0 * HM * HN * HK / e2e_ms / 1e9, "unit": "TOPS", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": (r_hi - r_lo) * HK * 2, "d2h_bytes_per_step": (o_hi - o_lo) * HN * 2, "bytes_are": "per rank", "mode": e2e_mode},
            "kernels": {"act_quant_ms": q_ms, "act_quant_gbs": HM * HK * 3 / q_ms / 1e6, "act_quant_frac_of_hbm": HM * HK * 3 / q_ms / 1e6 / hbm,
                        "act_quant_note": "algorithmic bytes M*K*(2 in + 1 out) per launch / mean CUDA-event time, inside the step loop",
                        "seg_gemm_ms": g_ms},
            "gpu_launches": launches, "clocks": clocks, "device_status": status,
        }
        if sharded:
            line["sharded"] = sharded
        if configs:
            line["configs"] = configs
        if world == 1 and args.configs != "none" and not args.quick:
            line["cpu_baseline"] = {k: v for k, v in cpu_headline().items() if k != "ms_per_step"}
        else:
            line["cpu_baseline"] = {"value": None, "unit": "TOPS", "cores": os.cpu_count(), "kind": "reference",
                                    "sample": "timed on rank 0 at N = 1 only (the host cores are busy driving the ranks here); see the N = 1 line or --impl reference"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# other workloads (not the default line): synthetic MMDiT denoise step, GEMM sweep, HBM kernels
# ---------------------------------------------------------------------------------------------
def run_mmdit(args):
    """config[3]: 24-block SD3.5-medium-like MMDiT, every linear W8A8 INT8 SegLinear, attention / norms bf16.
    Batch 2 on one GPU; batch 16 split over 2 / 4 / 8 GPUs (replicas, no collective inside the step)."""
    from segquant_b200 import ops
    from segquant_b200.mmdit import GraphedStep, SyntheticMMDiT, synthetic_inputs
    dist, world, rank, dev = _dist_setup()
    batch = 2 if world == 1 else 16 // world
    if args.mmdit_batch:
        batch = args.mmdit_batch
    model = SyntheticMMDiT(dev, out_proj_segments=args.out_proj_segments)
    inputs = synthetic_inputs(batch, dev, seed=100 + rank)
    model.calibrate(*inputs)
    torch.cuda.synchronize()
    eager = model
    if not args.no_graph:
        model = GraphedStep(eager, *inputs)
    for _ in range(max(args.warmup, 3)):
        y = model(*inputs)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    l0 = ops.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        y = model(*inputs)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches = ops.launch_count - l0
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    # end to end: host latents in, host noise prediction out
    host_in = [x.cpu().pin_memory() for x in inputs]
    host_out = torch.empty(y.shape, dtype=y.dtype).pin_memory()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e2.record()
    for _ in range(max(2, args.steps // 4)):
        dev_in = [x.to(dev, non_blocking=True) for x in host_in]
        host_out.copy_(model(*dev_in), non_blocking=True)
    e3.record()
    torch.cuda.synchronize()
    t2 = torch.tensor([e2.elapsed_time(e3) / max(2, args.steps // 4)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    clocks = None
    if rank == 0:
        time.sleep(0.15)
        clocks = sampler.summary()
        sampler.stop()
    status = ops.device_status()
    if rank == 0:
        peaks = load_peaks()
        lin_ops = eager.linear_ops(batch)
        tokens = eager.img_tokens + eager.txt_tokens
        attn_flops = 24 * batch * 4 * tokens * tokens * eager.hidden
        p8, p16 = 2.0 * (peaks.get("bf16_tflops") or 1590.0), peaks.get("bf16_tflops") or 1590.0
        bound_ms = (lin_ops / (p8 * 1e12) + attn_flops / (p16 * 1e12)) * 1e3
        line = {
            "metric": "mmdit_denoise_step_ms", "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": False,
            "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "int8 linears, bf16 attention", "data": "synthetic",
            "config": {"workload": f"config[3]: synthetic MMDiT, 24 joint blocks, hidden 1536, 4096+333 tokens, batch {batch} per GPU "
                                   f"({batch * world} total), attention output projections with {args.out_proj_segments} K-segment(s)",
                       "launch": "eager" if args.no_graph else "one CUDA graph per step", "parallelism": f"dp{world} replicas"},
            "linear_tops": lin_ops / ms / 1e9, "linear_ops_per_step": lin_ops, "attention_flops_per_step": attn_flops,
            "roofline": {"bound": "tensor", "bound_ms": bound_ms, "frac": bound_ms / ms, "unit": "ms",
                         "note": "bound = int8 linear ops / (2 x measured bf16) + bf16 attention flops / measured bf16; frac = bound / measured step"},
            "e2e": {"value": t2.item(), "unit": "ms", "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in host_in),
                    "d2h_bytes_per_step": host_out.numel() * host_out.element_size()},
            "gpu_launches": launches, "clocks": clocks, "device_status": status,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_mmdit_block(batch)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


SWEEP_NK = [(1536, 1536), (6144, 1536), (1536, 6144), (9216, 3072), (12288, 3072), (3072, 12288), (1280, 5120)]


def run_sweep(args):
    """config[4]: M x (N, K) x {INT8, FP8, W4A8 g=128} x segments {1,2,4,8}; each point column-sharded over the
    ranks.  Per point: layer time (quantise + GEMM on this rank's columns), and with N > 1 the total with each exchange
    (NCCL all-gather + interleave, block push, fused epilogue) and a check that all give the same matrix.  Every point is
    also CHECKED: 64 rows spread over the matrix against the CPU oracle (run outside every timed region, as the checker);
    the run fails if a point is more than one bf16 step off.  Prints one JSON line holding every point."""
    from segquant_b200 import _lib as L
    from segquant_b200 import ops
    from segquant_b200.sharded import all_gather_slices, shard_range
    dist, world, rank, dev = _dist_setup()
    g = torch.Generator().manual_seed(5)
    points = []
    modes = [("int8", "Wint8Aint8", L.SQ_Q_INT8, 0), ("fp8", "Wfpe4m3Afpe4m3", L.SQ_Q_E4M3, 0), ("w4a8", "Wint4Aint8", L.SQ_Q_INT4, 128)]
    Ms = [int(m) for m in args.sweep_m.split(",")]
    nks = SWEEP_NK if not args.sweep_nk else [tuple(int(v) for v in nk.split("x")) for nk in args.sweep_nk.split(",")]
    modes = [m for m in modes if m[0] in args.sweep_modes.split(",")]
    seg_counts = [int(v) for v in args.sweep_segs.split(",")]
    w4_group = args.sweep_w4_group
    modes = [(n_, k_, w_, (w4_group if n_ == "w4a8" else g_)) for (n_, k_, w_, g_) in modes]
    check = not args.no_check
    if check:
        import numpy as np
        from oracle import oracle as O
        okind = {"int8": O.GEMM_I8, "fp8": O.GEMM_F8, "w4a8": O.GEMM_W4A8}
        oq = {"int8": O.Q_INT8, "fp8": O.Q_E4M3, "w4a8": O.Q_INT8}
    worst = 0.0
    bar_ptrs, bar_words, epoch = None, None, [0]

    def rank_barrier():      # stream-ordered: every rank's kernels before it are complete, and their stores visible, after it
        epoch[0] += 1
        ops.peer_barrier(rank, bar_ptrs, epoch[0], dev)

    for (N, K) in nks:
        if N % world:
            continue
        lo, hi = shard_range(N, world, rank)
        n_loc = hi - lo
        full = peers = None
        if world > 1 and not args.no_symmetric:
            # every rank's [M, N] result buffer, mapped into all processes: epilogue stores / block pushes go to all of them
            import torch.distributed._symmetric_memory as symm
            full = symm.empty((max(Ms), N), dtype=torch.bfloat16, device=dev)
            handle = symm.rendezvous(full, dist.group.WORLD)
            peers = [int(p_) for r_, p_ in enumerate(handle.buffer_ptrs) if r_ != rank]
            if bar_ptrs is None:        # barrier words (ops.peer_barrier), zero before anybody's first epoch
                bar_words = symm.empty((64,), dtype=torch.int32, device=dev)
                bar_words.zero_()
                torch.cuda.synchronize()
                bar_ptrs = [int(p_) for p_ in symm.rendezvous(bar_words, dist.group.WORLD).buffer_ptrs]
                dist.barrier()
        w = (torch.randn(n_loc, K, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        for name, ktype, wkind, group in modes:
            qmax = {L.SQ_Q_INT8: 127.0, L.SQ_Q_E4M3: 448.0, L.SQ_Q_INT4: 7.0}[wkind]
            if group:
                sw_ng = (qmax / w.float().view(n_loc, K // group, group).abs().amax(-1)).contiguous()
                wq = torch.empty(n_loc * K // 2, dtype=torch.uint8, device=dev)
                ops.quantize_weight(w, wq, sw_ng, wkind, group_size=group)
                # the GEMM takes the group scales group-major, (K / g, N): one accumulation unit's scales are then contiguous
                sw = sw_ng.t().contiguous()
                wq3, strides = wq.view(1, n_loc, K // 2), (0, 0, n_loc, 1)
            else:
                sw = (qmax / w.float().abs().amax(-1)).contiguous()
                kb = K // 2 if wkind == L.SQ_Q_INT4 else K          # bytes per weight row
                wq = torch.empty(n_loc * kb, dtype=torch.uint8, device=dev)
                ops.quantize_weight(w, wq if wkind == L.SQ_Q_INT4 else wq.view(n_loc, K), sw, wkind)
                wq3, strides = wq.view(1, n_loc, kb), (0, 0, 0, 1)
            for M in Ms:
                for S in seg_counts:
                    if K % (S * 32):
                        continue
                    bounds = ops.uniform_bounds(K, S)
                    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
                    scale = log_uniform_scales(S, g)
                    for s_ in range(S):
                        x[:, bounds[s_]:bounds[s_ + 1]] *= scale[s_].to(torch.bfloat16)
                    x = x.to(dev)
                    aq = 448.0 if name == "fp8" else 127.0
                    sx = torch.stack([aq / x[:, bounds[s_]:bounds[s_ + 1]].float().abs().max() for s_ in range(S)]).contiguous()

                    def fwd():
                        return ops.seg_linear(ktype, x, wq3, n_loc, bounds, sx, sw, group_size=group, sw_strides=strides)

                    for _ in range(3):
                        y = fwd()
                    torch.cuda.synchronize()
                    err = None
                    if check:
                        # 64 rows spread over the matrix, through the oracle's own quantise and integer GEMM
                        rows = torch.linspace(0, M - 1, 64).long().unique()
                        xr = x[rows].float().cpu().numpy()
                        xq_ref = O.quantize_act(xr, bounds, sx.cpu().numpy(), out_kind=oq[name])
                        sw_o = sw.cpu().numpy()            # group-major (K / g, N) is also the oracle's layout
                        y_ref = O.seg_gemm(okind[name], xq_ref, wq.cpu().numpy() if wkind == L.SQ_Q_INT4 else wq.view(n_loc, K).cpu().numpy(),
                                           bounds, sx.cpu().numpy(), sw_o, group_size=group)
                        want = torch.from_numpy(y_ref).to(torch.bfloat16).float().numpy()
                        got = y[rows.to(dev)].float().cpu().numpy()
                        err = float(np.abs(got - want).max() / np.abs(want).max())
                        worst = max(worst, err)
                    it = args.sweep_iters
                    # `it` forwards recorded once into a CUDA graph: small layers are otherwise bound by the Python / ctypes
                    # launch path (~30 us per call), not by the GPU
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.stream(side):
                        with torch.cuda.graph(graph, stream=side):
                            for _ in range(it):
                                y = fwd()
                    torch.cuda.current_stream().wait_stream(side)
                    graph.replay()
                    torch.cuda.synchronize()
                    if world > 1:
                        all_gather_slices(y)          # communicator set-up and buffers happen outside the timed loop
                        torch.cuda.synchronize()
                    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                    e[0].record()
                    graph.replay()
                    e[1].record()
                    for _ in range(it if world > 1 else 0):
                        y = fwd()
                        gathered = all_gather_slices(y)
                    e[2].record()
                    torch.cuda.synchronize()
                    del graph
                    ms_fused = ms_push = None
                    same_ok = None
                    if full is not None:
                        ref_full = gathered.permute(1, 0, 2).reshape(M, N)
                        mine = full[:M, lo:hi]

                        def fwd_fused():
                            ops.seg_linear(ktype, x.unsqueeze(0), wq3, n_loc, bounds, sx, sw, group_size=group, sw_strides=strides,
                                           out=mine.unsqueeze(0), peer_outputs=(peers, N, lo))
                            rank_barrier()

                        def fwd_push():
                            ops.seg_linear(ktype, x.unsqueeze(0), wq3, n_loc, bounds, sx, sw, group_size=group, sw_strides=strides, out=mine.unsqueeze(0))
                            ops.push_columns(mine, [p_ + lo * 2 for p_ in peers], N * 2)
                            rank_barrier()
                        res = []
                        for fn in (fwd_fused, fwd_push):
                            full.zero_()
                            torch.cuda.synchronize()
                            dist.barrier()
                            ms_ = timed(fn, it, warmup=2)
                            tf = torch.tensor([ms_], dtype=torch.float64, device=dev)
                            dist.all_reduce(tf, op=dist.ReduceOp.MAX)
                            same = torch.tensor([int(torch.equal(full[:M], ref_full))], device=dev)
                            dist.all_reduce(same, op=dist.ReduceOp.MIN)
                            res.append((tf.item(), bool(same.item())))
                            dist.barrier()             # nobody clears its buffer while a peer may still compare against stores in flight
                        (ms_fused, ok_f), (ms_push, ok_p) = res
                        same_ok = ok_f and ok_p
                    t = torch.tensor([e[0].elapsed_time(e[1]) / it, e[1].elapsed_time(e[2]) / it], dtype=torch.float64, device=dev)
                    if world > 1:
                        dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    ms_c, ms_t = t.tolist()
                    points.append({"mode": name, "M": M, "N": N, "K": K, "S": S, "layer_ms": ms_c, "layer_tops": 2.0 * M * N * K / ms_c / 1e9,
                                   "max_rel_vs_oracle_64rows": err,
                                   "with_allgather_ms": ms_t if world > 1 else None, "with_fused_gather_ms": ms_fused, "with_block_push_ms": ms_push,
                                   "exchanges_equal_allgather": same_ok})
    status = ops.device_status()
    if world > 1:
        wt = torch.tensor([worst], dtype=torch.float64, device=dev)
        dist.all_reduce(wt, op=dist.ReduceOp.MAX)
        worst = wt.item()
    if rank == 0:
        best = {m: max((p["layer_tops"] for p in points if p["mode"] == m), default=0.0) for m in ("int8", "fp8", "w4a8")}
        print(json.dumps({"metric": "seglinear_gemm_tops_sweep", "unit": "TOPS", "n_gpus": world, "higher_is_better": True,
                          "scaling": "strong", "data": "synthetic", "value": max(best.values()), "best_tops": best,
                          "config": {"workload": "config[4]: GEMM sweep, layer = activation quantise + GEMM + epilogue, bf16 in/out, "
                                                 "N column-sharded over the ranks", "iters": args.sweep_iters},
                          "correctness": {"checked": check, "worst_max_rel_vs_oracle": worst if check else None,
                                          "bar": "bf16 output of 64 rows per point within one bf16 step of the largest value (2^-7 relative to it: 8 significant bits) of the "
                                                 "CPU oracle's fp32 result rounded to bf16"},
                          "device_status": status, "points": points}), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if check and worst > 2.0 ** -7:
        raise SystemExit(f"bench.py sweep: a point is {worst:.3e} away from the oracle (bar 2^-7, one bf16 step of the largest value)")


def run_configs(args):
    """The `configs` block of the default line on its own (configs 0-2 as layers; config 3 with --configs all / gpu):
    what the ncu captures of those kernels run."""
    from segquant_b200 import ops
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    out = config_entries(dev, load_peaks(), steps=args.steps)
    if args.configs != "none":
        out["config3_mmdit_step"] = mmdit_entry(dev, steps=max(2, args.steps // 4), cpu=args.configs == "all")
    print(json.dumps({"metric": "seglinear_configs", "n_gpus": 1, "data": "synthetic", "configs": out, "device_status": ops.device_status()}), flush=True)


def run_kernels(args):
    """The HBM-bound kernels alone on [rows, 12288] tensors (larger than L2): activation quantise (bf16 / fp32, single,
    DualScale, dynamic per-token), weight quantise (int8, packed int4 with group scales), int4 unpack, and the fused
    LayerNorm + modulation + quantise and the gated residual add on the same bytes seen as rows of 1536.
    GB/s = algorithmic bytes / mean CUDA-event time; frac = GB/s / measured copy bandwidth."""
    from segquant_b200 import _lib as L
    from segquant_b200 import ops
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    R, K = args.kernel_rows, 12288
    peaks = load_peaks()
    hbm = peaks.get("hbm_gbs") or 6650.0
    g = torch.Generator().manual_seed(11)
    x32 = torch.randn(R, K, generator=g).to(dev)
    x16 = x32.to(torch.bfloat16)
    bounds = ops.uniform_bounds(K, 4)
    sx = torch.full((4,), 30.0, device=dev)
    sxn = torch.full((4,), 60.0, device=dev)
    wq8 = torch.empty((R, K), dtype=torch.uint8, device=dev)
    wq4 = torch.empty(R * K // 2, dtype=torch.uint8, device=dev)
    sw_row = (127.0 / x16.float().abs().amax(-1)).contiguous()
    sw_grp = (7.0 / x16.float().view(R, K // 128, 128).abs().amax(-1)).contiguous()
    ops.quantize_weight(x16, wq4, sw_grp, L.SQ_Q_INT4, group_size=128)
    xn = x16.view(1, R * K // 1536, 1536)
    yn, on = torch.randn_like(xn), torch.empty_like(xn)
    mod = (torch.randn(1, 2 * 1536, generator=g) * 0.3).to(torch.bfloat16).to(dev)
    smooth = (torch.rand(K, generator=g) + 0.5).to(dev)
    cases = [
        ("act_quant bf16 -> int8, 4 segments", lambda: ops.quantize_act(x16, bounds, sx, None, L.SQ_Q_INT8), R * K * 3),
        ("act_quant bf16 -> e4m3 DualScale", lambda: ops.quantize_act(x16, bounds, sx, sxn, L.SQ_Q_E4M3), R * K * 4),
        ("act_quant GELU(bf16) -> int8 DualScale", lambda: ops.quantize_act(x16, bounds, sx, sxn, L.SQ_Q_INT8, pre_act="gelu_tanh"), R * K * 4),
        ("act_quant fp32 -> int8, 4 segments", lambda: ops.quantize_act(x32, bounds, sx, None, L.SQ_Q_INT8), R * K * 5),
        ("act_quant_dynamic bf16 -> int8 per token", lambda: ops.quantize_act_dynamic(x16, [0, K], L.SQ_Q_INT8), R * K * 3 + R * 4),
        ("act_quant_dynamic bf16 -> int8 per token, rows of 3072", lambda: ops.quantize_act_dynamic(x16.view(-1, 3072), [0, 3072], L.SQ_Q_INT8), R * K * 3 + R * 16),
        ("act_quant_dynamic bf16 / smooth -> int8 per token", lambda: ops.quantize_act_dynamic(x16, [0, K], L.SQ_Q_INT8, smooth=smooth), R * K * 3 + R * 4),
        ("weight_quant bf16 -> int8 per row", lambda: ops.quantize_weight(x16, wq8, sw_row, L.SQ_Q_INT8), R * K * 3),
        ("weight_quant bf16 -> packed int4, groups of 128", lambda: ops.quantize_weight(x16, wq4, sw_grp, L.SQ_Q_INT4, group_size=128),
         R * K * 2.5 + R * K // 128 * 4),
        ("unpack_int4", lambda: ops.unpack_int4(wq4), R * K * 1.5),
        ("gated_residual bf16 rows of 1536 (x + gate * y)", lambda: ops.gated_residual(xn, mod[:, :1536], yn, out=on), R * K * 6),
        # the same bytes seen as rows of 1536 (a DiT hidden size): LayerNorm + modulation + quantise in one pass
        ("norm_quant bf16 rows of 1536 -> int8, modulated", lambda: ops.norm_quantize_act(xn, [0, 1536], sx[:1], None, L.SQ_Q_INT8, shift=mod[:, :1536], scale=mod[:, 1536:]),
         R * K * 3),
        ("norm_quant bf16 rows of 1536 -> e4m3 DualScale, modulated",
         lambda: ops.norm_quantize_act(xn, [0, 1536], sx[:1], sxn[:1], L.SQ_Q_E4M3, shift=mod[:, :1536], scale=mod[:, 1536:]), R * K * 4),
    ]
    rows = []
    for name, fn, nbytes in cases:
        ms = timed(fn, args.steps, warmup=max(args.warmup, 3))
        rows.append({"kernel": name, "ms": ms, "gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / hbm, "bytes": nbytes})
    print(json.dumps({"metric": "hbm_kernel_gbs", "unit": "GB/s", "n_gpus": 1, "higher_is_better": True, "data": "synthetic",
                      "value": max(r["gbs"] for r in rows), "peak": hbm, "peak_source": "measured" if peaks.get("hbm_gbs") else "fallback",
                      "config": {"workload": f"HBM-bound kernels on [{R}, {K}] tensors ({R * K * 2 / 1e6:.0f} MB bf16 > 126 MB L2)",
                                 "steps": args.steps}, "kernels": rows, "device_status": ops.device_status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="layer", choices=["layer", "configs", "mmdit", "sweep", "kernels"],
                    help="layer (default, the headline line), configs (only the per-configuration entries of that line), mmdit "
                         "(synthetic denoise step), sweep (GEMM sweep), kernels (the HBM-bound quantise / unpack kernels against "
                         "the measured copy bandwidth)")
    ap.add_argument("--configs", default="all", choices=["all", "gpu", "none"],
                    help="layer at N = 1: also measure the other BASELINE configurations (all), without their CPU baselines (gpu), or not at all (none)")
    ap.add_argument("--quick", action="store_true",
                    help="layer: only the timed headline loop (no sustained leg, one end-to-end step, no configs, no CPU baseline): "
                         "what the ncu captures of the headline kernels run")
    ap.add_argument("--exchange", default="auto", choices=["auto", "push", "fused", "nccl"], help="layer at N > 1: how output column blocks are exchanged")
    ap.add_argument("--out-proj-segments", type=int, default=1, help="mmdit: K-segments of the attention output projections (1 or 24)")
    ap.add_argument("--mmdit-batch", type=int, default=0, help="mmdit: batch per GPU (default 2 on one GPU, 16 / N on N)")
    ap.add_argument("--no-graph", action="store_true", help="mmdit: launch every kernel from Python instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu", action="store_true", help="mmdit: skip the CPU baseline (one fake-quant block on the host cores)")
    ap.add_argument("--sweep-m", default="256,1024,4096,16384")
    ap.add_argument("--sweep-iters", type=int, default=10)
    ap.add_argument("--fused-gather", action="store_true", help="sweep at N > 1: accepted for old command lines; the symmetric-memory "
                                                               "exchanges are timed unless --no-symmetric is given")
    ap.add_argument("--no-symmetric", action="store_true",
                    help="sweep at N > 1: time only the NCCL all-gather, not the exchanges through symmetric memory (fused epilogue stores, block push)")
    ap.add_argument("--no-check", action="store_true", help="sweep: skip the per-point check against the CPU oracle")
    ap.add_argument("--sweep-nk", default="", help="sweep: comma list of NxK pairs (default: the seven shapes of config[4])")
    ap.add_argument("--sweep-modes", default="int8,fp8,w4a8")
    ap.add_argument("--sweep-segs", default="1,2,4,8")
    ap.add_argument("--sweep-w4-group", type=int, default=128, help="sweep: weight-scale group size of the W4A8 points (0 = per channel)")
    ap.add_argument("--kernel-rows", type=int, default=16384, help="kernels: rows of the [rows, 12288] tensors the HBM-bound kernels run on")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "mmdit":
        run_mmdit(args)
    elif args.workload == "sweep":
        run_sweep(args)
    elif args.workload == "kernels":
        run_kernels(args)
    elif args.workload == "configs":
        run_configs(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
