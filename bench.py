#!/usr/bin/env python
"""Benchmark of the real-quantized segmented linear path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the metric is quoted on): the DualScale W8A8 FP8-e4m3 MLP
down-projection -- X = GELU(Z), Z bf16 [4096, 6144] ~ N(0,1); W bf16 [1536, 6144] ~ N(0, 0.02) with
per-output-channel e4m3 scales; bias ~ N(0, 0.01); seed 1.  Synthetic data, random-init weights.
One step = one layer forward on one batch: activation quantise (positive / negative split) +
dual tcgen05 GEMM + scale / bias / bf16-cast epilogue.

Prints ONE JSON line (rank 0).  `value` is useful TOPS = 2*M*N*K*ranks / step time with inputs
resident in HBM; `e2e` is the same through SegmentLinear.forward with pinned HOST input and a
device->host read of the output inside the timed region.  With N > 1 every rank runs its own
batch (batch-data-parallel, no collective on the data path: weak scaling); the column-sharded
variant with an NCCL all-gather of output slices is timed too and reported under "sharded".

`--impl reference` times the reference's CPU path for the same layer: the fake-quant
SegmentLinear forward restated in oracle/fake_path.py with torch CPU kernels on all host
cores, on a bounded row sample.
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

M, K, N = 4096, 6144, 1536
SEED = 1
ROTATE = 4            # independent layer instances cycled through so that every step's operands come from HBM
CPU_SAMPLE_ROWS = 1024


def make_inputs(seed, m=M, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(m, K, generator=g, dtype=torch.float32).to(torch.bfloat16)
    x = torch.nn.functional.gelu(z.float()).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    b = (torch.randn(N, generator=g, dtype=torch.float32) * 0.01).to(torch.bfloat16)
    return x.to(device), w.to(device), b.to(device)


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
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()   # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(int(s[1]) for s in self.samples if s[1].isdigit())
        mx = [int(s[2]) for s in self.samples if s[2].isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            for name, v in zip(names, s[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# CPU baseline (the reference's fake-quant path, restated)
# ---------------------------------------------------------------------------------------------
def cpu_baseline(steps=3, warmup=1, rows=CPU_SAMPLE_ROWS):
    from oracle import fake_path as F
    torch.set_num_threads(os.cpu_count() or 1)
    x, w, b = make_inputs(SEED, m=rows)
    x, w, b = x.float(), w.float(), b.float()     # bf16 tensors up-cast: the reference's fp32 path
    w_fake, _ = F.fake_weight_fp8(w)
    sp, sn = F.dual_scales(x, 448.0, 448.0)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        F.seg_linear_fake(x.clone(), w_fake, b, [0, K], act="fp8", sx_pos=[sp], sx_neg=[sn])
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    t = sum(times) / len(times)
    return {"value": 2.0 * rows * N * K / t / 1e12, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"first {rows} of {M} rows of the same layer, fp32 fake-quant forward (quantise-dequantise + matmul + bias), "
                      f"mean of {steps} runs after {warmup} warm-up", "ms_per_step": t * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb = cpu_baseline(steps=max(1, args.steps), warmup=max(1, min(args.warmup, 3)))
    line = {
        "impl": "reference", "metric": "seglinear_gemm_tops", "value": cb["value"], "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config[1]: DualScale W8A8 FP8-e4m3 down-projection, M=4096 K=6144 N=1536, seed 1",
                   "note": "reference's own CPU path (fake-quant SegmentLinear forward) on host cores"},
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def build_layer(x, w, b, device):
    from segquant_b200.layers.SegmentLinear import SegmentLinear
    lin = SegmentLinear(K, N, bias=True, seg_mode="weight", chunks=1, custom_weight_tensor=w, custom_bias_tensor=b,
                        input_quant_type="fpe4m3", weight_quant_type="fpe4m3",
                        input_quant_args={"real_quant": True, "axis": None, "dual_scale": True},
                        weight_quant_args={"real_quant": True, "axis": 1},
                        opt_type="default", opt_kwargs={}, calib_type="amax", calib_kwargs={}, device=device)
    lin.calibrate(x)
    lin.finish_calibrate()
    return lin


def run_ours(args):
    import torch.distributed as dist
    from segquant_b200 import _lib as L
    from segquant_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this library has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L.load()

    # ---- ROTATE independent layer instances (different seeds per rank and slot)
    layers, xs = [], []
    for r in range(ROTATE):
        x, w, b = make_inputs(SEED + 1000 * rank + r if (rank or r) else SEED, device=dev)
        layers.append(build_layer(x, w, b, dev))
        xs.append(x)
    torch.cuda.synchronize()

    # pre-extract the fused-call arguments so the timed region is exactly the two kernels
    fused = []
    for lin in layers:
        lin.optimizer._build_fused()
        fused.append(lin.optimizer._fused)
    kind, a_kind, _ = ops.KERNELS["Wfpe4m3Afpe4m3"]
    xq = [torch.empty((1, M, K), dtype=torch.uint8, device=dev) for _ in range(ROTATE)]
    xqn = [torch.empty((1, M, K), dtype=torch.uint8, device=dev) for _ in range(ROTATE)]
    ys = [torch.empty((1, M, N), dtype=torch.bfloat16, device=dev) for _ in range(ROTATE)]

    def step(i, ev=None):
        r = i % ROTATE
        f = fused[r]
        if ev is not None:
            ev[2].record()
        ops.quantize_act(xs[r], f["bounds"], f["sx"], f["sx_neg"], a_kind, out=xq[r], out_neg=xqn[r])
        if ev is not None:
            ev[0].record()
        ops.gemm(kind, xq[r], f["wq"], N, f["bounds"], f["sx"], f["sw"], xq_neg=xqn[r], sx_neg=f["sx_neg"],
                 sw_strides=f["sw_strides"], bias=layers[r].bias_data, out_dtype=torch.bfloat16, out=ys[r])
        if ev is not None:
            ev[1].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    launches0 = ops.launch_count
    gemm_events = [tuple(torch.cuda.Event(enable_timing=True) for _ in range(3)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i, gemm_events[i])
    e1.record()
    barrier()
    launches = ops.launch_count - launches0
    ms_total = e0.elapsed_time(e1)
    gemm_ms = sum(a.elapsed_time(b) for a, b, _ in gemm_events) / args.steps
    quant_ms = sum(c.elapsed_time(a) for a, _, c in gemm_events) / args.steps
    t = torch.tensor([ms_total, gemm_ms, quant_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t[0].item() / args.steps
    gemm_ms = t[1].item()
    quant_ms = t[2].item()

    # ---- end to end through the public layer API with host buffers
    host_x = [x.cpu().pin_memory() for x in xs]
    host_y = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()

    # A user streaming batches through the layer: host->device copy of step i+1, the layer forward of step i and the
    # device->host read of step i-1 run on three streams with double-buffered device tensors, ordered by events.  Every
    # step's input copy and result read are inside the timed region.
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    x_dev = [torch.empty((M, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    y_dev = [torch.empty((1, M, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        r, b = i % ROTATE, i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[b])              # the forward two steps ago has consumed x_dev[b]
            x_dev[b].copy_(host_x[r], non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_cmp):
            s_cmp.wait_event(ev_in[b])
            s_cmp.wait_event(ev_out[b])             # y_dev[b] has been read back
            layers[r](x_dev[b].unsqueeze(0), out=y_dev[b])
            ev_cmp[b].record(s_cmp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[b])
            host_y.copy_(y_dev[b][0], non_blocking=True)
            ev_out[b].record(s_out)

    def e2e_join():
        cur = torch.cuda.current_stream()
        for st_ in (s_in, s_cmp, s_out):
            cur.wait_stream(st_)

    for st_ in (s_in, s_cmp, s_out):
        st_.wait_stream(torch.cuda.current_stream())
    for i in range(4):
        e2e_step(i)
    e2e_join()
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for st_ in (s_in, s_cmp, s_out):
        st_.wait_stream(torch.cuda.current_stream())
    for i in range(args.steps):
        e2e_step(i)
    e2e_join()
    e3.record()
    barrier()
    t2 = torch.tensor([e2.elapsed_time(e3)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms = t2.item() / args.steps
    clocks = sampler.stop() if rank == 0 else None

    # ---- column-sharded variant (N split over ranks, all-gather of output slices)
    sharded = None
    if world > 1 and N % world == 0:
        from segquant_b200.sharded import ColumnShardedSegLinear
        x0, w0, b0 = make_inputs(SEED, device=dev)
        cs = ColumnShardedSegLinear.from_full(x0, w0, b0, rank, world, kernel_type="Wfpe4m3Afpe4m3", dual_scale=True)
        for _ in range(3):
            cs.forward(x0)
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            cs.forward(x0)
        s1.record()
        barrier()
        ts = torch.tensor([s0.elapsed_time(s1)], dtype=torch.float64, device=dev)
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        sh_ms = ts.item() / args.steps
        sharded = {"ms_per_step": sh_ms, "tops": 2.0 * M * N * K / sh_ms / 1e9, "scaling": "strong",
                   "what": f"same layer, N={N} split into {world} column slices, NCCL all-gather of [M, N/{world}] bf16 slices"}
        # fused form: the GEMM epilogue stores every tile into all ranks' [M, N] buffers (symmetric memory), no gather kernel
        try:
            ok_local = 1
            try:
                cs.enable_fused_gather(M)
            except Exception as e:      # all ranks must agree before anyone enters the fused collectives
                ok_local, err = 0, e
            okt = torch.tensor([ok_local], device=dev)
            dist.all_reduce(okt, op=dist.ReduceOp.MIN)
            if not okt.item():
                raise RuntimeError(f"symmetric memory set-up failed on some rank: {err if not ok_local else 'peer'}")
            ref_full = cs.forward(x0)
            for _ in range(3):
                y_f = cs.forward_fused(x0)
            barrier()
            same = torch.tensor([int(torch.equal(y_f, ref_full))], device=dev)
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            for _ in range(args.steps):
                cs.forward_fused(x0)
            f1.record()
            barrier()
            tf = torch.tensor([f0.elapsed_time(f1)], dtype=torch.float64, device=dev)
            dist.all_reduce(tf, op=dist.ReduceOp.MAX)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            sharded["fused_gather_ms_per_step"] = tf.item() / args.steps
            sharded["fused_equals_allgather"] = bool(same.item())
        except Exception as e:   # symmetric memory unavailable on this box: the NCCL numbers above stand
            sharded["fused_gather_error"] = f"{type(e).__name__}: {e}"[:200]

    status = ops.device_status()
    if rank == 0:
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except OSError:
            pass
        bf16 = peaks.get("bf16_tflops")
        peak = 2.0 * bf16 if bf16 else 2.0 * 1590.0
        issued_tflop = 4.0 * M * N * K / 1e12          # DualScale: two MMAs per K step
        achieved = issued_tflop / (gemm_ms / 1e3)
        cb = cpu_baseline()
        line = {
            "metric": "seglinear_gemm_tops", "value": 2.0 * M * N * K * world / ms_step / 1e9, "unit": "TOPS",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": "config[1]: DualScale W8A8 FP8-e4m3 down-projection, M=4096 K=6144 N=1536 per GPU, seed 1",
                       "ops_counted": "useful 2*M*N*K (the kernel issues 4*M*N*K: positive and negative activation tiles)",
                       "cache": f"{ROTATE} independent layer instances cycled (operands {ROTATE * (M * K * 4 + N * K + M * N * 2) / 1e6:.0f} MB > 126 MB L2)",
                       "parallelism": f"dp{world}"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload
                         # (one ncu capture; 65.6 MB against 72.3 MB of algorithmic operand + output bytes)
                         "traffic": 65.6e6, "traffic_unit": "bytes per launch (ncu)",
                         "kernel": "seg_gemm2_kernel<F8, dual, KSUB=2>", "kernel_ms": gemm_ms,
                         "note": ("achieved = issued 4*M*N*K per launch / mean launch time (CUDA events on the launch stream); "
                                  "peak = 2 x measured bf16 burst (of measured)" if bf16 else
                                  "achieved = issued 4*M*N*K per launch / mean launch time; peak = 2 x 1.59 PFLOP/s (of fallback)")},
            "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": 2.0 * M * N * K * world / e2e_ms / 1e9, "unit": "TOPS", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                    "mode": "SegmentLinear.forward(x, out=) fed from pinned host memory; copy-in, forward and read-back of "
                            "consecutive steps overlap on three streams (double-buffered)"},
            "kernels": {"act_quant_ms": quant_ms, "act_quant_gbs": M * K * 4 / quant_ms / 1e6,
                        "act_quant_note": "algorithmic bytes M*K*(2 in + 2 out) per launch / mean CUDA-event time",
                        "seg_gemm_ms": gemm_ms},
            "gpu_launches": launches, "clocks": clocks, "device_status": status,
        }
        if sharded:
            line["sharded"] = sharded
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# other BASELINE workloads (not the default line): synthetic MMDiT denoise step, GEMM sweep
# ---------------------------------------------------------------------------------------------
def _dist_setup():
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return dist, world, rank, dev


def run_mmdit(args):
    """config[3]: 24-block SD3.5-medium-like MMDiT, every linear W8A8 INT8 SegLinear, attention / norms bf16.
    Batch 2 on one GPU; batch 16 split over 2 / 4 / 8 GPUs (replicas, no collective inside the step)."""
    from segquant_b200 import ops
    from segquant_b200.mmdit import GraphedStep, SyntheticMMDiT, synthetic_inputs
    dist, world, rank, dev = _dist_setup()
    batch = 2 if world == 1 else 16 // world
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
    clocks = sampler.stop() if rank == 0 else None
    status = ops.device_status()
    if rank == 0:
        lin_ops = eager.linear_ops(batch)
        tokens = eager.img_tokens + eager.txt_tokens
        attn_flops = 24 * batch * 4 * tokens * tokens * eager.hidden
        line = {
            "metric": "mmdit_denoise_step_ms", "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": False,
            "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "int8 linears, bf16 attention", "data": "synthetic",
            "config": {"workload": f"config[3]: synthetic MMDiT, 24 joint blocks, hidden 1536, 4096+333 tokens, batch {batch} per GPU "
                                   f"({batch * world} total), attention output projections with {args.out_proj_segments} K-segment(s)",
                       "launch": "eager" if args.no_graph else "one CUDA graph per step", "parallelism": f"dp{world} replicas"},
            "linear_tops": lin_ops / ms / 1e9, "linear_ops_per_step": lin_ops, "attention_flops_per_step": attn_flops,
            "e2e": {"value": t2.item(), "unit": "ms", "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in host_in),
                    "d2h_bytes_per_step": host_out.numel() * host_out.element_size()},
            "gpu_launches": launches, "clocks": clocks, "device_status": status,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


SWEEP_NK = [(1536, 1536), (6144, 1536), (1536, 6144), (9216, 3072), (12288, 3072), (3072, 12288), (1280, 5120)]


def run_sweep(args):
    """config[4]: M x (N, K) x {INT8, FP8, W4A8 g=128} x segments {1,2,4,8}; each point column-sharded over the
    ranks with an NCCL all-gather of the output slices.  Prints one JSON line holding every point."""
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
    for (N, K) in nks:
        if N % world:
            continue
        lo, hi = shard_range(N, world, rank)
        n_loc = hi - lo
        full = peers = flag = None
        if world > 1 and args.fused_gather:
            # every rank's [M, N] result buffer, mapped into all processes: the GEMM epilogue stores tiles to all of them
            import torch.distributed._symmetric_memory as symm
            full = symm.empty((max(Ms), N), dtype=torch.bfloat16, device=dev)
            handle = symm.rendezvous(full, dist.group.WORLD)
            peers = [int(p_) for r_, p_ in enumerate(handle.buffer_ptrs) if r_ != rank]
            flag = torch.zeros(1, dtype=torch.int32, device=dev)
        w = (torch.randn(n_loc, K, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        for name, ktype, wkind, group in modes:
            qmax = {L.SQ_Q_INT8: 127.0, L.SQ_Q_E4M3: 448.0, L.SQ_Q_INT4: 7.0}[wkind]
            if group:
                sw = (qmax / w.float().view(n_loc, K // group, group).abs().amax(-1)).contiguous()
                wq = torch.empty(n_loc * K // 2, dtype=torch.uint8, device=dev)
                ops.quantize_weight(w, wq, sw, wkind, group_size=group)
                wq3, strides = wq.view(1, n_loc, K // 2), (0, 0, 1, K // group)
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
                    scale = torch.exp(torch.empty(S).uniform_(-1.386, 3.466, generator=g))   # log-uniform in [0.25, 32]
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
                    ms_fused, fused_ok = None, None
                    if full is not None:
                        def fwd_fused():
                            ops.seg_linear(ktype, x.unsqueeze(0), wq3, n_loc, bounds, sx, sw, group_size=group, sw_strides=strides,
                                           out=full[:M, lo:hi].unsqueeze(0), peer_outputs=(peers, N, lo))
                            dist.all_reduce(flag)      # stream-ordered: every rank's kernel is complete after it
                        for _ in range(2):
                            fwd_fused()
                        torch.cuda.synchronize()
                        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        f0.record()
                        for _ in range(it):
                            fwd_fused()
                        f1.record()
                        torch.cuda.synchronize()
                        tf = torch.tensor([f0.elapsed_time(f1) / it], dtype=torch.float64, device=dev)
                        dist.all_reduce(tf, op=dist.ReduceOp.MAX)
                        ms_fused = tf.item()
                        same = torch.tensor([int(torch.equal(full[:M], gathered.permute(1, 0, 2).reshape(M, N)))], device=dev)
                        dist.all_reduce(same, op=dist.ReduceOp.MIN)
                        fused_ok = bool(same.item())
                    t = torch.tensor([e[0].elapsed_time(e[1]) / it, e[1].elapsed_time(e[2]) / it], dtype=torch.float64, device=dev)
                    if world > 1:
                        dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    ms_c, ms_t = t.tolist()
                    points.append({"mode": name, "M": M, "N": N, "K": K, "S": S, "layer_ms": ms_c, "layer_tops": 2.0 * M * N * K / ms_c / 1e9,
                                   "with_allgather_ms": ms_t if world > 1 else None, "with_fused_gather_ms": ms_fused,
                                   "fused_equals_allgather": fused_ok})
    status = ops.device_status()
    if rank == 0:
        best = {m: max((p["layer_tops"] for p in points if p["mode"] == m), default=0.0) for m in ("int8", "fp8", "w4a8")}
        print(json.dumps({"metric": "seglinear_gemm_tops_sweep", "unit": "TOPS", "n_gpus": world, "higher_is_better": True,
                          "scaling": "strong", "data": "synthetic", "value": max(best.values()), "best_tops": best,
                          "config": {"workload": "config[4]: GEMM sweep, layer = activation quantise + GEMM + epilogue, bf16 in/out, "
                                                 "N column-sharded over the ranks", "iters": args.sweep_iters},
                          "device_status": status, "points": points}), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
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
    cases = [
        ("act_quant bf16 -> int8, 4 segments", lambda: ops.quantize_act(x16, bounds, sx, None, L.SQ_Q_INT8), R * K * 3),
        ("act_quant bf16 -> e4m3 DualScale", lambda: ops.quantize_act(x16, bounds, sx, sxn, L.SQ_Q_E4M3), R * K * 4),
        ("act_quant GELU(bf16) -> int8 DualScale", lambda: ops.quantize_act(x16, bounds, sx, sxn, L.SQ_Q_INT8, pre_act="gelu_tanh"), R * K * 4),
        ("act_quant fp32 -> int8, 4 segments", lambda: ops.quantize_act(x32, bounds, sx, None, L.SQ_Q_INT8), R * K * 5),
        ("act_quant_dynamic bf16 -> int8 per token", lambda: ops.quantize_act_dynamic(x16, [0, K], L.SQ_Q_INT8), R * K * 3 + R * 4),
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
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        rows.append({"kernel": name, "ms": ms, "gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / hbm, "bytes": nbytes})
    print(json.dumps({"metric": "hbm_kernel_gbs", "unit": "GB/s", "n_gpus": 1, "higher_is_better": True, "data": "synthetic",
                      "value": max(r["gbs"] for r in rows), "peak": hbm, "peak_source": "measured" if peaks.get("hbm_gbs") else "fallback",
                      "config": {"workload": f"HBM-bound kernels on [{R}, {K}] tensors ({R * K * 2 / 1e6:.0f} MB bf16 > 126 MB L2)",
                                 "steps": args.steps}, "kernels": rows, "device_status": ops.device_status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="layer", choices=["layer", "mmdit", "sweep", "kernels"],
                    help="layer (default, the headline line), mmdit (synthetic denoise step), sweep (GEMM sweep), "
                         "kernels (the HBM-bound quantise / unpack kernels against the measured copy bandwidth)")
    ap.add_argument("--out-proj-segments", type=int, default=1, help="mmdit: K-segments of the attention output projections (1 or 24)")
    ap.add_argument("--no-graph", action="store_true", help="mmdit: launch every kernel from Python instead of replaying a CUDA graph")
    ap.add_argument("--sweep-m", default="256,1024,4096,16384")
    ap.add_argument("--sweep-iters", type=int, default=10)
    ap.add_argument("--fused-gather", action="store_true",
                    help="sweep at N > 1: also time the fused form (epilogue stores every tile into all ranks' buffers over NVLink)")
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
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
