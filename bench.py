#!/usr/bin/env python
"""MoE-layer forward benchmark (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c2]

A step is one forward pass of the layer over one batch of synthetic tokens.
  N = 1   "c2": 4096 tokens (8 x 512), d=1024, h=4096, 8 SwiGLU experts, top-2, bf16.
  N > 1   "c5": expert parallel, 64 experts sharded over the ranks, d=4096, h=14336, top-2, bf16,
          8192 tokens per rank (weak scaling); launched by torchrun, one rank per GPU.
`value` is tokens/s of the whole job with inputs resident in HBM; `e2e` is the same metric with
the step's tokens copied host->device and its output copied device->host inside the timed
region. `--impl reference` times the CPU restatement of the reference's PYTORCH path
(oracle/moe_oracle.py) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: tokens (per rank), d, h, o, E (total), k
    "c2": dict(tokens=4096, batch=8, seq=512, d=1024, h=4096, o=1024, E=8, k=2, fp8=False),
    "c3": dict(tokens=16384, batch=32, seq=512, d=4096, h=14336, o=4096, E=8, k=2, fp8=True),
    "c4": dict(tokens=8192, batch=16, seq=512, d=2048, h=8192, o=2048, E=64, k=8, fp8=False, zipf=1.2),
    "c5": dict(tokens=8192, batch=16, seq=512, d=4096, h=14336, o=4096, E=64, k=2, fp8=False),
}


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel (up-projection
# grouped GEMM), from the ncu capture summarised in profiles/grouped_gemm_c2.md. Only the
# configuration that was captured has a figure; the others report null.
NCU_TRAFFIC_BYTES = {"c2": 151.15e6 + 46.79e6}


def layer_flops(c, tokens):
    A = tokens * c["k"]
    return 2 * tokens * c["d"] * c["E"] + 4 * A * c["d"] * c["h"] + 2 * A * c["h"] * c["o"]


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Polls nvidia-smi during the timed region (clocks, power, throttle reasons)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [l for t, l in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for _, l in self.lines]
        for l in rows:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def make_inputs(c, rank, device, dtype=torch.bfloat16):
    """Seeded synthetic data: x ~ N(0,1) (per-rank seed), weights / gate ~ N(0, 0.02) (shared seed)."""
    g = torch.Generator().manual_seed(1234 + rank)
    x = torch.randn(c["batch"], c["seq"], c["d"], generator=g)
    if c.get("fp8"):
        rows = torch.randperm(c["tokens"], generator=g)[: c["tokens"] // 100]
        x.view(-1, c["d"])[rows] *= 50.0
    return x.to(dtype)


def build_layer(c, device, e_local=None, e_first=0):
    import fast_moe_b200 as fm

    torch.manual_seed(0)
    layer = fm.SwiGLUFastMoELayer(c["d"], c["h"], c["o"], c["E"], dtype=torch.bfloat16, fp8=bool(c.get("fp8")))
    with torch.no_grad():
        layer.gate.gate.weight.normal_(0, 0.02)
        layer.gate.gate.bias.zero_()
        if c.get("zipf"):
            # biased router: expert loads follow Zipf(s) over a seeded permutation of the experts
            g = torch.Generator().manual_seed(7)
            ranks = torch.randperm(c["E"], generator=g).float() + 1.0
            p = ranks.pow(-c["zipf"])
            layer.gate.gate.bias.copy_((p / p.sum()).log())
    return layer.to(device)


def graph_kernel_ms(fn, device, n=10):
    """Device time of one call of fn: n calls recorded in a CUDA graph, one replay timed with CUDA
    events on the launching stream (no host work between the launches)."""
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream(device).wait_stream(side)
    torch.cuda.synchronize(device)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(n):
            fn()
    g.replay()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) / n


def routing_sweep(c, device):
    """Gate + top-k and the counting sort alone at several token counts: device time per call from
    a CUDA graph of 20 calls, warm and with a 256 MB L2 flush before every call (the flush's own
    time, measured the same way, subtracted). Prints one JSON line."""
    import fast_moe_b200 as fm

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    g = torch.Generator().manual_seed(5)
    gw = (torch.randn(c["E"], c["d"], generator=g) * 0.02).to(device)
    gb = torch.zeros(c["E"], device=device)
    flush_ms = graph_kernel_ms(lambda: flush.zero_(), device, n=20)
    rows_out = []
    for tokens in (1024, 4096, 16384, 65536):
        x = torch.randn(tokens, c["d"], generator=g).to(torch.bfloat16).to(device)
        idx, _, _ = fm.gate_topk(x, gw, gb, c["k"])
        gate = lambda: fm.gate_topk(x, gw, gb, c["k"])
        sort = lambda: fm.route_metadata(idx, c["E"])
        cold = lambda fn: (lambda: (flush.zero_(), fn()))
        rows_out.append(dict(tokens=tokens,
                         gate_warm_us=1e3 * graph_kernel_ms(gate, device, n=20),
                         gate_cold_us=1e3 * (graph_kernel_ms(cold(gate), device, n=20) - flush_ms),
                         sort_warm_us=1e3 * graph_kernel_ms(sort, device, n=20),
                         sort_cold_us=1e3 * (graph_kernel_ms(cold(sort), device, n=20) - flush_ms)))
    # the HBM-bound kernels of the path at the benchmark shapes: algorithmic bytes / device time
    from fast_moe_b200.kernels import moe as ops
    from fast_moe_b200.kernels import moe_fp8 as ops_fp8

    peak = load_peaks().get("hbm_gbs")
    hbm = []

    def add(name, shape, fn, nbytes):
        ms = graph_kernel_ms(fn, device, n=10)
        hbm.append(dict(kernel=name, shape=shape, us=1e3 * ms, algorithmic_mb=nbytes / 1e6,
                        achieved_gbs=nbytes / ms / 1e6, frac_of_measured_hbm=(nbytes / ms / 1e6) / peak if peak else None))

    for shape, L, E, k, D in (("c2", 4096, 8, 2, 1024), ("c4", 8192, 64, 8, 2048), ("c5", 8192, 64, 2, 4096)):
        idx = torch.rand(L, E, generator=g).topk(k, dim=1).indices.to(device)
        meta = fm.route_metadata(idx, E)
        x = torch.randn(L, D, generator=g).to(torch.bfloat16).to(device)
        rows = torch.randn(L * k, D, generator=g).to(torch.bfloat16).to(device)
        w = torch.rand(L, k, generator=g).to(torch.bfloat16).to(device)
        add("gather_rows", shape, lambda: ops.gather_rows(x, meta.gate_index, k), 2 * L * k * D * 2)
        add("mul_merge_k_add", shape,
            lambda: ops.mul_merge_k_add(meta.token_index, meta.reverse_index, rows, weight=w, weight_index=meta.gate_index),
            (L * k * D + L * D) * 2)
    for shape, R, C in (("c3 tokens", 16384, 4096), ("c3 hidden", 32768, 14336)):
        a = torch.randn(R, C, generator=g).to(torch.bfloat16).to(device)
        add("rowwise_quant_fp8", shape, lambda: ops_fp8.rowwise_quant_fp8(a), R * C * 3 + 4 * R)
        del a
    print(json.dumps(dict(routing_sweep=rows_out, d=c["d"], E=c["E"], k=c["k"], hbm_kernels=hbm,
                          hbm_peak_gbs=peak)), flush=True)


def up_projection_ms(layer, x_dev, k, fp8):
    """The dominant kernel alone (gate/up grouped GEMM + SwiGLU epilogue on the expert-sorted rows
    of this batch's routing), timed as graph_kernel_ms does. The rows are gathered beforehand by
    the copy kernel, as the operator itself does at these sizes; the copy is not in this time."""
    from fast_moe_b200.kernels import moe as ops
    from fast_moe_b200.kernels import moe_fp8 as ops_fp8

    with torch.no_grad():
        x_flat = x_dev.reshape(-1, x_dev.shape[-1])
        _, meta = layer._route(x_flat, k)
        dt = x_flat.dtype
        if fp8:
            (wg, sg), (wu, su) = layer._q["w_gate"], layer._q["w_up"]
            xq, xs = ops_fp8.rowwise_quant_fp8(x_flat)
            xq = ops.gather_rows(xq, meta.gate_index, k)
            xs = ops.gather_rows(xs.view(-1, 1), meta.gate_index, k).view(-1)
            fn = lambda: ops_fp8.index_select_jagged_bmm_fp8_quantized(
                meta.offsets, None, xq, xs, wg, sg, None, out_dtype=dt, weight_p_q=wu, weight_p_scale=su)
        else:
            wg = layer._cast.get("wg", layer.w_gate, dt).permute(0, 2, 1)
            wu = layer._cast.get("wu", layer.w_up, dt).permute(0, 2, 1)
            xg = ops.gather_rows(x_flat, meta.gate_index, k)
            fn = lambda: ops.index_select_jagged_bmm_swiglu(0, meta.offsets, None, xg, wg, None, wu, None)
        return graph_kernel_ms(fn, x_dev.device)


def cpu_oracle_step(c, x_cpu, params, k):
    from oracle import moe_oracle as O

    return O.moe_layer_swiglu(x_cpu, params["gate_w"], params["gate_b"], params["w_gate"], params["w_up"],
                              params["w_down"], k)


def cpu_sample(c, tokens, seconds_per_step):
    """Bounded CPU sample of a config: (tokens, experts). Large layers keep the per-expert row
    count and the per-token FLOPs but use only a few of the experts (their fp32 weights would not
    even fit in host memory otherwise); then tokens are halved until a step fits the time budget
    at an assumed 0.2 TFLOP/s."""
    E = c["E"]
    e_s = E if c["d"] * c["h"] * E <= 4e8 else max(c["k"], 4)
    sample = max(256, tokens * e_s // E)
    cs = dict(c, E=e_s)
    while layer_flops(cs, sample) / 2e11 > seconds_per_step and sample > 256:
        sample //= 2
    return sample, e_s


def cpu_params(c, tokens, experts=None):
    g = torch.Generator().manual_seed(0)
    E, d, h, o = experts or c["E"], c["d"], c["h"], c["o"]
    return dict(
        gate_w=torch.randn(E, d, generator=g) * 0.02, gate_b=torch.zeros(E),
        w_gate=(torch.randn(E, h, d, generator=g) * 0.02).permute(0, 2, 1),
        w_up=(torch.randn(E, h, d, generator=g) * 0.02).permute(0, 2, 1),
        w_down=(torch.randn(E, o, h, generator=g) * 0.02).permute(0, 2, 1),
    )


def time_cpu_baseline(c, tokens, budget_s=20.0):
    """The CPU restatement of the reference's PYTORCH path on a bounded sample of the workload:
    the token count is scaled down until one forward takes a few seconds."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample, e_s = cpu_sample(c, tokens, budget_s / 4)
    p = cpu_params(c, sample, e_s)
    x = torch.randn(1, sample, c["d"], generator=torch.Generator().manual_seed(99))
    with torch.no_grad():
        cpu_oracle_step(c, x, p, c["k"])   # warm-up
        times = []
        t_all = time.perf_counter()
        while len(times) < 3 and time.perf_counter() - t_all < budget_s:
            t0 = time.perf_counter()
            cpu_oracle_step(c, x, p, c["k"])
            times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return dict(value=sample / t, unit="tokens/s", cores=cores, kind="port",
                sample=f"{sample} of {tokens} tokens over {e_s} of {c['E']} experts, fp32, torch CPU ({cores} threads), "
                       f"median of {len(times)} runs",
                seconds_per_run=t)


def time_ep_single_gpu(device, args):
    """c5 (64 experts, d=4096, h=14336, 8192 tokens) with every expert on this GPU."""
    from fast_moe_b200.modules.expert_parallel import ExpertParallelSwiGLUMoE

    c = CONFIGS["c5"]
    layer = ExpertParallelSwiGLUMoE(c["d"], c["h"], c["o"], c["E"], dtype=torch.bfloat16, device=device)
    x = make_inputs(c, 0, device).to(device)
    steps = max(3, min(args.steps, 10))
    for _ in range(3):
        layer(x, c["k"])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        layer(x, c["k"])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return dict(value=c["tokens"] / (ms * 1e-3), unit="tokens/s", ms_per_step=ms, steps=steps,
                layer_tflops=layer_flops(c, c["tokens"]) / (ms * 1e-3) / 1e12,
                workload=workload_config(c, "c5", 1)["workload"])


def run_reference(args, c, name):
    """Reference arm: the CPU restatement of the reference's PYTORCH path, all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    tokens = c["tokens"]
    sample, e_s = cpu_sample(c, tokens, 4.0)
    p = cpu_params(c, sample, e_s)
    x = torch.randn(1, sample, c["d"], generator=torch.Generator().manual_seed(99))
    with torch.no_grad():
        for _ in range(max(1, min(args.warmup, 3))):
            cpu_oracle_step(c, x, p, c["k"])
        t0 = time.perf_counter()
        for _ in range(args.steps):
            cpu_oracle_step(c, x, p, c["k"])
        dt = (time.perf_counter() - t0) / args.steps
    val = sample / dt
    sample_desc = (f"each step = {sample} of {tokens} tokens per rank over {e_s} of {c['E']} experts, fp32, "
                   f"torch CPU, {cores} threads")
    line = dict(
        impl="reference", metric="moe_layer_fwd_tokens_per_s", value=val, unit="tokens/s", n_gpus=args.gpus,
        steps=args.steps, warmup=args.warmup, ms_per_step=dt * 1e3, higher_is_better=True, scaling="weak",
        vs_baseline=None, dtype="f32", data="synthetic", config=workload_config(c, name, args.gpus),
        cpu_baseline=dict(value=val, unit="tokens/s", cores=cores, kind="port", sample=sample_desc),
        e2e=dict(value=val, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
    )
    print(json.dumps(line), flush=True)


def workload_config(c, name, n_gpus):
    return dict(
        workload=f"{name}: SwiGLU MoE layer forward, {c['tokens']} tokens/rank, d={c['d']}, h={c['h']}, "
                 f"E={c['E']}, top-{c['k']}" + (", fp8 e4m3 rowwise" if c.get("fp8") else ", bf16"),
        tokens_per_rank=c["tokens"], global_tokens=c["tokens"] * n_gpus, d=c["d"], h=c["h"], E=c["E"], k=c["k"],
        parallelism="single GPU" if n_gpus == 1 else f"expert parallel ep{n_gpus} ({c['E'] // n_gpus} experts/rank)",
        l2="working set (weights + activations) is larger than the 126 MB L2; no explicit flush",
    )


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ep-reference", action="store_true")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of a CUDA-graph replay")
    ap.add_argument("--routing-sweep", action="store_true",
                    help="only time the routing operators and the HBM-bound kernels alone (one JSON line)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    name = args.config or ("c2" if args.gpus == 1 else "c5")
    c = CONFIGS[name]
    if args.impl == "reference":
        run_reference(args, c, name)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the layer has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if args.routing_sweep:
        if rank == 0:
            routing_sweep(c, device)
        return
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)

    from fast_moe_b200 import _lib

    k = c["k"]
    x_host = make_inputs(c, rank, device).pin_memory()
    x_dev = x_host.to(device)
    if world > 1:
        from fast_moe_b200.modules.expert_parallel import ExpertParallelSwiGLUMoE

        torch.manual_seed(0)
        layer = ExpertParallelSwiGLUMoE(c["d"], c["h"], c["o"], c["E"], dtype=torch.bfloat16, device=device)
    else:
        layer = build_layer(c, device)
    if c.get("fp8"):
        layer.quantize_weights()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    # Single GPU: the forward is captured once as a CUDA graph and a step is one replay (same
    # kernels, one launch). The expert-parallel layer synchronises with the host for its split
    # sizes and runs eagerly. A second, eager pass with CUDA events around each stage gives the
    # per-kernel times the roofline figure uses.
    for _ in range(args.warmup):
        y = layer(x_dev, k)
    barrier()
    captured = None
    if world == 1 and not args.eager:
        from fast_moe_b200 import CapturedForward

        captured = CapturedForward(layer, x_dev, k)
        step = captured.replay
    else:
        step = lambda: layer(x_dev, k)
    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = _lib.kernel_launch_count()
    barrier()
    t_wall0 = time.perf_counter()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        y = step()
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    # eager pass with stage events (also what counts launches when the timed pass was a graph);
    # graph capture empties the allocator cache, so the eager path is warmed up again first
    for _ in range(3):
        layer(x_dev, k)
    barrier()
    timer = _lib.StageTimer()
    _lib.set_stage_timer(timer)
    launches_eager0 = _lib.kernel_launch_count()
    ee0, ee1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ee0.record()
    for _ in range(args.steps):
        layer(x_dev, k)
    ee1.record()
    barrier()
    t_wall1 = time.perf_counter()
    ms_eager = ee0.elapsed_time(ee1) / args.steps
    launches = _lib.kernel_launch_count() - launches_eager0   # kernels per K steps (the graph replays the same ones)
    _lib.set_stage_timer(None)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    stage_ms = {n: (tot / cnt) for n, (tot, cnt) in timer.totals_ms().items()}
    up_alone_ms = up_projection_ms(layer, x_dev, k, bool(c.get("fp8"))) if world == 1 else None
    status = _lib.device_status(device)

    # ---- end to end: host tokens in, host result out, every step, through the package's
    # streaming executor: every step copies its tokens from pinned host memory and its result
    # back to pinned host memory; the copies of neighbouring steps overlap the forward.
    from fast_moe_b200 import StreamingForward

    slots = 3
    pipe = StreamingForward(layer, x_dev, k, slots=slots, capture=captured is not None)
    y_hosts = [torch.empty((c["batch"], c["seq"], c["o"]), dtype=torch.bfloat16).pin_memory() for _ in range(slots)]
    y_host = y_hosts[0]
    for i in range(max(3, slots)):
        pipe.submit(x_host, y_hosts[i % slots])
    pipe.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        pipe.submit(x_host, y_hosts[i % slots])
    pipe.drain()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    e2e_check = float((y_hosts[(args.steps - 1) % slots].float() - y.detach().float().cpu().view_as(y_host)).abs().max())

    t = torch.tensor([ms_total, ms_e2e], device=device, dtype=torch.float64)
    stage_ms_ranks = None
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        stage_ms_ranks = [None] * world
        dist.all_gather_object(stage_ms_ranks, {n: round(v, 4) for n, v in stage_ms.items()})
    ms_total, ms_e2e = t.tolist()

    if rank == 0:
        peaks = load_peaks()
        ms_step = ms_total / args.steps
        tokens_total = c["tokens"] * world
        A = c["tokens"] * k
        # the dominant kernel's duration: alone, back to back in a graph (single GPU), else the
        # eager stage events (which include host launch gaps when the host is the slower side)
        up_ms = up_alone_ms if up_alone_ms is not None else stage_ms.get("up")
        up_flops = 4 * A * c["d"] * c["h"]
        # the up-projection kernel is timed alone between two events: burst peak is its yardstick
        peak_tf = peaks["bf16_tflops"] * (2.0 if c.get("fp8") else 1.0)
        roofline = None
        if up_ms:
            ach = up_flops / (up_ms * 1e-3) / 1e12
            roofline = dict(bound="tensor", kernel="grouped_gemm_kernel (gate/up GEMM + SwiGLU on expert-sorted rows)",
                            achieved=ach, peak=peak_tf, unit="TFLOP/s", frac=ach / peak_tf,
                            traffic=NCU_TRAFFIC_BYTES.get(name) if world == 1 else None,
                            algorithmic_bytes=(2 * c["E"] * c["d"] * c["h"] + A * c["d"] + A * c["h"]) * (1 if c.get("fp8") else 2),
                            peak_source=peaks["source"] + (" (2x bf16 burst for fp8)" if c.get("fp8") else " burst"),
                            flops_per_launch=up_flops, avg_launch_ms=up_ms,
                            timing="10 launches back to back in a CUDA graph, CUDA events" if up_alone_ms is not None
                            else "CUDA events around the eager launch")
        line = dict(
            metric="moe_layer_fwd_tokens_per_s", value=tokens_total / (ms_step * 1e-3), unit="tokens/s",
            n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms_step, higher_is_better=True,
            scaling="weak", vs_baseline=None, dtype="e4m3" if c.get("fp8") else "bf16", data="synthetic",
            config=workload_config(c, name, world),
            layer_tflops_per_gpu=layer_flops(c, c["tokens"]) / (ms_step * 1e-3) / 1e12,
            launch_mode="cuda graph replay" if captured is not None else "eager", ms_per_step_eager=ms_eager,
            stage_ms=stage_ms, stage_ms_per_rank=stage_ms_ranks, roofline=roofline, clocks=clocks, gpu_launches=int(launches),
            device_status=status,
            e2e=dict(value=tokens_total / (ms_e2e / args.steps * 1e-3), unit="tokens/s",
                     h2d_bytes_per_step=x_host.numel() * x_host.element_size(),
                     d2h_bytes_per_step=y_host.numel() * y_host.element_size(), ms_per_step=ms_e2e / args.steps,
                     mode="%d-slot pipeline: H2D, forward and D2H of consecutive steps overlap" % slots,
                     max_abs_diff_vs_resident=e2e_check),
        )
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = time_cpu_baseline(c, c["tokens"])
        if world == 1 and args.config is None and not args.no_ep_reference:
            # the per-rank workload of the multi-GPU runs (c5, expert parallel) on one GPU: the
            # denominator for weak-scaling efficiency of the N > 1 lines
            del layer, y
            torch.cuda.empty_cache()
            line["c5_ep_1gpu"] = time_ep_single_gpu(device, args)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
