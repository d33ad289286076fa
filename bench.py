#!/usr/bin/env python
"""MoE-layer forward benchmark (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c2]

A step is one forward pass of the layer over one batch of synthetic tokens.
  N = 1   "c2": 4096 tokens (8 x 512), d=1024, h=4096, 8 SwiGLU experts, top-2, bf16.
          The line also carries sub-records for "c3" (FP8 e4m3 rowwise, 16384 tokens, d=4096,
          h=14336), "c4" (Zipf-skewed routing over 64 experts, top-8) and "c5_ep_1gpu" (the
          per-rank workload of the multi-GPU runs with all 64 experts on one GPU), a `sustained`
          record (the same step replayed for at least a second) and a `parity` block.
  N > 1   "c5": expert parallel, 64 experts sharded over the ranks, d=4096, h=14336, top-2, bf16,
          8192 tokens per rank (weak scaling); launched by torchrun, one rank per GPU. Rank 0
          first times the per-rank workload alone on its GPU: `weak_scaling` holds that time, the
          efficiency t1 / tN and the compute / HBM bounds of both.
`value` is tokens/s of the whole job with inputs resident in HBM; `e2e` is the same metric with
the step's tokens copied host->device and its output copied device->host inside the timed
region. `parity` compares the benchmarked layer's output, outside the timed region, with the CPU
oracle: routing tensors bit for bit on the whole batch, outputs on a seeded sample of tokens.
`--impl reference` times the CPU restatement of the reference's PYTORCH path
(oracle/moe_oracle.py) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
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
    # Zipf(1.2) expert loads. With top-8 of 64 experts an expert can receive at most one row per
    # token, i.e. 1/8 of the assignments (not the 25 % a top-1 router could give it); the bias is
    # sharpened (x 1.5) so that the most loaded experts sit at that cap, a long tail of experts
    # receives a handful of rows and several receive none.
    "c4": dict(tokens=8192, batch=16, seq=512, d=2048, h=8192, o=2048, E=64, k=8, fp8=False, zipf=1.2,
               zipf_sharpen=1.5),
    "c5": dict(tokens=8192, batch=16, seq=512, d=4096, h=14336, o=4096, E=64, k=2, fp8=False),
}


def layer_flops(c, tokens):
    A = tokens * c["k"]
    return 2 * tokens * c["d"] * c["E"] + 4 * A * c["d"] * c["h"] + 2 * A * c["h"] * c["o"]


def layer_min_bytes(c, tokens, experts_local=None):
    """Weights read once + tokens in + result out + hidden written and read."""
    E = experts_local if experts_local is not None else c["E"]
    w = 1 if c.get("fp8") else 2
    A = tokens * c["k"]
    return E * (2 * c["d"] * c["h"] + c["h"] * c["o"]) * w + tokens * c["d"] * 2 + tokens * c["o"] * 2 + 2 * A * c["h"] * w


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def ncu_traffic(name):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, read
    from the committed ncu summary of that configuration (a line `traffic_bytes_per_launch:
    <bytes> ... commit <hash>` in profiles/grouped_gemm_<name>.md). None when there is no capture."""
    path = os.path.join(ROOT, "profiles", f"grouped_gemm_{name}.md")
    try:
        with open(path) as f:
            text = f.read()
    except OSError:
        return None, None
    m = re.search(r"traffic_bytes_per_launch:\s*([0-9.eE+]+)(?:.*?commit\s+([0-9a-f]{7,40}))?", text)
    if not m:
        return None, None
    return float(m.group(1)), m.group(2)


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

    def window(self, t0: float, t1: float):
        """Summary of the samples taken between two perf_counter times."""
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [l for t, l in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for _, l in self.lines]
        for l in rows:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                pw.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    power_w=statistics.median(pw) if pw else None, reasons=sorted(reasons), samples=len(sm))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        return self.window(t0, t1)


# ------------------------------------------------------------------------------------ workloads
def make_inputs(c, rank):
    """Seeded synthetic tokens [batch, seq, d] bf16 on the host: x ~ N(0,1) (per-rank seed); the FP8
    configuration scales 1 % of the rows by 50 to stress the per-row scales."""
    g = torch.Generator().manual_seed(1234 + rank)
    x = torch.randn(c["batch"], c["seq"], c["d"], generator=g)
    if c.get("fp8"):
        rows = torch.randperm(c["tokens"], generator=g)[: c["tokens"] // 100]
        x.view(-1, c["d"])[rows] *= 50.0
    return x.to(torch.bfloat16)


def zipf_gate_bias(E, s, sharpen=1.0, seed=7):
    """Router bias that makes expert loads follow Zipf(s) over a seeded permutation of the
    experts: log of the target probabilities, times `sharpen`."""
    g = torch.Generator().manual_seed(seed)
    ranks = torch.randperm(E, generator=g).float() + 1.0
    p = ranks.pow(-s)
    return (p / p.sum()).log() * sharpen


def build_layer(c, device):
    """SwiGLU layer of configuration c with seeded N(0, 0.02) weights, created on the device."""
    import fast_moe_b200 as fm

    torch.manual_seed(0)
    torch.cuda.manual_seed(0)
    with torch.device(device):
        layer = fm.SwiGLUFastMoELayer(c["d"], c["h"], c["o"], c["E"], dtype=torch.bfloat16, fp8=bool(c.get("fp8")))
    with torch.no_grad():
        layer.gate.gate.weight.normal_(0, 0.02)
        layer.gate.gate.bias.zero_()
        if c.get("zipf"):
            layer.gate.gate.bias.copy_(zipf_gate_bias(c["E"], c["zipf"], c.get("zipf_sharpen", 1.0)).to(device))
    if c.get("fp8"):
        layer.quantize_weights()
    return layer


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
    # the backward pass's layout and elementwise passes at the C2 shapes
    from fast_moe_b200.kernels import autograd as AG

    L, E, k, d_, h_ = 4096, 8, 2, 1024, 4096
    idx = torch.rand(L, E, generator=g).topk(k, dim=1).indices.to(device)
    meta = fm.route_metadata(idx, E)
    A = L * k
    hid = torch.randn(A, h_, generator=g).to(torch.bfloat16).to(device)
    hid2 = torch.randn(A, h_, generator=g).to(torch.bfloat16).to(device)
    dh = torch.randn(A, h_, generator=g).to(torch.bfloat16).to(device)
    kseg, padded = AG._padded_reduction(meta.offsets, E, torch.bfloat16, A)
    add("jagged_transpose_pad", f"c2 hidden {A} x {h_}", lambda: AG._transpose_pad(hid, meta.offsets, kseg, padded, E, A),
        2 * A * h_ * 2)
    da, db = torch.empty_like(hid), torch.empty_like(hid)
    add("activation_backward (SwiGLU)", f"c2 {A} x {h_}", lambda: AG.activation_backward(1, dh, hid, hid2, da, db), 5 * A * h_ * 2)
    add("jagged_colsum (d_bias)", f"c2 {A} x {h_}", lambda: AG.grad_bias(meta.offsets, dh, E, torch.bfloat16), A * h_ * 2)
    sc = torch.rand(L, k, generator=g).to(device)
    dy = torch.randn(L, d_, generator=g).to(torch.bfloat16).to(device)
    rows2 = torch.randn(A, d_, generator=g).to(torch.bfloat16).to(device)
    add("gather_scale_rows", f"c2 {A} x {d_}", lambda: AG.gather_scale_rows(dy, meta.token_index, 1, sc, meta.gate_index),
        (L + A) * d_ * 2)
    add("row_dot", f"c2 {A} x {d_}", lambda: AG.row_dot(rows2, dy, meta.token_index), (L + A) * d_ * 2)
    print(json.dumps(dict(routing_sweep=rows_out, d=c["d"], E=c["E"], k=c["k"], hbm_kernels=hbm,
                          hbm_peak_gbs=peak)), flush=True)


def layer_sweep(c, device):
    """The C2 layer (d, h, experts, top-k of configuration c) over a range of batch sizes: graph-replay
    forward time, tokens/s and layer TFLOP/s per token count. Prints one JSON line."""
    from fast_moe_b200 import CapturedForward

    layer = build_layer(c, device)
    rows = []
    g = torch.Generator().manual_seed(11)
    for tokens in (256, 1024, 4096, 16384, 65536, 262144):
        x = torch.randn(1, tokens, c["d"], generator=g).to(torch.bfloat16).to(device)
        for _ in range(3):
            layer(x, c["k"])
        cap = CapturedForward(layer, x, c["k"])
        for _ in range(3):
            cap.replay()
        ms = time_steps(cap.replay, 20, torch.cuda.synchronize)[0] / 20
        rows.append(dict(tokens=tokens, ms=ms, tokens_per_s=tokens / (ms * 1e-3),
                         layer_tflops=layer_flops(c, tokens) / (ms * 1e-3) / 1e12))
        del cap, x
        torch.cuda.empty_cache()
    print(json.dumps(dict(layer_sweep=rows, d=c["d"], h=c["h"], E=c["E"], k=c["k"], dtype="bf16")), flush=True)


def train_step_only(c, device, steps, warmup):
    """A training step (forward + backward, eager autograd) of the C2 SwiGLU layer and nothing else:
    the command the launch list of the backward pass is taken from. Prints one JSON line."""
    layer = build_layer(c, device)
    layer.autograd = True
    x = make_inputs(c, 0).to(device).requires_grad_(True)

    def step():
        for p_ in layer.parameters():
            p_.grad = None
        x.grad = None
        y_ = layer(x, c["k"])
        y_.backward(torch.ones_like(y_))

    for _ in range(warmup):
        step()
    ms = time_steps(step, steps, torch.cuda.synchronize)[0] / steps
    print(json.dumps(dict(train_step_ms_eager=ms, steps=steps, warmup=warmup, tokens=c["tokens"], d=c["d"], h=c["h"],
                          E=c["E"], k=c["k"], dtype="bf16")), flush=True)


def gemm_alone_ms(layer, x_dev, k, fp8):
    """The two grouped GEMMs alone on this batch's routing, each timed as graph_kernel_ms does:
    (gate/up GEMM + SwiGLU epilogue on the expert-sorted rows, down GEMM + fused combine). The
    rows are gathered beforehand by the copy kernel, as the operator itself does at these sizes;
    the copy is not in the first time. For k > 2 the layers use the two-kernel combine, so the
    second time is the down GEMM + the combine kernel."""
    from fast_moe_b200.kernels import moe as ops
    from fast_moe_b200.kernels import moe_fp8 as ops_fp8

    with torch.no_grad():
        x_flat = x_dev.reshape(-1, x_dev.shape[-1])
        score, meta = layer._route(x_flat, k)
        dt = x_flat.dtype
        fused = k <= 2
        if fp8:
            (wg, sg), (wu, su), (wd, sd) = layer._q["w_gate"], layer._q["w_up"], layer._q["w_down"]
            xq, xs = ops_fp8.rowwise_quant_fp8(x_flat)
            xq = ops.gather_rows(xq, meta.gate_index, k)
            xs = ops.gather_rows(xs.view(-1, 1), meta.gate_index, k).view(-1)
            up = lambda: ops_fp8.index_select_jagged_bmm_fp8_quantized(
                meta.offsets, None, xq, xs, wg, sg, None, out_dtype=dt, weight_p_q=wu, weight_p_scale=su)
            hq, hs = ops_fp8.rowwise_quant_fp8(up())
            down = lambda: ops_fp8.fp8_jagged_bmm_combine_quantized(
                meta.offsets, hq, hs, wd, sd, None, score, meta.gate_index, x_flat.shape[0], out_dtype=dt)
        else:
            wg = layer._cast.get("wg", layer.w_gate, dt).permute(0, 2, 1)
            wu = layer._cast.get("wu", layer.w_up, dt).permute(0, 2, 1)
            wd = layer._cast.get("wd", layer.w_down, dt).permute(0, 2, 1)
            xg = ops.gather_rows(x_flat, meta.gate_index, k)
            up = lambda: ops.index_select_jagged_bmm_swiglu(0, meta.offsets, None, xg, wg, None, wu, None)
            hidden = up()
            down = lambda: ops.silu_jagged_bmm_combine(
                0, meta.offsets, hidden, wd, None, meta.token_index, meta.reverse_index, gating_scores=score,
                gates_index=meta.gate_index, has_silu=False, fused=fused, round_scores=True)
        return graph_kernel_ms(up, x_dev.device), graph_kernel_ms(down, x_dev.device)


def fp8_dense_peak(device):
    """Yardstick for the e4m3 GEMMs, measured in this run: cuBLASLt's dense e4m3 x e4m3 -> bf16
    product (torch._scaled_mm, 8192^3, per-tensor scales), best of 10 launches, CUDA events."""
    try:
        n = 8192
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=device)
        fn = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            fn()
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize(device)
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception as exc:   # the yardstick is optional; say why it is missing
        return f"unavailable: {type(exc).__name__}: {exc}"[:200]


# ------------------------------------------------------------------------------------ parity
def _routing_block(idx_gpu, score_gpu, meta, x_rows_cpu, gate_w, gate_b, k, E):
    """Routing of the whole batch against the oracle: expert sets per token (near ties counted
    apart), renormalised scores, and - given the GPU's own top-k slots - offsets, gate_index,
    token_index and reverse_index bit for bit."""
    from oracle import moe_oracle as O
    from oracle import sampled as S

    idx_ref, scores_ref, _, _, _, _, gap = S.route_full(x_rows_cpu, gate_w, gate_b, k)
    blk = S.routing_exactness(idx_gpu, idx_ref, gap)
    ig = idx_gpu.cpu()
    dense = torch.zeros(ig.shape[0], E).scatter_(1, ig, score_gpu.float().cpu())
    # scores of the chosen experts, compared per (token, expert)
    dense_ref = torch.zeros(ig.shape[0], E).scatter_(1, idx_ref, scores_ref)
    same = (torch.sort(ig, 1).values == torch.sort(idx_ref, 1).values).all(1)
    blk["max_score_diff"] = float((dense[same] - dense_ref[same]).abs().max()) if bool(same.any()) else 0.0
    gi, ti, _, off, rev, _ = O.routing_metadata(dense.clamp_min(1e-30) * (dense > 0), ig)
    lengths_ok = torch.equal(O.histogram_lengths(ig, E), (meta.offsets[1:] - meta.offsets[:-1]).cpu())
    blk["metadata_bit_exact"] = bool(
        lengths_ok and torch.equal(gi, meta.gate_index.cpu()) and torch.equal(ti, meta.token_index.cpu())
        and torch.equal(rev, meta.reverse_index.cpu()) and int(meta.offsets[-1]) == ig.numel())
    return blk, idx_ref, gap


def parity_block(layer, c, x_cpu, y_dev, expert_weights, gate, n_sample=96, seed=0, max_experts=None):
    """Compares one forward of the benchmarked layer (y_dev) with the CPU oracle, outside any timed
    region. Routing tensors: whole batch, bit for bit. Outputs: a seeded sample of tokens (the
    oracle needs only those rows and their experts' weights). bf16: |y - ref| <= 1e-2 max(1, S) +
    1e-2 |ref| per element against the fp32 oracle on the same bf16-rounded inputs, S = the
    largest gate-weighted expert row of the token (1 whenever outputs stay below 1, as at c2;
    see oracle/sampled.py:compare_tokens); the count under plain rtol / atol is reported too. FP8: against the oracle's
    quantise -> e4m3 product -> descale chain within 4e-2 of the row's largest magnitude, and the
    row-wise relative error against the unquantised fp32 oracle (bound 6e-2 per quantised GEMM,
    two GEMMs in the chain)."""
    import fast_moe_b200 as fm
    from oracle import sampled as S

    k, E, d = c["k"], c["E"], c["d"]
    dev = y_dev.device
    x_rows = x_cpu.reshape(-1, d)
    gate_w, gate_b = gate.weight.detach().float().cpu(), gate.bias.detach().float().cpu()
    x_dev = x_rows.to(dev)
    idx_gpu, score_gpu, _ = fm.gate_topk(x_dev, gate.weight.detach(), gate.bias.detach(), k)
    meta = fm.route_metadata(idx_gpu, E)
    routing, idx_ref, gap = _routing_block(idx_gpu, score_gpu, meta, x_rows, gate_w, gate_b, k, E)
    experts = None
    if max_experts is not None and max_experts < E:
        # the most loaded experts that fit the host budget (ties broken by id)
        load = torch.bincount(idx_ref.reshape(-1), minlength=E)
        experts = torch.argsort(load, descending=True, stable=True)[:max_experts].tolist()
    sel = S.pick_tokens(idx_ref, n_sample, seed=seed, experts=experts, gap=gap)
    y_rows = y_dev.reshape(-1, c["o"])[sel.to(dev)].float().cpu()
    out = dict(routing=routing, sample=dict(tokens=int(sel.numel()), of=int(x_rows.shape[0]), seed=seed,
                                            experts_held=len(experts) if experts else E))
    if sel.numel() == 0:
        out["ok"] = False
        out["error"] = "no token qualifies for the sample"
        return out
    y_ref, _, op_scale = S.swiglu_layer_on_tokens(x_rows[sel], gate_w, gate_b, k, expert_weights, with_operand_scale=True)
    if c.get("fp8"):
        y_emu, _ = S.swiglu_fp8_layer_on_tokens(x_rows[sel], gate_w, gate_b, k, expert_weights)
        y_emu = y_emu.float()
        row = y_emu.abs().amax(dim=1, keepdim=True).clamp_min(1e-6)
        close = ((y_rows - y_emu).abs() / row).amax(dim=1)
        rel = (y_rows - y_ref).norm(dim=1) / y_ref.norm(dim=1).clamp_min(1e-6)
        rel_emu = (y_emu - y_ref).norm(dim=1) / y_ref.norm(dim=1).clamp_min(1e-6)
        out["outputs"] = dict(
            tokens=int(sel.numel()), bound_vs_fp8_oracle="max |y - emu| / rowmax <= 4e-2",
            tokens_out_of_tolerance=int((close > 4e-2).sum()), max_vs_fp8_oracle=float(close.max()),
            rel_err_vs_fp32_median=float(rel.median()), rel_err_vs_fp32_max=float(rel.max()),
            fp8_oracle_rel_err_vs_fp32_median=float(rel_emu.median()),
            bound_vs_fp32="row-wise relative error <= 6e-2 per quantised GEMM (two in the chain)")
        ok_out = out["outputs"]["tokens_out_of_tolerance"] == 0 and float(rel.median()) < 2 * 6e-2
    else:
        out["outputs"] = S.compare_tokens(y_rows, y_ref, operand_scale=op_scale)
        ok_out = out["outputs"]["tokens_out_of_tolerance"] == 0
    out["ok"] = bool(ok_out and routing["mismatched"] == 0 and routing["metadata_bit_exact"])
    return out


def layer_expert_weights(layer):
    """e -> (w_gate [h, d], w_up [h, d], w_down [o, h]) on the host, from a single-GPU layer."""
    return lambda e: (layer.w_gate.detach()[e].cpu(), layer.w_up.detach()[e].cpu(), layer.w_down.detach()[e].cpu())


# ------------------------------------------------------------------------------------ CPU arm
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
                 f"E={c['E']}, top-{c['k']}" + (", fp8 e4m3 rowwise" if c.get("fp8") else ", bf16")
                 + (f", Zipf({c['zipf']}) expert loads" if c.get("zipf") else ""),
        tokens_per_rank=c["tokens"], global_tokens=c["tokens"] * n_gpus, d=c["d"], h=c["h"], E=c["E"], k=c["k"],
        parallelism="single GPU" if n_gpus == 1 else f"expert parallel ep{n_gpus} ({c['E'] // n_gpus} experts/rank)",
        l2="working set (weights + activations) is larger than the 126 MB L2; no explicit flush",
    )


# ------------------------------------------------------------------------------------ timing
def time_steps(step, steps, sync):
    """CUDA-event time of `steps` calls of step() on the current stream, synchronised on both sides."""
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    out = None
    for _ in range(steps):
        out = step()
    e1.record()
    sync()
    return e0.elapsed_time(e1), out


def sustained_record(step, ms_step_hint, c, tokens, sampler, peaks, seconds=1.2):
    """The same step repeated for at least `seconds` of device time, with the clocks sampled
    alongside: what the part sustains under its power cap (the headline's K steps may be a burst)."""
    n = max(10, int(math.ceil(seconds * 1e3 / max(ms_step_hint, 1e-3))))
    t0 = time.perf_counter()
    ms, _ = time_steps(step, n, torch.cuda.synchronize)
    t1 = time.perf_counter()
    ms_step = ms / n
    tf = layer_flops(c, tokens) / (ms_step * 1e-3) / 1e12
    rec = dict(steps=n, seconds=ms * 1e-3, ms_per_step=ms_step, value=tokens / (ms_step * 1e-3), unit="tokens/s",
               layer_tflops=tf, frac_of_sustained_peak=None if c.get("fp8") else tf / peaks["bf16_tflops_sustained"],
               sustained_peak_tflops=peaks["bf16_tflops_sustained"], peak_source=peaks["source"])
    if sampler is not None:
        rec["clocks"] = sampler.window(t0, t1)
    return rec


def single_gpu_record(name, device, args, peaks, fp8_peak, sampler=None, sustained=False, parity=True):
    """Builds configuration `name` on this GPU and measures it: graph-replay step time, the two
    GEMMs alone, a parity block. Used for the c3 / c4 sub-records of the N = 1 line."""
    from fast_moe_b200 import CapturedForward, _lib

    c = CONFIGS[name]
    k = c["k"]
    layer = build_layer(c, device)
    x_cpu = make_inputs(c, 0)
    x_dev = x_cpu.to(device)
    for _ in range(3):
        y = layer(x_dev, k)
    torch.cuda.synchronize()
    cap = CapturedForward(layer, x_dev, k)
    for _ in range(3):
        cap.replay()
    steps = max(3, min(args.steps, 10))
    ms, y = time_steps(cap.replay, steps, torch.cuda.synchronize)
    ms_step = ms / steps
    timer = _lib.StageTimer()
    _lib.set_stage_timer(timer)
    for _ in range(3):
        layer(x_dev, k)
    _lib.set_stage_timer(None)
    stage_ms = {n: tot / cnt for n, (tot, cnt) in timer.totals_ms().items()}
    up_ms, down_ms = gemm_alone_ms(layer, x_dev, k, bool(c.get("fp8")))
    A = c["tokens"] * k
    gemm_peak = fp8_peak if (c.get("fp8") and isinstance(fp8_peak, float)) else peaks["bf16_tflops"]
    up_tf = 4 * A * c["d"] * c["h"] / (up_ms * 1e-3) / 1e12
    down_tf = 2 * A * c["h"] * c["o"] / (down_ms * 1e-3) / 1e12
    rec = dict(
        workload=workload_config(c, name, 1)["workload"], value=c["tokens"] / (ms_step * 1e-3), unit="tokens/s",
        ms_per_step=ms_step, steps=steps, launch_mode="cuda graph replay",
        layer_tflops=layer_flops(c, c["tokens"]) / (ms_step * 1e-3) / 1e12, stage_ms_eager=stage_ms,
        up_gemm=dict(ms=up_ms, tflops=up_tf, frac=up_tf / gemm_peak),
        down_gemm=dict(ms=down_ms, tflops=down_tf, frac=down_tf / gemm_peak,
                       includes="combine fused in the epilogue" if k <= 2 else "separate combine kernel"),
        gemm_peak_tflops=gemm_peak,
        gemm_peak_source=("torch._scaled_mm e4m3 8192^3, this run" if c.get("fp8") and isinstance(fp8_peak, float)
                          else peaks["source"] + " bf16 burst"),
        device_status=_lib.device_status(device),
    )
    hbm = peaks["hbm_gbs"]
    if c.get("fp8"):
        # the activation quantisation kernels of the FP8 layer: algorithmic bytes / eager stage time
        for st, nbytes in (("quant_x", c["tokens"] * c["d"] * 3), ("quant_hidden", A * c["h"] * 3)):
            if st in stage_ms:
                rec[st] = dict(ms=stage_ms[st], gbs=nbytes / stage_ms[st] / 1e6, frac_of_hbm=nbytes / stage_ms[st] / 1e6 / hbm)
    if "combine" in stage_ms:
        nbytes = (A + c["tokens"]) * c["o"] * 2
        rec["combine"] = dict(ms=stage_ms["combine"], gbs=nbytes / stage_ms["combine"] / 1e6,
                              frac_of_hbm=nbytes / stage_ms["combine"] / 1e6 / hbm)
    if c.get("zipf"):
        idx = None
        import fast_moe_b200 as fm

        idx, _, _ = fm.gate_topk(x_dev.reshape(-1, c["d"]), layer.gate.gate.weight.detach(), layer.gate.gate.bias.detach(), k)
        load = torch.bincount(idx.reshape(-1), minlength=c["E"]).float()
        rec["expert_load"] = dict(max_share_of_assignments=float(load.max() / load.sum()),
                                  empty_experts=int((load == 0).sum()), min_nonzero=int(load[load > 0].min()))
    if sustained:
        rec["sustained"] = sustained_record(cap.replay, ms_step, c, c["tokens"], sampler, peaks)
    if parity:
        torch.set_num_threads(os.cpu_count() or 1)
        rec["parity"] = parity_block(layer, c, x_cpu, y, layer_expert_weights(layer), layer.gate.gate,
                                     n_sample=64, max_experts=3 if c.get("fp8") else 24)
    del cap, layer, y, x_dev
    torch.cuda.empty_cache()
    return rec


def _guarded(fn):
    """A secondary record must not take the line down with it: its failure is reported in its place."""
    try:
        return fn()
    except Exception as exc:      # noqa: BLE001 - reported, not swallowed
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        return dict(error=f"{type(exc).__name__}: {exc}"[:500])


def sg_flops_of(A, L, d, h, o, E):
    """Forward FLOPs of the sparsely-gated layer: two expert products, the shared map, the gate."""
    return 2 * A * d * h + 2 * A * h * o + 2 * L * d * o + 2 * L * d * E


def next_rows_record(device, peaks, steps=10):
    """Device times of the widened rows at the C2 sizes (4096 tokens, d 1024, h 4096, 8 experts,
    top-2, bf16): a training step (forward + backward) of both layers, the sparsely-gated layer's
    forward with and without noisy gating, and the two operators no layer uses. Parity of each is
    held by the GPU tests against fixtures recorded from the reference; these are timings only."""
    import fast_moe_b200 as fm
    from fast_moe_b200 import _lib
    from fast_moe_b200.kernels import moe as ops

    c = CONFIGS["c2"]
    L, d, h, o, E, k = c["tokens"], c["d"], c["h"], c["o"], c["E"], c["k"]
    A = L * k
    rec = {}

    def eager_ms(fn, n=steps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / n, (time.perf_counter() - t0) / n * 1e3

    # ---- backward pass: training step of the two layers
    x = make_inputs(c, 0).to(device)
    for name, build in (("swiglu_layer", lambda: build_layer(c, device)),
                        ("silu_layer", lambda: fm.FastMoELayer(d, h, o, E, dtype=torch.bfloat16).to(device))):
        layer = build()
        layer.autograd = True
        xg = x.clone().requires_grad_(True)

        def train_step():
            for p_ in layer.parameters():
                p_.grad = None
            xg.grad = None
            y_ = layer(xg, k)
            y_.backward(torch.ones_like(y_))

        ms_eager, ms_wall = eager_ms(train_step)
        for p_ in layer.parameters():
            p_.grad = None
        graph_step = fm.CapturedTrainStep(layer, x, k)
        ms_dev, _ = eager_ms(graph_step.replay)
        proj = 3 if name == "swiglu_layer" else 2
        fwd_flops = 2 * A * d * h * (proj - 1) + 2 * A * h * o
        rec_flops = 4 * A * d * h if name == "swiglu_layer" else 0        # SwiGLU backward recomputes the up projection
        rec["train_" + name] = dict(
            ms_per_step=ms_dev, launch_mode="forward + backward as one CUDA graph (CapturedTrainStep), CUDA events around 10 replays",
            ms_per_step_eager=ms_eager, ms_per_step_eager_wall=ms_wall,
            model_tflops=3 * fwd_flops / (ms_dev * 1e-3) / 1e12,
            executed_tflops=(3 * fwd_flops + rec_flops) / (ms_dev * 1e-3) / 1e12,
            frac_of_bf16_burst=(3 * fwd_flops + rec_flops) / (ms_dev * 1e-3) / 1e12 / peaks["bf16_tflops"],
            tokens_per_s=L / (ms_dev * 1e-3), device_status=_lib.device_status(device))
        if name == "silu_layer":
            # the reference's primary layer class (FastMoELayer: SiLU experts with biases), forward only
            layer.autograd = False
            ms_fwd = graph_kernel_ms(lambda: layer(x, k), device)
            rec["silu_layer_forward"] = dict(ms_per_step=ms_fwd, tokens_per_s=L / (ms_fwd * 1e-3),
                                             layer_tflops=(fwd_flops + 2 * L * d * E) / (ms_fwd * 1e-3) / 1e12,
                                             launch_mode="10 forwards in a CUDA graph")
        del graph_step, layer, xg
    # ---- sparsely-gated layer forward (d -> h -> o MLP experts + shared linear map)
    torch.manual_seed(0)
    sg = fm.SGMoELayer(d, o, fm.SGConfig(model_d=h, num_experts=E, num_activated_experts=k)).to(device)
    sgn = fm.SGMoELayer(d, o, fm.SGConfig(model_d=h, num_experts=E, num_activated_experts=k, enable_noisy_gating=True)).to(device)
    with torch.no_grad():
        sgn._w_gate.normal_(0, 0.05)
        sgn._w_noise.normal_(0, 0.05)
    x2 = x.reshape(L, d)
    nw = torch.ones(d, device=device)
    nb = torch.zeros(d, device=device)
    sg.train(False)
    ms_eval = graph_kernel_ms(lambda: sg(x2, None, 0, False, 1, d, nw, nb, 1e-5), device)
    sgn.train(True)
    ms_noisy, _ = eager_ms(lambda: sgn(x2, None, 0, False, 1, d, nw, nb, 1e-5))
    sg_flops = sg_flops_of(A, L, d, h, o, E)
    sg.train(True)
    sg.autograd = True
    xs = x2.clone().requires_grad_(True)

    def sg_train_step():
        for p_ in sg.parameters():
            p_.grad = None
        xs.grad = None
        out_ = sg(xs, None, 0, False, 1, d, nw, nb, 1e-5)
        (out_.x.float().sum() + out_.loss).backward()

    ms_sg_eager, ms_sg_wall = eager_ms(sg_train_step)
    for p_ in sg.parameters():
        p_.grad = None
    sg_graph = fm.CapturedTrainStep(sg, x2, k, forward_fn=lambda m_, t_: m_(t_, None, 0, False, 1, d, nw, nb, 1e-5).x)
    ms_sg_train, _ = eager_ms(sg_graph.replay)
    rec["train_sg_moe_layer"] = dict(ms_per_step=ms_sg_train,
                                     launch_mode="forward + backward of the output as one CUDA graph (CapturedTrainStep)",
                                     ms_per_step_eager=ms_sg_eager, ms_per_step_eager_wall=ms_sg_wall,
                                     eager_includes="the loss's backward as well",
                                     model_tflops=3 * sg_flops_of(A, L, d, h, o, E) / (ms_sg_train * 1e-3) / 1e12,
                                     tokens_per_s=L / (ms_sg_train * 1e-3))
    del sg_graph
    for p_ in sg.parameters():
        p_.grad = None
    sg.autograd = False
    rec["sg_moe_forward"] = dict(ms_per_step=ms_eval, tokens_per_s=L / (ms_eval * 1e-3),
                                 layer_tflops=sg_flops / (ms_eval * 1e-3) / 1e12, launch_mode="10 forwards in a CUDA graph",
                                 noisy_gating_training_ms=ms_noisy, noisy_launch_mode="eager (fresh torch.randn per step)")
    del sg, sgn
    # ---- the two operators no layer calls
    torch.manual_seed(1)
    idx = torch.stack([torch.randperm(E, device=device)[:k] for _ in range(64)]).repeat(L // 64, 1)
    meta = fm.route_metadata(idx, E)
    index = meta.gate_index.view(-1, k)
    xa = x2
    xb = torch.randn_like(x2)
    wa = (torch.randn(E, h, d, device=device) * 0.02).bfloat16().permute(0, 2, 1)
    wb = (torch.randn(E, h, d, device=device) * 0.02).bfloat16().permute(0, 2, 1)
    ms_gate2 = graph_kernel_ms(lambda: ops.index_select_jagged_gating_bmm(0, meta.offsets, index, xa, xb, wa, None, wb, None), device)
    rec["gating_bmm_two_inputs"] = dict(ms=ms_gate2, tflops=4 * A * d * h / (ms_gate2 * 1e-3) / 1e12,
                                        frac_of_bf16_burst=4 * A * d * h / (ms_gate2 * 1e-3) / 1e12 / peaks["bf16_tflops"],
                                        shape=f"{A} rows, K={d}, N={h}, two inputs, two weights")
    x3 = torch.randn(L, E, 256, device=device).bfloat16()
    w3 = (torch.randn(E, 1024, 256, device=device) * 0.02).bfloat16().permute(0, 2, 1)
    ms_3d = graph_kernel_ms(lambda: ops.index_select_jagged_bmm_3D(0, meta.offsets, index, x3, w3, None), device)
    rec["bmm_3D"] = dict(ms=ms_3d, tflops=2 * A * 256 * 1024 / (ms_3d * 1e-3) / 1e12,
                         shape=f"input [{L}, {E}, 256], {A} rows, N=1024")
    rec["parity"] = ("tests/test_gpu_backward.py, tests/test_gpu_sg_moe.py, tests/test_gpu_parity.py: gradients, layer outputs "
                     "and operator outputs against fixtures recorded from the reference")
    torch.cuda.empty_cache()
    return rec


def ep_single_gpu_record(device, args, peaks, with_e2e=True, parity=True):
    """c5 (64 experts, d=4096, h=14336, 8192 tokens) with every expert on this GPU: the per-rank
    workload of the multi-GPU runs, i.e. the denominator of their weak-scaling efficiency."""
    from fast_moe_b200 import CapturedForward, StreamingForward, _lib
    from fast_moe_b200.modules.expert_parallel import ExpertParallelSwiGLUMoE

    c = CONFIGS["c5"]
    k = c["k"]
    layer = ExpertParallelSwiGLUMoE(c["d"], c["h"], c["o"], c["E"], dtype=torch.bfloat16, device=device, world_size=1)
    x_cpu = make_inputs(c, 0)
    x_host = x_cpu.pin_memory()
    x = x_host.to(device)
    steps = max(3, min(args.steps, 10))
    for _ in range(3):
        layer(x, k)
    torch.cuda.synchronize()
    cap = CapturedForward(layer, x, k)
    for _ in range(3):
        cap.replay()
    ms, y = time_steps(cap.replay, steps, torch.cuda.synchronize)
    ms /= steps
    rec = dict(value=c["tokens"] / (ms * 1e-3), unit="tokens/s", ms_per_step=ms, steps=steps,
               launch_mode="cuda graph replay",
               layer_tflops=layer_flops(c, c["tokens"]) / (ms * 1e-3) / 1e12,
               bound_ms_compute=layer_flops(c, c["tokens"]) / (peaks["bf16_tflops"] * 1e12) * 1e3,
               bound_ms_hbm=layer_min_bytes(c, c["tokens"]) / (peaks["hbm_gbs"] * 1e9) * 1e3,
               workload=workload_config(c, "c5", 1)["workload"], device_status=_lib.device_status(device))
    if with_e2e:
        slots = 3
        pipe = StreamingForward(layer, x, k, slots=slots, capture=True)
        y_hosts = [torch.empty((c["batch"], c["seq"], c["o"]), dtype=torch.bfloat16).pin_memory() for _ in range(slots)]
        for i in range(slots):
            pipe.submit(x_host, y_hosts[i])
        pipe.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            pipe.submit(x_host, y_hosts[i % slots])
        pipe.drain()
        e1.record()
        torch.cuda.synchronize()
        ms_e2e = e0.elapsed_time(e1) / steps
        rec["e2e"] = dict(value=c["tokens"] / (ms_e2e * 1e-3), unit="tokens/s", ms_per_step=ms_e2e,
                          h2d_bytes_per_step=x_host.numel() * 2, d2h_bytes_per_step=y_hosts[0].numel() * 2)
        del pipe
    if parity:
        torch.set_num_threads(os.cpu_count() or 1)
        rec["parity"] = parity_block(layer, c, x_cpu, y, lambda e: tuple(t.cpu() for t in layer.materialize_expert(e)),
                                     layer.gate, n_sample=64, max_experts=8)
    del cap, layer, y, x
    torch.cuda.empty_cache()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ep-reference", action="store_true", help="skip the 1-GPU run of the multi-GPU workload")
    ap.add_argument("--no-sub-records", action="store_true", help="N = 1: skip the c3 / c4 sub-records")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison (profiling runs)")
    ap.add_argument("--no-sustained", action="store_true")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: rows through peer-mapped buffers (default) or NCCL all-to-all")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of a CUDA-graph replay")
    ap.add_argument("--train-step", action="store_true", help="only a training step of the layer (profiling runs)")
    ap.add_argument("--layer-sweep", action="store_true", help="forward time of the layer over a range of batch sizes")
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
    if args.routing_sweep or args.layer_sweep or args.train_step:
        if rank == 0:
            if args.train_step:
                train_step_only(c, device, args.steps, args.warmup)
            else:
                (routing_sweep if args.routing_sweep else layer_sweep)(c, device)
        return
    peaks = load_peaks()
    dist = None
    json_fd = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        # stdout carries the one JSON line and nothing else: whatever the libraries write to file
        # descriptor 1 on the way (the communicator's version banner) goes to stderr, and the line
        # itself is written to the descriptor saved here
        sys.stdout.flush()
        json_fd = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=device)

    from fast_moe_b200 import _lib

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- N > 1: rank 0 first times the per-rank workload alone (all 64 experts on its GPU)
    t1_rec = None
    if world > 1 and not args.no_ep_reference:
        if rank == 0:
            t1_rec = ep_single_gpu_record(device, args, peaks, with_e2e=True, parity=False)
        barrier()

    k = c["k"]
    x_cpu = make_inputs(c, rank)
    x_host = x_cpu.pin_memory()
    x_dev = x_host.to(device)
    if world > 1:
        from fast_moe_b200.modules.expert_parallel import ExpertParallelSwiGLUMoE

        torch.manual_seed(0)
        layer = ExpertParallelSwiGLUMoE(c["d"], c["h"], c["o"], c["E"], dtype=torch.bfloat16, device=device,
                                        exchange=args.exchange, max_tokens_per_rank=c["tokens"])
    else:
        layer = build_layer(c, device)

    # ---- device-resident timing
    # Single GPU: the forward is captured once as a CUDA graph and a step is one replay (same
    # kernels, one launch). A second, eager pass with CUDA events around each stage gives the
    # per-stage times.
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
    t_wall0 = time.perf_counter()
    ms_total, y = time_steps(step, args.steps, barrier)
    # eager pass with stage events (also what counts launches when the timed pass was a graph);
    # graph capture empties the allocator cache, so the eager path is warmed up again first
    for _ in range(3):
        layer(x_dev, k)
    barrier()
    timer = _lib.StageTimer()
    _lib.set_stage_timer(timer)
    launches_eager0 = _lib.kernel_launch_count()
    ms_eager, _ = time_steps(lambda: layer(x_dev, k), args.steps, barrier)
    ms_eager /= args.steps
    t_wall1 = time.perf_counter()
    launches = _lib.kernel_launch_count() - launches_eager0   # kernels per K steps (the graph replays the same ones)
    _lib.set_stage_timer(None)
    clocks = sampler.window(t_wall0, t_wall1) if rank == 0 else None
    stage_ms = {n: (tot / cnt) for n, (tot, cnt) in timer.totals_ms().items()}
    up_alone_ms = down_alone_ms = route_alone_ms = None
    if world == 1:
        up_alone_ms, down_alone_ms = gemm_alone_ms(layer, x_dev, k, bool(c.get("fp8")))
        if hasattr(layer, "_route_with_passes") and not c.get("fp8"):
            # the routing chain alone, as the layer runs it (gate + top-k, counting sort, and - in the
            # fused small-batch form - the row gather and the clearing of the combine buffer)
            with torch.no_grad():
                xf = x_dev.reshape(-1, c["d"])
                route_alone_ms = graph_kernel_ms(lambda: layer._route_with_passes(xf, k, 2 * c["h"], c["o"], k <= 2), device)
    status = _lib.device_status(device)

    sustained = None
    if world == 1 and not args.no_sustained:
        sustained = sustained_record(step, ms_total / args.steps, c, c["tokens"], sampler if rank == 0 else None, peaks)

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
    e2e_legs = pipe.leg_times_ms() if hasattr(pipe, "leg_times_ms") else None
    e2e_mode = "%d-slot pipeline: H2D, forward and D2H of consecutive steps overlap" % slots
    e2e_alt = None
    del pipe
    if captured is not None:
        # the same pipeline with one launch per step: every slot's copy-in, forward and copy-out are
        # one CUDA graph on the slot's own stream (the per-step host work above - stream switches,
        # event records and waits - is the slowest part at this batch size)
        from fast_moe_b200 import HostPipeline

        hp = HostPipeline(layer, x_dev, k, slots=slots)
        for s_ in range(slots):
            hp.host_in[s_].copy_(x_host)
        for i in range(max(3, slots)):
            hp.launch(i % slots)
        hp.synchronize()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for i in range(args.steps):
            hp.launch(i % slots)
        hp.drain()
        g1.record()
        barrier()
        ms_graph = g0.elapsed_time(g1)
        check2 = float((hp.host_out[(args.steps - 1) % slots].float() - y.detach().float().cpu().view_as(y_host)).abs().max())
        e2e_alt = dict(one_graph_launch_per_step_ms=ms_graph / args.steps, three_stream_events_ms=ms_e2e / args.steps)
        if ms_graph < ms_e2e:
            ms_e2e, e2e_check = ms_graph, check2
            e2e_mode = ("%d-slot pipeline, one CUDA-graph launch per step (copy-in, forward, copy-out of a slot in "
                        "one graph on the slot's stream); the event-ordered three-stream form took %.4f ms/step"
                        % (slots, e0.elapsed_time(e1) / args.steps))
        del hp

    # ---- parity of this very layer and batch against the CPU oracle (outside the timed regions)
    parity = None
    if not args.no_parity:
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // max(1, world)))
        if world > 1:
            mine = parity_block(layer, c, x_cpu, y, lambda e: tuple(t.cpu() for t in layer.materialize_expert(e)),
                                layer.gate, n_sample=48, seed=rank, max_experts=8)
            mine["rank"] = rank
            allp = [None] * world
            dist.all_gather_object(allp, mine)
            parity = dict(ok=all(p["ok"] for p in allp),
                          tokens=sum(p["sample"]["tokens"] for p in allp),
                          tokens_out_of_tolerance=sum(p["outputs"]["tokens_out_of_tolerance"] for p in allp if "outputs" in p),
                          routing_mismatched=sum(p["routing"]["mismatched"] for p in allp),
                          oracle="oracle/sampled.py on every rank's own tokens, the weights of the sampled experts "
                                 "rebuilt from their global seed", per_rank=allp)
        else:
            parity = parity_block(layer, c, x_cpu, y, layer_expert_weights(layer), layer.gate.gate,
                                  n_sample=c["tokens"] if name == "c2" else 64,
                                  max_experts=None if name == "c2" else (3 if c.get("fp8") else 24))

    t = torch.tensor([ms_total, ms_e2e], device=device, dtype=torch.float64)
    stage_ms_ranks = None
    legs_ranks = None
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        stage_ms_ranks = [None] * world
        dist.all_gather_object(stage_ms_ranks, {n: round(v, 4) for n, v in stage_ms.items()})
        legs_ranks = [None] * world
        dist.all_gather_object(legs_ranks, e2e_legs)
    ms_total, ms_e2e = t.tolist()

    if rank == 0:
        sampler.stop(t_wall0, t_wall1)
        ms_step = ms_total / args.steps
        tokens_total = c["tokens"] * world
        A = c["tokens"] * k
        fp8_peak = fp8_dense_peak(device) if (world == 1 and (c.get("fp8") or not args.no_sub_records)) else None
        # the dominant kernel's duration: alone, back to back in a graph (single GPU), else the
        # eager stage events (which include host launch gaps when the host is the slower side)
        up_ms = up_alone_ms if up_alone_ms is not None else stage_ms.get("up")
        up_flops = 4 * A * c["d"] * c["h"]
        # the up-projection kernel is timed alone between two events: burst peak is its yardstick
        if c.get("fp8") and isinstance(fp8_peak, float):
            peak_tf, peak_src = fp8_peak, "torch._scaled_mm e4m3 8192^3 measured in this run"
        else:
            peak_tf, peak_src = peaks["bf16_tflops"], peaks["source"] + " burst"
        roofline = None
        if up_ms:
            ach = up_flops / (up_ms * 1e-3) / 1e12
            traffic, traffic_commit = ncu_traffic(name) if world == 1 else (None, None)
            roofline = dict(bound="tensor", kernel="grouped_gemm_kernel (gate/up GEMM + SwiGLU on expert-sorted rows)",
                            achieved=ach, peak=peak_tf, unit="TFLOP/s", frac=ach / peak_tf,
                            traffic=traffic, traffic_source=(f"profiles/grouped_gemm_{name}.md, captured at commit "
                                                             f"{traffic_commit}") if traffic else None,
                            algorithmic_bytes=(2 * c["E"] * c["d"] * c["h"] + A * c["d"] + A * c["h"]) * (1 if c.get("fp8") else 2),
                            peak_source=peak_src,
                            flops_per_launch=up_flops, avg_launch_ms=up_ms,
                            timing="10 launches back to back in a CUDA graph, CUDA events" if up_alone_ms is not None
                            else "CUDA events around the eager launch")
            if down_alone_ms:
                dtf = 2 * A * c["h"] * c["o"] / (down_alone_ms * 1e-3) / 1e12
                roofline["down_gemm"] = dict(ms=down_alone_ms, tflops=dtf, frac=dtf / peak_tf)
            if route_alone_ms:
                roofline["routing_chain"] = dict(
                    ms=route_alone_ms, includes="gate + top-k, counting sort, row gather into expert order, clearing of "
                    "the combine buffer; 10 repetitions in a CUDA graph, warm")
        line = dict(
            metric="moe_layer_fwd_tokens_per_s", value=tokens_total / (ms_step * 1e-3), unit="tokens/s",
            n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms_step, higher_is_better=True,
            scaling="weak", vs_baseline=None, dtype="e4m3" if c.get("fp8") else "bf16", data="synthetic",
            config=workload_config(c, name, world),
            layer_tflops_per_gpu=layer_flops(c, c["tokens"]) / (ms_step * 1e-3) / 1e12,
            launch_mode="cuda graph replay" if captured is not None else "eager", ms_per_step_eager=ms_eager,
            stage_ms=stage_ms, stage_ms_per_rank=stage_ms_ranks, roofline=roofline, clocks=clocks, gpu_launches=int(launches),
            device_status=status, parity=parity, sustained=sustained,
            e2e=dict(value=tokens_total / (ms_e2e / args.steps * 1e-3), unit="tokens/s",
                     h2d_bytes_per_step=x_host.numel() * x_host.element_size(),
                     d2h_bytes_per_step=y_host.numel() * y_host.element_size(), ms_per_step=ms_e2e / args.steps,
                     mode=e2e_mode, both_forms_ms_per_step=e2e_alt,
                     max_abs_diff_vs_resident=e2e_check, leg_ms_per_rank=legs_ranks if legs_ranks else e2e_legs),
        )
        if world > 1 and t1_rec is not None:
            El = c["E"] // world
            line["weak_scaling"] = dict(
                t1_ms=t1_rec["ms_per_step"], tN_ms=ms_step, efficiency=t1_rec["ms_per_step"] / ms_step,
                t1=t1_rec,
                e2e_efficiency=(t1_rec["e2e"]["ms_per_step"] / (ms_e2e / args.steps)) if "e2e" in t1_rec else None,
                bound_ms_compute=layer_flops(c, c["tokens"]) / (peaks["bf16_tflops"] * 1e12) * 1e3,
                bound_ms_hbm=layer_min_bytes(c, c["tokens"], El) / (peaks["hbm_gbs"] * 1e9) * 1e3,
                bound_ms_nvlink=2 * A * c["d"] * 2 * (world - 1) / world / 770e9 * 1e3,
                note="t1 = the same per-rank workload (8192 tokens, all 64 experts) alone on rank 0's GPU in this run; "
                     "efficiency = t1 / tN; above 1 because one GPU streams 64 experts' weights (HBM-bound) and a "
                     "rank of the sharded run only its own")
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = time_cpu_baseline(c, c["tokens"])
        if world == 1 and args.config is None:
            del layer, y, captured, step
            torch.cuda.empty_cache()
            line["fp8_dense_peak_tflops"] = fp8_peak
            if not args.no_sub_records:
                for sub in ("c3", "c4"):
                    line[sub] = _guarded(lambda: single_gpu_record(sub, device, args, peaks, fp8_peak, parity=not args.no_parity))
                line["next_rows"] = _guarded(lambda: next_rows_record(device, peaks))
            if not args.no_ep_reference:
                line["c5_ep_1gpu"] = _guarded(lambda: ep_single_gpu_record(device, args, peaks, with_e2e=True,
                                                                           parity=not args.no_parity))
        if json_fd is None:
            print(json.dumps(line), flush=True)
        else:
            sys.stdout.flush()
            with os.fdopen(json_fd, "w") as out:
                out.write(json.dumps(line) + "\n")
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
