"""Benchmark of the xLSTM recurrent-cell kernels on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--case NAME]

Headline case (default, "chunkwise"): one step = one forward of the mLSTM cell over B=4 sequences x NH=8 heads x
S=8192 tokens, DHQK=256, DHV=512 (the head shapes of xLSTM-7B), bf16 inputs, fp32 state, zero initial state; seeded
synthetic inputs: q, k ~ N(0,1)/sqrt(256), v ~ N(0,1), input-gate pre-activations ~ N(0,1), forget-gate
pre-activations ~ N(3,1).  The metric counts B*S tokens per step (one token = all 8 heads of one xLSTM-7B layer).  At
N > 1 every rank runs its own batch of sequences (documents are data-parallel, no collective on the data path): weak
scaling.

The default run adds, in the same JSON line under "sub", the other measurements of the path, each taken in the same
process: the xLSTM-7B-shaped model (prefill 8 x 8192 tokens + 512 greedy tokens, heads tensor-parallel over the N
ranks), and at N = 1 the decode-step kernel, the sLSTM kernel and the fused operators next to the cell.  `--case NAME`
prints one of them as a line of its own:
  step          mLSTM decode step, 256 streams x 8 heads (xLSTM-7B head shapes), state resident in HBM
  slstm         sLSTM forward at the block-stack benchmark's cell shape (B=16, S=2048, NH=4, DH=256), next to the
                reference's own CUDA backend when the reference package is present
  headwise      the four headwise gate projections + concatenation of the sLSTM layer at the same shape
  layer_ops     residual add + RMSNorm and per-head norm + output gate at the 7B prefill shapes
  chunkwise_b1  the headline kernel on one sequence (B=1): the size used for profiler captures
  model7b       the xLSTM-7B-shaped model (random init, bf16): prefill 8 x 8192 + 512 greedy tokens, strong scaling
  decode7b      one graph-replayed decode step of that model at batch 8
  continuous7b  continuous batching: packed prefill of log-normal documents into a pool of decode slots with refill

`--impl reference` times the reference's native CPU formulation (the oracle port) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(B=4, NH=8, S=8192, DHQK=256, DHV=512, chunk=64)
STEP_CFG = dict(B=256, NH=8, DHQK=256, DHV=512)
SLSTM_CFG = dict(B=16, S=2048, NH=4, DH=256)


# ---------------------------------------------------------------------------------------------- algorithmic work
def chunkwise_bytes(B, NH, S, DHQK, DHV, **_):
    """q,k,v in and h out (bf16) plus i,f (fp32) per token-head; final C/n/m once per (batch, head)."""
    return B * NH * (S * (2 * (2 * DHQK + 2 * DHV) + 8) + (DHQK * DHV + DHQK + 1) * 4)


def chunkwise_flops(B, NH, S, DHQK, DHV, chunk, **_):
    return B * NH * S * (4 * DHQK * DHV + 2 * chunk * (DHQK + DHV) + 4 * DHQK)


def step_bytes(B, NH, DHQK, DHV, **_):
    """C read+write, n read+write, m read+write (fp32); q,k,v in, h out (bf16); i,f (fp32)."""
    return B * NH * (2 * DHQK * DHV * 4 + 2 * DHQK * 4 + 8 + 2 * DHQK * 2 + 2 * DHV * 2 + 8)


def slstm_bytes(B, S, NH, DH, **_):
    H = NH * DH
    return S * B * 4 * H * 2 + S * B * H * 2 + NH * DH * 4 * DH * 2 + 2 * 4 * B * H * 4


# ---------------------------------------------------------------------------------------------- helpers
def chunkwise_inputs(seed, B, NH, S, DHQK, DHV, **_):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, NH, S, DHQK, generator=g) / DHQK ** 0.5).bfloat16()
    k = (torch.randn(B, NH, S, DHQK, generator=g) / DHQK ** 0.5).bfloat16()
    v = torch.randn(B, NH, S, DHV, generator=g).bfloat16()
    i = torch.randn(B, NH, S, generator=g)
    f = torch.randn(B, NH, S, generator=g) + 3.0
    return [q, k, v, i, f]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while kernels run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def count(self):
        return len(self.lines)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0])); mx = float(parts[1])
            except ValueError:
                continue
            for nme, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nme)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


def measured_peak_hbm():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ---------------------------------------------------------------------------------------------- CPU reference arm
def cpu_chunkwise_seconds(threads):
    """Reference's native chunkwise formulation (oracle port) on one sequence of the workload, all host cores."""
    from oracle import mlstm as O
    torch.set_num_threads(threads)
    q, k, v, i, f = [t.float() for t in chunkwise_inputs(0, **dict(CFG, B=1))]
    t0 = time.perf_counter()
    O.mlstm_chunkwise(q, k, v, i, f, chunk_size=CFG["chunk"])
    return time.perf_counter() - t0


CPU_SAMPLE = "one sequence (B=1 of 4, all 8 heads, S=8192) per step; native chunkwise formulation in fp32 torch"


def headline_config(world):
    """The `config` object of the headline line: the same for both arms."""
    return {"workload": "mlstm_chunkwise_7b_heads", **CFG, "parallelism": f"dp{world}",
            "l2": "inputs (%d MB per step) exceed the 126 MB L2" % (chunkwise_bytes(**CFG) // 10 ** 6)}


def run_reference(args, rank, json_out):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    times = []
    for it in range(args.warmup + args.steps):
        dt = cpu_chunkwise_seconds(threads)
        if it >= args.warmup:
            times.append(dt)
    total = sum(times)
    val = CFG["S"] * len(times) / total
    print(json.dumps({
        "impl": "reference", "metric": "mlstm_chunkwise_prefill_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": CPU_SAMPLE},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), file=json_out, flush=True)


# ---------------------------------------------------------------------------------------------- the reference's own sLSTM CUDA backend
def reference_root():
    for cand in (os.environ.get("XLSTM_REFERENCE"), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "xlstm")):
            return cand
    return None


def slstm_reference_cuda(cfg, dev, our_ms):
    """Times the reference's sLSTM cell with backend="cuda" (xlstm/blocks/slstm/src/cuda/slstm_forward.cu:217-267: a host
    loop of one cuBLAS call and one pointwise kernel per time step, JIT-compiled as compute_80 PTX) at the same cell
    shape on this GPU.  Needs the reference package and a working nvcc on the machine; reports why when it cannot."""
    root = reference_root()
    if root is None:
        return {"reference_cuda_unavailable": "reference package not found (XLSTM_REFERENCE or baseline/_ref)"}
    try:
        if root not in sys.path:
            sys.path.insert(0, root)
        os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(ROOT, "baseline", "_ref_ext"))
        from xlstm.blocks.slstm.cell import sLSTMCell, sLSTMCellConfig
        B, S, NH, DH = cfg["B"], cfg["S"], cfg["NH"], cfg["DH"]
        torch.manual_seed(0)
        cell = sLSTMCell(sLSTMCellConfig(hidden_size=NH * DH, num_heads=NH, backend="cuda", dtype="bfloat16", batch_size=B,
                                         recurrent_weight_init="standard")).to(dev).eval()
        x = torch.randn(B, S, 4 * NH * DH, device=dev).bfloat16()
        with torch.no_grad():
            for _ in range(2):
                cell(x)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                cell(x)
            e1.record()
            torch.cuda.synchronize()
        ref_ms = e0.elapsed_time(e1) / 3
        return {"reference_cuda_ms": ref_ms, "speedup_vs_reference_cuda": ref_ms / our_ms,
                "reference_cuda": "sLSTMCell(backend='cuda') forward through the reference's own cell class, same shape"}
    except Exception as e:   # no compiler, no reference sources, ...
        return {"reference_cuda_unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


def slstm_training(cfg, dev):
    """The training path of the same cell: the cache-writing forward, the backward-through-time kernel and the two sums
    for the recurrent matrix and the bias (library GEMM), device-timed; beside it the reference's backend="cuda" cell
    doing forward + backward at the same shape (slstm.cc:53-254: host loops of cuBLAS calls and pointwise kernels)."""
    from xlstm_b200 import ops
    B, S, NH, DH = cfg["B"], cfg["S"], cfg["NH"], cfg["DH"]
    H = NH * DH
    g = torch.Generator(device=dev).manual_seed(9)
    wx = torch.randn(B, S, 4 * H, device=dev, generator=g).bfloat16()
    R = ((torch.rand(NH, DH, 4, DH, device=dev, generator=g) * 2 - 1) / H ** 0.5).bfloat16()
    bias = torch.randn(NH, 4, DH, device=dev, generator=g) * 0.5
    gh = torch.randn(B, NH, S, DH, device=dev, generator=g).bfloat16()

    def timed(fn, n=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    out = {}
    h, last, cache = ops.slstm_forward(wx, R, bias, train_cache=True)
    out["forward_with_cache_ms"] = timed(lambda: ops.slstm_forward(wx, R, bias, train_cache=True))
    out["backward_kernel_ms"] = timed(lambda: ops.slstm_backward(cache, R, gh))
    dwx, _ = ops.slstm_backward(cache, R, gh)
    out["weight_grads_ms"] = timed(lambda: ops.slstm_weight_grads(dwx, h))
    out["fwd_bwd_ms"] = out["forward_with_cache_ms"] + out["backward_kernel_ms"] + out["weight_grads_ms"]
    out["cache_bytes"] = cache.numel()
    out["kernel"] = "slstm_backward_kernel<%d>" % DH
    del cache, dwx
    root = reference_root()
    if root is None:
        out["reference_cuda_unavailable"] = "reference package not found (XLSTM_REFERENCE or baseline/_ref)"
        return {"training": out}
    try:
        if root not in sys.path:
            sys.path.insert(0, root)
        os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(ROOT, "baseline", "_ref_ext"))
        from xlstm.blocks.slstm.cell import sLSTMCell, sLSTMCellConfig
        torch.manual_seed(0)
        cell = sLSTMCell(sLSTMCellConfig(hidden_size=H, num_heads=NH, backend="cuda", dtype="bfloat16", batch_size=B,
                                         recurrent_weight_init="standard")).to(dev).train()
        x = wx.clone().requires_grad_()

        def ref_step():
            cell.zero_grad(set_to_none=True)
            x.grad = None
            o, _ = cell(x)
            o.backward(gh)

        out["reference_cuda_fwd_bwd_ms"] = timed(ref_step, n=3)
        out["speedup_vs_reference_cuda"] = out["reference_cuda_fwd_bwd_ms"] / out["fwd_bwd_ms"]
    except Exception as e:
        out["reference_cuda_unavailable"] = f"{type(e).__name__}: {str(e)[:200]}"
    return {"training": out}


def slstm_gate_projections(cfg, dev):
    """The front of the same sLSTM layer: four headwise gate projections + concatenation at the cell's shape, as ONE
    kernel (xl_headwise_proj) and as the reference layer's eager operators (four einsum calls and torch.cat,
    xlstm/components/linear_headwise.py:75-82, xlstm/blocks/slstm/layer.py:145-154), device-timed."""
    import xlstm_b200
    B, S, NH, DH = cfg["B"], cfg["S"], cfg["NH"], cfg["DH"]
    D = NH * DH
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(B, S, D, device=dev, generator=g).bfloat16()
    xc = torch.randn(B, S, D, device=dev, generator=g).bfloat16()
    ws = [(torch.randn(NH, DH, DH, device=dev, generator=g) / DH ** 0.5).bfloat16() for _ in range(4)]

    def eager():
        outs = []
        for w, inp in zip(ws, (xc, xc, x, x)):
            outs.append(torch.einsum("...hd,hod->...ho", inp.view(B, S, NH, DH), w).reshape(B, S, D))
        return torch.cat(outs, dim=-1)

    def timed(fn, n=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    ours = timed(lambda: xlstm_b200.headwise_proj([x, xc], ws, [1, 1, 0, 0]))
    ref = timed(eager)
    nbytes = (2 + 4) * B * S * D * 2 + 4 * NH * DH * DH * 2   # both inputs read, four gate planes written, weights once
    peak, src = measured_peak_hbm()
    return {"gate_projections": {"kernel": "headwise_proj_pair_kernel<%d>" % DH, "ms": ours, "eager_ms": ref, "speedup_vs_eager": ref / ours,
                                 "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / ours / 1e6,
                                 "frac_of_hbm_peak": nbytes / ours / 1e6 / peak, "peak_source": src,
                                 "flops": 2 * 4 * B * S * NH * DH * DH}}


# ---------------------------------------------------------------------------------------------- GPU cases
def build_case(name, dev, rank):
    """Returns dict(step=callable on device-resident inputs, e2e_step=callable with host buffers or None,
    units=work units per step, ...)."""
    import xlstm_b200
    if name in ("chunkwise", "chunkwise_b1"):
        cfg = dict(CFG) if name == "chunkwise" else dict(CFG, B=1)
        host = [t.pin_memory() for t in chunkwise_inputs(1234 + rank, **cfg)]
        q, k, v, i, f = [t.to(dev) for t in host]
        h_host = torch.empty(cfg["B"], cfg["NH"], cfg["S"], cfg["DHV"], dtype=torch.bfloat16).pin_memory()
        c_host = torch.empty(cfg["B"], cfg["NH"], cfg["DHQK"], cfg["DHV"], dtype=torch.float32).pin_memory()

        def step():
            return xlstm_b200.mlstm_sequence(q, k, v, i, f, kernel="chunkwise")

        def e2e_step():   # host buffers in, host buffers out: uploads, kernels and downloads of the pieces overlap
            xlstm_b200.mlstm_sequence_from_host(*host, h_host, c_host, device=dev)

        return dict(step=step, e2e_step=e2e_step, units=cfg["B"] * cfg["S"], unit="tokens/s",
                    metric="mlstm_chunkwise_prefill_tokens_per_s", workload="mlstm_chunkwise_7b_heads", cfg=cfg,
                    bytes=chunkwise_bytes(**cfg), flops=chunkwise_flops(**cfg), kernel="mlstm_chunkwise_kernel<256>",
                    h2d=sum(t.numel() * t.element_size() for t in host), d2h=h_host.numel() * 2 + c_host.numel() * 4,
                    l2="inputs (%d MB per step) exceed the 126 MB L2" % (chunkwise_bytes(**cfg) // 10 ** 6), launches=1,
                    traffic=178.2e6 * cfg["B"],
                    traffic_source="constant: ncu dram__bytes_read.sum + dram__bytes_write.sum of ONE captured launch at B=1, scaled by the number of sequences, not measured in this run")
    if name == "step":
        cfg = dict(STEP_CFG)
        B, NH, DQ, DV = cfg["B"], cfg["NH"], cfg["DHQK"], cfg["DHV"]
        g = torch.Generator().manual_seed(99 + rank)
        host = [(torch.randn(B, NH, DQ, generator=g) / DQ ** 0.5).bfloat16().pin_memory(),
                (torch.randn(B, NH, DQ, generator=g) / DQ ** 0.5).bfloat16().pin_memory(),
                torch.randn(B, NH, DV, generator=g).bfloat16().pin_memory(),
                torch.randn(B, NH, 1, generator=g).pin_memory(), (torch.randn(B, NH, 1, generator=g) + 3).pin_memory()]
        q, k, v, i, f = [t.to(dev) for t in host]
        state = [torch.zeros(B, NH, DQ, DV, device=dev), torch.zeros(B, NH, DQ, device=dev), torch.zeros(B, NH, 1, device=dev)]
        h_host = torch.empty(B, NH, DV, dtype=torch.bfloat16).pin_memory()

        def step():
            h, (c, n, m) = xlstm_b200.mlstm_step(q, k, v, i, f, *state)
            state[1], state[2] = n, m
            return h

        def e2e_step():
            dq, dk, dv, di, df = [t.to(dev, non_blocking=True) for t in host]
            h, (c, n, m) = xlstm_b200.mlstm_step(dq, dk, dv, di, df, *state)
            state[1], state[2] = n, m
            h_host.copy_(h, non_blocking=True)

        return dict(step=step, e2e_step=e2e_step, units=B, unit="stream-steps/s (8 heads of one layer)",
                    metric="mlstm_step_stream_steps_per_s", workload="mlstm_step_7b_heads", cfg=cfg, bytes=step_bytes(**cfg),
                    flops=B * NH * 4 * DQ * DV, kernel="mlstm_step_kernel<bf16>",
                    h2d=sum(t.numel() * t.element_size() for t in host), d2h=h_host.numel() * 2,
                    l2="state pool (%d MB) exceeds the 126 MB L2" % (B * NH * DQ * DV * 4 // 10 ** 6), launches=1,
                    traffic=2.101e9, traffic_source="constant: ncu dram__bytes_read.sum + dram__bytes_write.sum of ONE captured launch of this workload, not measured in this run")
    if name == "slstm":
        cfg = dict(SLSTM_CFG)
        B, S, NH, DH = cfg["B"], cfg["S"], cfg["NH"], cfg["DH"]
        H = NH * DH
        g = torch.Generator().manual_seed(7 + rank)
        wx_h = torch.randn(B, S, 4 * H, generator=g).bfloat16().pin_memory()
        R = ((torch.rand(NH, DH, 4, DH, generator=g) * 2 - 1) / H ** 0.5).bfloat16().to(dev)
        bias = (torch.randn(NH, 4, DH, generator=g) * 0.5).to(dev)
        wx = wx_h.to(dev)
        o_host = torch.empty(B, NH, S, DH, dtype=torch.bfloat16).pin_memory()

        def step():
            return xlstm_b200.slstm_forward(wx, R, bias)

        def e2e_step():
            d = wx_h.to(dev, non_blocking=True)
            o, st = xlstm_b200.slstm_forward(d, R, bias)
            o_host.copy_(o, non_blocking=True)

        return dict(step=step, e2e_step=e2e_step, units=B * S, unit="tokens/s", metric="slstm_forward_tokens_per_s",
                    workload="slstm_cell_config3", cfg=cfg, bytes=slstm_bytes(**cfg), flops=S * B * NH * 2 * DH * 4 * DH,
                    kernel="slstm_forward_kernel<256>", h2d=wx_h.numel() * 2, d2h=o_host.numel() * 2,
                    l2="inputs (%d MB) exceed the 126 MB L2" % (slstm_bytes(**cfg) // 10 ** 6), launches=1,
                    traffic=323.9e6, traffic_source="constant: ncu dram__bytes_read.sum + dram__bytes_write.sum of ONE captured launch of this workload, not measured in this run",
                    extra=lambda m: {**slstm_reference_cuda(cfg, dev, m["kernel_ms"]), **slstm_gate_projections(cfg, dev), **slstm_training(cfg, dev)})
    if name == "slstm_train":
        # one training step of the same cell: cache-writing forward, backward through time, dR / dbias GEMMs
        from xlstm_b200 import ops
        cfg = dict(SLSTM_CFG)
        B, S, NH, DH = cfg["B"], cfg["S"], cfg["NH"], cfg["DH"]
        H = NH * DH
        g = torch.Generator().manual_seed(7 + rank)
        wx_h = torch.randn(B, S, 4 * H, generator=g).bfloat16().pin_memory()
        gh_h = torch.randn(B, NH, S, DH, generator=g).bfloat16().pin_memory()
        R = ((torch.rand(NH, DH, 4, DH, generator=g) * 2 - 1) / H ** 0.5).bfloat16().to(dev)
        bias = (torch.randn(NH, 4, DH, generator=g) * 0.5).to(dev)
        wx, gh = wx_h.to(dev), gh_h.to(dev)
        dwx_host = torch.empty(B, S, 4 * H, dtype=torch.bfloat16).pin_memory()

        def train(wx_d, gh_d):
            h, last, cache = ops.slstm_forward(wx_d, R, bias, train_cache=True)
            dwx, ds0 = ops.slstm_backward(cache, R, gh_d)
            dR, db = ops.slstm_weight_grads(dwx, h)
            return dwx, dR, db

        def step():
            return train(wx, gh)

        def e2e_step():
            dwx, dR, db = train(wx_h.to(dev, non_blocking=True), gh_h.to(dev, non_blocking=True))
            dwx_host.copy_(dwx, non_blocking=True)

        cache_bytes = ((B + 15) // 16) * NH * (DH // 32) * S * 128 * 96
        # Wx and h of the forward, the cache written and read back, dh in, dWx out, then h and dWx once more for the GEMMs
        nbytes = slstm_bytes(**cfg) + 2 * cache_bytes + B * S * H * 2 + B * S * 4 * H * 2 + B * S * 5 * H * 2
        return dict(step=step, e2e_step=e2e_step, units=B * S, unit="tokens/s", metric="slstm_forward_backward_tokens_per_s",
                    workload="slstm_cell_training_config3", cfg=cfg, bytes=nbytes, flops=3 * S * B * NH * 2 * DH * 4 * DH,
                    kernel="slstm_backward_kernel<256>", h2d=(wx_h.numel() + gh_h.numel()) * 2, d2h=dwx_host.numel() * 2,
                    l2="cache and activations (%d MB per step) exceed the 126 MB L2" % (nbytes // 10 ** 6), launches=2,
                    traffic=None, traffic_source="not captured")
    if name == "headwise":
        # the four headwise gate projections + concatenation in front of the sLSTM cell, at the cell's benchmark shape
        cfg = dict(SLSTM_CFG)
        B, S, NH, DH = cfg["B"], cfg["S"], cfg["NH"], cfg["DH"]
        D = NH * DH
        g = torch.Generator().manual_seed(5 + rank)
        host = [torch.randn(B, S, D, generator=g).bfloat16().pin_memory() for _ in range(2)]
        x, xc = [t.to(dev) for t in host]
        ws = [(torch.randn(NH, DH, DH, generator=g) / DH ** 0.5).bfloat16().to(dev) for _ in range(4)]
        out_host = torch.empty(B, S, 4 * D, dtype=torch.bfloat16).pin_memory()

        def step():
            return xlstm_b200.headwise_proj([x, xc], ws, [1, 1, 0, 0])

        def e2e_step():
            xd, xcd = [t.to(dev, non_blocking=True) for t in host]
            out_host.copy_(xlstm_b200.headwise_proj([xd, xcd], ws, [1, 1, 0, 0]), non_blocking=True)

        nbytes = (2 + 4) * B * S * D * 2 + 4 * NH * DH * DH * 2
        return dict(step=step, e2e_step=e2e_step, units=B * S, unit="tokens/s", metric="slstm_gate_projections_tokens_per_s",
                    workload="slstm_layer_gate_projections_config3", cfg=cfg, bytes=nbytes, flops=2 * 4 * B * S * NH * DH * DH,
                    kernel="headwise_proj_pair_kernel<256>", h2d=2 * B * S * D * 2, d2h=4 * B * S * D * 2,
                    l2="operands (%d MB per step) exceed the 126 MB L2" % (nbytes // 10 ** 6), launches=1,
                    traffic=355.2e6, traffic_source="constant: ncu dram__bytes_read.sum + dram__bytes_write.sum of ONE captured launch of this workload (part of the last stores is still in L2 when the kernel ends), not measured in this run")
    if name == "layer_ops":
        # the two fused operators next to the cell, at the 7B layer's prefill shapes (8 x 8192 tokens, D = 4096)
        B, S, NH, DH = 8, 8192, 8, 512
        D = NH * DH
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        x = torch.randn(B, S, D, device=dev, generator=g).bfloat16()
        y = torch.randn(B, S, D, device=dev, generator=g).bfloat16()
        h = torch.randn(B, NH, S, DH, device=dev, generator=g).bfloat16()
        o = torch.randn(B, S, D, device=dev, generator=g).bfloat16()
        w = torch.ones(D, device=dev).bfloat16()
        host = [t.cpu().pin_memory() for t in (x, y, h, o)]
        out_host = [torch.empty(B, S, D, dtype=torch.bfloat16).pin_memory() for _ in range(2)]

        def step():
            xlstm_b200.add_rmsnorm(x, w, y)
            return xlstm_b200.headnorm_gate(h, o, w)

        def e2e_step():
            xd, yd, hd, od = [t.to(dev, non_blocking=True) for t in host]
            out_host[0].copy_(xlstm_b200.add_rmsnorm(xd, w, yd)[1], non_blocking=True)
            out_host[1].copy_(xlstm_b200.headnorm_gate(hd, od, w), non_blocking=True)

        cfg = dict(B=B, S=S, NH=NH, DH=DH, D=D)
        # add+norm reads x, y and writes x_new, normed; norm+gate reads h, o and writes out (the weights stay in L2)
        return dict(step=step, e2e_step=e2e_step, units=B * S, unit="tokens/s", metric="layer_adjacent_ops_tokens_per_s",
                    workload="xlstm7b_layer_add_rmsnorm_plus_headnorm_gate", cfg=cfg, bytes=7 * B * S * D * 2, flops=0,
                    kernel="add_rmsnorm_kernel<bf16> + headnorm_gate_kernel<bf16>", h2d=4 * B * S * D * 2,
                    d2h=2 * B * S * D * 2, l2="operands (7 x %d MB per step) exceed the 126 MB L2" % (B * S * D * 2 // 10 ** 6), launches=2,
                    traffic=863.3e6 * B / 2, traffic_source="constant: ncu dram__bytes_read.sum + dram__bytes_write.sum of ONE captured launch of both kernels at B=2, scaled by B, not measured in this run")
    if name == "continuous7b":
        # Continuous batching on the xLSTM-7B-shaped model (random init): 512 documents of log-normal length (median 1024,
        # sigma 1.0, clipped to [16, 16384]) are prefilled PACKED into rows of 32768 tokens (cu_seqlens, state reset inside
        # the kernels) and decoded in 256 state slots for 256 greedy tokens each; finished streams hand their slot to the
        # next queued document.  Documents are data-parallel: every rank takes its share (longest-first balancing) and
        # 256 / world slots; no collective on the data path.
        from xlstm_b200.large_model import ContinuousDecoder, LargeConfig, LargeModel, procedural_state_dict
        from xlstm_b200.sharding import shard_documents
        import torch.distributed as dist
        world = dist.get_world_size() if dist.is_initialized() else 1
        mcfg = LargeConfig(embedding_dim=4096, num_heads=8, num_blocks=32, vocab_size=50304)
        sd = procedural_state_dict(mcfg, seed=0, dtype=torch.bfloat16, device=dev, gen_device=dev)
        model = LargeModel(mcfg, sd, dev, torch.bfloat16)
        del sd
        torch.cuda.empty_cache()
        NDOC, NSLOT, GEN = 512, 256, 256
        g = torch.Generator().manual_seed(11)
        lens_all = torch.exp(torch.randn(NDOC, generator=g) + math.log(1024.0)).clamp(16, 16384).long().tolist()
        mine = shard_documents(lens_all, world)[rank if world > 1 else 0]
        lens = [lens_all[d] for d in mine]
        prompts_host = [torch.randint(0, mcfg.vocab_size, (n,), generator=g).pin_memory() for n in lens]
        prompts = [t.to(dev) for t in prompts_host]
        dec = ContinuousDecoder(model, NSLOT // world, row_len=32768, max_rows_per_prefill=2)

        def step():
            return dec.run(prompts, GEN)

        def e2e_step():   # prompts from pinned host memory; run() reads the generated tokens back to the host
            return dec.run([t.to(dev, non_blocking=True) for t in prompts_host], GEN)

        cfg = dict(model="xLSTM-7B-shaped (random init)", documents=NDOC, slots=NSLOT, new_tokens=GEN,
                   prompt_tokens=sum(lens_all), lengths="exp(N(ln 1024, 1)) clipped to [16,16384]", row_len=32768,
                   admission="packed prefill with cu_seqlens, per-document final states scattered into the slots")
        steps_est = len(mine) * GEN // max(NSLOT // world, 1)
        weight_bytes = sum(t.numel() * t.element_size() for t in model.parameters_on_device() if t is not model.embedding)
        return dict(step=step, e2e_step=e2e_step, teardown=model.release_graph, units=sum(lens) + len(mine) * GEN, unit="tokens/s",
                    metric="xlstm7b_continuous_decode_tokens_per_s", workload="xlstm7b_512docs_256slots_refill", cfg=cfg,
                    bytes=steps_est * (weight_bytes + 32 * step_bytes(NSLOT // world, 8, 256, 512)) + 32 * chunkwise_bytes(1, 8, sum(lens), 256, 512),
                    flops=0, kernel="whole run: packed prefills and graph-replayed decode steps over the slot pool",
                    h2d=sum(lens) * 8, d2h=(NSLOT // world) * steps_est * 8, l2="weights (13.7 GB) exceed the 126 MB L2",
                    launches=steps_est + 32 * 8, heavy=True,
                    extra=lambda m: {"prefill_calls_per_run": dec.prefill_calls // max(m["steps"] + m["warmup"] + m["e2e_steps"], 1)})
    if name == "decode7b":
        # one graph-replayed decode step of the 7B-shaped mirror at batch 8 (the unit the launch-list profile lists)
        from xlstm_b200.large_model import LargeConfig, LargeModel, procedural_state_dict
        mcfg = LargeConfig(embedding_dim=4096, num_heads=8, num_blocks=32, vocab_size=50304)
        sd = procedural_state_dict(mcfg, seed=0, dtype=torch.bfloat16, device=dev, gen_device=dev)
        model = LargeModel(mcfg, sd, dev, torch.bfloat16)
        del sd
        torch.cuda.empty_cache()
        tok = torch.randint(0, mcfg.vocab_size, (8, 128), generator=torch.Generator().manual_seed(5)).to(dev)
        model.generate(tok, 4, use_cuda_graph=True)   # prefill, capture
        weight_bytes = sum(t.numel() * t.element_size() for t in model.parameters_on_device() if t is not model.embedding)
        return dict(step=lambda: model._graph.replay(), e2e_step=lambda: model._graph.replay(), teardown=model.release_graph,
                    units=8, unit="tokens/s", metric="xlstm7b_decode_step_tokens_per_s", workload="xlstm7b_decode_step_batch8",
                    cfg=dict(model="xLSTM-7B-shaped (random init)", batch=8), bytes=weight_bytes + 32 * step_bytes(8, 8, 256, 512),
                    flops=0, kernel="one replay of the captured decode step (261 kernels)", h2d=0, d2h=0,
                    l2="weights (13.7 GB) exceed the 126 MB L2", launches=261)
    if name == "model7b":
        # xLSTM-7B-shaped model, random-init bf16: prefill 8 x 8192 tokens, then 512 greedy tokens.  Heads are
        # tensor-parallel over the ranks (strong scaling): dense layers are library GEMMs, the cell is ours.
        from xlstm_b200.large_model import LargeConfig, LargeModel, procedural_state_dict
        import torch.distributed as dist
        world = dist.get_world_size() if dist.is_initialized() else 1
        mcfg = LargeConfig(embedding_dim=4096, num_heads=8, num_blocks=32, vocab_size=50304)
        sd = procedural_state_dict(mcfg, seed=0, dtype=torch.bfloat16, device=dev, gen_device=dev)
        model = LargeModel(mcfg, sd, dev, torch.bfloat16, tp_rank=rank if world > 1 else 0, tp_world=world)
        del sd
        torch.cuda.empty_cache()
        B, S, GEN = 8, 8192, 512
        tok_host = torch.randint(0, mcfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(5)).pin_memory()
        tok_dev = tok_host.to(dev)
        out_host = torch.empty(B, GEN, dtype=torch.long).pin_memory()

        def step():   # the decode loop replays a CUDA graph (with tensor parallelism the NCCL all-reduces are part of it)
            return model.generate(tok_dev, GEN, use_cuda_graph=True)[0]

        def e2e_step():
            out_host.copy_(model.generate(tok_host.to(dev, non_blocking=True), GEN, use_cuda_graph=True)[0], non_blocking=True)

        streamed = [t for blk in model.blocks for k_, t in blk.items() if not k_.endswith("_full") and k_ not in ("qkvo", "if_w")]
        streamed += [model.out_norm, model.lm_head]
        weight_bytes = sum(t.numel() * t.element_size() for t in streamed)            # what one decode step streams per rank
        flops_per_token = 2 * (32 * (4096 * (2 * 2048 + 2 * 4096) + 4096 * 16 + 4096 * 4096 + 3 * 4096 * 10944)) + 32 * 8 * 623616

        def extra(m):
            """Prefill and decode timed apart, the collectives of the prefill, and both against their bounds."""
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            ev[0].record()
            model.forward(tok_dev, last_only=True)
            ev[1].record()
            model.forward(tok_dev, last_only=True, time_collectives=world > 1)
            ev[2].record()
            torch.cuda.synchronize()
            prefill_ms = ev[0].elapsed_time(ev[1])
            decode_ms = (m["kernel_ms"] - prefill_ms) / (GEN - 1)
            try:
                with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
                    pk = json.load(fh)
                tflops, hbm = float(pk["bf16_tflops_sustained"]), float(pk["hbm_gbs"])
            except Exception:
                tflops, hbm = 1400.0, 6650.0
            prefill_bound_ms = B * S * flops_per_token / (tflops * 1e12 * world) * 1e3
            decode_bound_ms = (weight_bytes + 32 * step_bytes(B, 8 // world, 256, 512)) / (hbm * 1e9) * 1e3
            out = {"prefill_ms": prefill_ms, "prefill_tokens_per_s": B * S / (prefill_ms * 1e-3), "decode_ms_per_step": decode_ms,
                   "prefill_frac_of_tensor_bound": prefill_bound_ms / prefill_ms, "decode_frac_of_weight_streaming_bound": decode_bound_ms / decode_ms,
                   "bounds": "prefill: %.1f GFLOP per token over the sustained bf16 peak of all ranks; decode: the rank's weights and "
                             "states streamed once per step over the measured HBM peak" % (flops_per_token / 1e9)}
            if world > 1:
                out["prefill_collectives"] = {
                    "scheme": "per block one all-gather (normed activations) + one reduce-scatter (out_proj partial sums) over the "
                              "token axis, two batch pieces on two streams; decode: two reductions per block inside the step graph",
                    "calls": model.comm_calls, "bytes_per_call": model.comm_bytes // max(model.comm_calls, 1),
                    "event_ms_sum": model.comm_ms,
                    "note": "CUDA-event time around each collective on its own stream, summed; the two streams overlap, so the sum "
                            "can exceed the share of the prefill the collectives expose",
                    "decode_all_reduce_bytes": B * 4096 * 2, "decode_all_reduces_per_step": 65,
                    "decode_reduce": ("one kernel per all-reduce + residual add + RMSNorm over peer memory (one-shot push)"
                                      if model.peer is not None else "NCCL all-reduce + add/norm kernel (%s)" % model.peer_unavailable)}
            return out

        cfg = dict(model="xLSTM-7B-shaped (random init)", embedding_dim=4096, num_heads=8, num_blocks=32, vocab_size=50304,
                   global_batch=B, seq_len=S, decode_tokens=GEN)
        return dict(step=step, e2e_step=e2e_step, teardown=model.release_graph, extra=extra, units=B * (S + GEN), unit="tokens/s",
                    metric="xlstm7b_prefill_decode_tokens_per_s", workload="xlstm7b_prefill8x8192_decode512", cfg=cfg,
                    # algorithmic bytes of one step per rank: the weights once per decoded token (and once for the prefill)
                    # plus the cell's prefill traffic; the decode loop is what the time goes to
                    bytes=(GEN + 1) * weight_bytes + 32 * chunkwise_bytes(B, 8 // world, S, 256, 512),
                    flops=B * S * flops_per_token / world, kernel="whole step: prefill (32 chunkwise launches + library GEMMs) and 511 graph replays",
                    h2d=tok_host.numel() * 8, d2h=out_host.numel() * 8,
                    l2="weights (13.7 GB) and activations exceed the 126 MB L2", launches=32 + 32 * GEN, scaling="strong",
                    parallelism="tp", heavy=True)
    raise SystemExit(f"unknown case {name}")


def measure(case, steps, warmup, world, rank, dev, e2e=True, sampler=None, hold_clocks=False):
    """Times `case` on the device (exactly `steps` steps between barriers, CUDA events on the launching stream, max over
    ranks) and end to end from host buffers.  Returns a dict of raw numbers."""
    import torch.distributed as dist
    import xlstm_b200

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step = case["step"]
    for _ in range(warmup):
        step()
    xlstm_b200.check_device_status(dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    barrier()
    if not case.get("heavy"):
        # one more untimed step directly in front of the first event: the host then queues the timed steps while the GPU
        # still works, as it does in steady state -- otherwise the first timed interval contains the host's launch
        # latency with the GPU idle (0.3 ms per step at 3 steps against 0.25 ms at 50)
        step()
    torch.cuda.profiler.start()   # (a profiler run with --profile-from-start off sees the timed steps only)
    ev[0].record()
    for i in range(steps):
        step()
        ev[i + 1].record()
    barrier()
    torch.cuda.profiler.stop()
    total_ms = ev[0].elapsed_time(ev[-1])
    kernel_ms = sum(ev[i].elapsed_time(ev[i + 1]) for i in range(steps)) / steps
    clocks = None
    e2e_ms, e2e_steps = float("nan"), 0
    if e2e:
        # the clock record needs a few hundred ms under load: keep the same step running, untimed, until it has samples
        # (not when the step holds collectives: rank 0 alone would wait for its peers for ever)
        if hold_clocks and rank == 0 and sampler is not None and sampler.proc is not None and case.get("parallelism") != "tp":
            t_end = time.time() + 3.0
            base = sampler.count()
            while sampler.count() < base + 8 and time.time() < t_end:
                for _ in range(1 if case.get("heavy") else 20):
                    step()
                torch.cuda.synchronize()
        if sampler is not None and rank == 0:
            clocks = sampler.stop()
        e2e_steps = 1 if case.get("heavy") else max(3, min(steps, 10))
        for _ in range(0 if case.get("heavy") else 2):
            case["e2e_step"]()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(e2e_steps):
            case["e2e_step"]()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)
    if world > 1:   # (every rank's own figures on stderr; the line carries the maximum)
        print(f"rank {rank}: {total_ms / steps:.4f} ms per step, kernel {kernel_ms:.4f} ms", file=sys.stderr, flush=True)
    t = torch.tensor([total_ms, e2e_ms, kernel_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, kernel_ms = t.tolist()
    xlstm_b200.check_device_status(dev)
    return dict(total_ms=total_ms, kernel_ms=kernel_ms, e2e_ms=e2e_ms, e2e_steps=e2e_steps, clocks=clocks, steps=steps, warmup=warmup)


def record(case, m, world):
    """The JSON fields of one measured case."""
    strong = case.get("scaling") == "strong"
    nrep = 1 if strong else world   # weak scaling: every rank processes its own units
    peak, peak_kind = measured_peak_hbm()
    achieved = case["bytes"] / (m["kernel_ms"] * 1e-3) / 1e9
    out = {
        "metric": case["metric"], "value": nrep * case["units"] * m["steps"] / (m["total_ms"] * 1e-3), "unit": case["unit"],
        "n_gpus": world, "steps": m["steps"], "warmup": m["warmup"], "ms_per_step": m["total_ms"] / m["steps"],
        "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": case["workload"], **case["cfg"], "parallelism": f"{case.get('parallelism', 'dp')}{world}", "l2": case["l2"]},
        "gpu_launches": m["steps"] * case["launches"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": case.get("traffic"),
                     "traffic_source": case.get("traffic_source", "not captured"),
                     "peak_source": peak_kind, "kernel": case["kernel"], "kernel_ms": m["kernel_ms"],
                     "algorithmic_bytes": case["bytes"], "tensor_tflops": case["flops"] / (m["kernel_ms"] * 1e-3) / 1e12},
    }
    if m["e2e_steps"]:
        out["e2e"] = {"value": nrep * case["units"] * m["e2e_steps"] / (m["e2e_ms"] * 1e-3), "unit": case["unit"],
                      "h2d_bytes_per_step": case["h2d"], "d2h_bytes_per_step": case["d2h"], "steps": m["e2e_steps"]}
    return out


def sub_record(name, dev, rank, world, steps, warmup):
    """One of the secondary measurements, reduced to what the headline line carries under "sub"."""
    case = build_case(name, dev, rank)
    m = measure(case, steps, warmup, world, rank, dev, e2e=True)
    r = record(case, m, world)
    out = {k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "scaling", "gpu_launches", "e2e")}
    out["config"] = r["config"]
    out["roofline"] = {k: r["roofline"][k] for k in ("bound", "achieved", "peak", "unit", "frac", "traffic", "traffic_source", "kernel", "kernel_ms")}
    if case.get("extra"):
        out.update(case["extra"](m))
    if case.get("teardown"):
        case["teardown"]()
    del case
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--case", default="all", choices=["all", "chunkwise", "chunkwise_b1", "step", "slstm", "slstm_train", "headwise", "layer_ops", "model7b", "decode7b", "continuous7b"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="profiling runs: device-resident loop only")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # stdout carries the one JSON line and nothing else: whatever libraries print on the way (the reference's JIT build
    # of its sLSTM extension prints its compiler flags) goes to stderr
    sys.stdout.flush()
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args, rank, json_out)
        return
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    import xlstm_b200  # noqa: F401

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    headline = "chunkwise" if args.case == "all" else args.case
    case = build_case(headline, dev, rank)
    sampler = ClockSampler(local)
    if rank == 0 and not args.no_e2e:
        sampler.start()
    heavy = bool(case.get("heavy"))
    m = measure(case, min(args.steps, 2) if heavy else args.steps, 1 if heavy else args.warmup, world, rank, dev,
                e2e=not args.no_e2e, sampler=sampler, hold_clocks=True)
    line = record(case, m, world)
    line["clocks"] = m["clocks"]
    if case.get("extra"):
        line.update(case["extra"](m))
    if case.get("teardown"):
        case["teardown"]()   # a live CUDA graph with NCCL kernels keeps the communicator from shutting down
    del case
    torch.cuda.empty_cache()

    if args.case == "all" and not args.no_e2e:
        # the other measurements of the path, in the same process (the model at tensor parallelism = world size)
        sub = {}
        if world == 1:
            for name in ("step", "slstm", "layer_ops"):
                sub[name] = sub_record(name, dev, rank, world, 20, 3)
        sub["model7b"] = sub_record("model7b", dev, rank, world, 1, 1)
        # continuous batching on the same model shape: documents data-parallel over the ranks (weak in slots per rank)
        sub["continuous7b"] = sub_record("continuous7b", dev, rank, world, 1, 1)
        line["sub"] = sub
    if headline == "chunkwise" and not args.no_cpu_baseline and world == 1 and not args.no_e2e and rank == 0:
        threads = os.cpu_count() or 1
        dt = cpu_chunkwise_seconds(threads)
        line["cpu_baseline"] = {"value": CFG["S"] / dt, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": CPU_SAMPLE}
    if rank == 0:
        print(json.dumps(line), file=json_out, flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
