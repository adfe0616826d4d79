"""Benchmark of the mLSTM chunkwise prefill kernel on BASELINE config 2 (xLSTM-7B head shapes).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload ("config.workload" = mlstm_chunkwise_7b_heads): one step = one forward of the mLSTM cell over
B=4 sequences x NH=8 heads x S=8192 tokens, DHQK=256, DHV=512, bf16 inputs, fp32 state, zero initial state;
seeded synthetic inputs with the distributions BASELINE.json states.  The metric counts B*S tokens per step
(each token = all 8 heads of one 7B layer).  At N > 1 every rank runs its own batch of sequences (documents
are data-parallel, no collective on the data path): weak scaling.

`--impl reference` times the reference's native CPU formulation (the oracle port) on the host cores.
"""
from __future__ import annotations

import argparse
import json
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
METRIC = "mlstm_chunkwise_prefill_tokens_per_s"


def algorithmic_bytes(B, NH, S, DHQK, DHV, **_):
    """q,k,v in and h out (bf16) plus i,f (fp32) per token-head, final C/n/m once per (batch, head)."""
    per_token_head = 2 * (2 * DHQK + 2 * DHV) + 8
    per_bh = (DHQK * DHV + DHQK + 1) * 4
    return B * NH * (S * per_token_head + per_bh)


def algorithmic_flops(B, NH, S, DHQK, DHV, chunk, **_):
    return B * NH * S * (4 * DHQK * DHV + 2 * chunk * (DHQK + DHV) + 4 * DHQK)


def make_inputs(seed, device, B, NH, S, DHQK, DHV, pinned=False, **_):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, NH, S, DHQK, generator=g) / DHQK ** 0.5).bfloat16()
    k = (torch.randn(B, NH, S, DHQK, generator=g) / DHQK ** 0.5).bfloat16()
    v = torch.randn(B, NH, S, DHV, generator=g).bfloat16()
    i = torch.randn(B, NH, S, generator=g)
    f = torch.randn(B, NH, S, generator=g) + 3.0
    host = [q, k, v, i, f]
    if pinned:
        host = [t.pin_memory() for t in host]
    return host, [t.to(device) for t in host]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

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


def cpu_native(sample_B, sample_NH, threads):
    """The reference's native chunkwise formulation on the host cores (oracle port), on a slice of the workload."""
    from oracle import mlstm as O
    torch.set_num_threads(threads)
    cfg = dict(CFG, B=sample_B, NH=sample_NH)
    host, _ = make_inputs(0, "cpu", **cfg)
    q, k, v, i, f = [t.float() for t in host]
    t0 = time.perf_counter()
    O.mlstm_chunkwise(q, k, v, i, f, chunk_size=CFG["chunk"])
    return time.perf_counter() - t0


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    # one step = the full head set of one sequence (B=1): 1/4 of the GPU step, scaled by tokens
    times = []
    for it in range(args.warmup + args.steps):
        dt = cpu_native(1, CFG["NH"], threads)
        if it >= args.warmup:
            times.append(dt)
    tok = CFG["S"] * len(times)
    total = sum(times)
    val = tok / total
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "mlstm_chunkwise_7b_heads", **CFG, "sample": "B=1 of 4 per step"},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": "one sequence (B=1, all 8 heads, S=8192) per step; native chunkwise formulation in fp32 torch"},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    import xlstm_b200

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    host, devt = make_inputs(1234 + rank, dev, pinned=True, **CFG)
    q, k, v, i, f = devt
    tokens_per_step = CFG["B"] * CFG["S"]

    def step():
        return xlstm_b200.mlstm_sequence(q, k, v, i, f, kernel="chunkwise")

    for _ in range(args.warmup):
        step()
    xlstm_b200.check_device_status(dev)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # ---- device-resident throughput: K steps, inputs (824 MB) exceed L2 (126 MB) so every step streams from HBM
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    ev[0].record()
    for s in range(args.steps):
        step()
        ev[s + 1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    kernel_ms = sum(ev[s].elapsed_time(ev[s + 1]) for s in range(args.steps)) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the public call with HOST buffers: pinned H2D of q,k,v,i,f, kernel, D2H of h and the state
    h_host = torch.empty(CFG["B"], CFG["NH"], CFG["S"], CFG["DHV"], dtype=torch.bfloat16).pin_memory()
    c_host = torch.empty(CFG["B"], CFG["NH"], CFG["DHQK"], CFG["DHV"], dtype=torch.float32).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = h_host.numel() * 2 + c_host.numel() * 4

    def e2e_step():
        dq, dk, dv, di, df = [t.to(dev, non_blocking=True) for t in host]
        h, (c, n, m) = xlstm_b200.mlstm_sequence(dq, dk, dv, di, df, kernel="chunkwise")
        h_host.copy_(h, non_blocking=True)
        c_host.copy_(c, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    t = torch.tensor([total_ms, e2e_ms, kernel_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, kernel_ms = t.tolist()
    xlstm_b200.check_device_status(dev)

    if rank == 0:
        value = world * tokens_per_step * args.steps / (total_ms * 1e-3)
        e2e_val = world * tokens_per_step * e2e_steps / (e2e_ms * 1e-3)
        peak, peak_kind = measured_peak_hbm()
        abytes = algorithmic_bytes(**CFG)
        achieved = abytes / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "mlstm_chunkwise_7b_heads", **CFG, "parallelism": f"dp{world}",
                       "l2": "inputs (824 MB per step) exceed the 126 MB L2"},
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
            "gpu_launches": args.steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": peak_kind, "kernel": "mlstm_chunkwise_kernel<256>",
                         "kernel_ms": kernel_ms, "algorithmic_bytes": abytes,
                         "tensor_tflops": algorithmic_flops(**CFG) / (kernel_ms * 1e-3) / 1e12},
        }
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            dt = cpu_native(1, CFG["NH"], threads)
            line["cpu_baseline"] = {"value": CFG["S"] / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": "one sequence (B=1, all 8 heads, S=8192), native chunkwise formulation, fp32 torch"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
