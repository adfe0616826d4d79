"""Benchmark of the xLSTM recurrent-cell kernels on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--case NAME]

Headline case (default, "chunkwise"): BASELINE config 2 -- one step = one forward of the mLSTM cell over
B=4 sequences x NH=8 heads x S=8192 tokens, DHQK=256, DHV=512, bf16 inputs, fp32 state, zero initial state;
seeded synthetic inputs with the distributions BASELINE.json states.  The metric counts B*S tokens per step
(one token = all 8 heads of one xLSTM-7B layer).  At N > 1 every rank runs its own batch of sequences
(documents are data-parallel, no collective on the data path): weak scaling.

Other cases print the same kind of line for the other kernels of the path:
  step          mLSTM decode step, 256 streams x 8 heads (xLSTM-7B head shapes), state resident in HBM
  slstm         sLSTM forward, BASELINE config 3 cell shape (B=16, S=2048, NH=4, DH=256)
  chunkwise_b1  the headline kernel on one sequence (B=1): the size used for profiler captures
  model7b       BASELINE config 4: xLSTM-7B-shaped model (random init, bf16), prefill 8 x 8192 tokens + 512 greedy
                tokens; heads tensor-parallel over the ranks (strong scaling); use e.g. --steps 2 --warmup 3

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


def run_reference(args, rank):
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
        "config": {"workload": "mlstm_chunkwise_7b_heads", **CFG, "sample": "B=1 of 4 per step"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": CPU_SAMPLE},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


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
                    # dram read+write of one captured launch at B=1 (profiles/mlstm_chunkwise_config2.md), scaled by B
                    traffic=178.2e6 * cfg["B"])
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
                    traffic=2.101e9)  # profiles/mlstm_step_256streams.md
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
                    traffic=323.9e6)  # profiles/slstm_forward_config3.md
    if name == "layer_ops":
        # the two fused operators next to the cell, at the 7B layer's prefill shapes (8 x 8192 tokens, D = 4096)
        B, S, NH, DH = int(os.environ.get("XL_LAYER_OPS_B", "8")), 8192, 8, 512   # (a smaller B for profiler captures)
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
                    # dram read+write of both kernels captured at B=2 (profiles/layer_adjacent_ops.md), scaled by B
                    traffic=863.3e6 * B / 2)
    if name == "continuous7b":
        # BASELINE config 5 in small: documents of log-normal length through a pool of decode slots with refill
        # (xLSTM-7B-shaped mirror, random init; 128 documents, 64 slots, 64 greedy tokens each)
        from xlstm_b200.large_model import ContinuousDecoder, LargeConfig, LargeModel, procedural_state_dict
        mcfg = LargeConfig(embedding_dim=4096, num_heads=8, num_blocks=32, vocab_size=50304)
        sd = procedural_state_dict(mcfg, seed=0, dtype=torch.bfloat16, device=dev, gen_device=dev)
        model = LargeModel(mcfg, sd, dev, torch.bfloat16)
        del sd
        torch.cuda.empty_cache()
        NDOC, NSLOT, GEN = 128, 64, 64
        g = torch.Generator().manual_seed(11)
        lens = torch.exp(torch.randn(NDOC, generator=g) + 6.0).clamp(16, 2048).long().tolist()
        prompts_host = [torch.randint(0, mcfg.vocab_size, (n,), generator=g).pin_memory() for n in lens]
        prompts = [t.to(dev) for t in prompts_host]
        dec = ContinuousDecoder(model, NSLOT)

        def step():
            return dec.run(prompts, GEN)

        def e2e_step():   # prompts from pinned host memory; run() reads the generated tokens back to the host
            return dec.run([t.to(dev, non_blocking=True) for t in prompts_host], GEN)

        cfg = dict(model="xLSTM-7B-shaped (random init)", documents=NDOC, slots=NSLOT, new_tokens=GEN,
                   prompt_tokens=sum(lens), lengths="exp(N(6,1)) clipped to [16,2048]")
        steps_est = NDOC * GEN // NSLOT
        return dict(step=step, e2e_step=e2e_step, teardown=model.release_graph, units=sum(lens) + NDOC * GEN, unit="tokens/s",
                    metric="xlstm7b_continuous_decode_tokens_per_s", workload="xlstm7b_128docs_64slots_refill", cfg=cfg,
                    bytes=(steps_est + NDOC) * sum(t.numel() * t.element_size() for t in model.parameters_on_device() if t is not model.embedding),
                    flops=0, kernel="whole run: single-document prefills and graph-replayed decode steps over the slot pool",
                    h2d=sum(lens) * 8, d2h=NSLOT * steps_est * 8, l2="weights (13.7 GB) exceed the 126 MB L2",
                    launches=steps_est + 32 * NDOC, heavy=True)
    if name == "model7b":
        # BASELINE config 4: xLSTM-7B-shaped model, random-init bf16, prefill 8 x 8192 tokens then 512 greedy tokens.
        # Heads are tensor-parallel over the ranks (strong scaling): dense layers are library GEMMs, the cell is ours.
        from xlstm_b200.large_model import LargeConfig, LargeModel, procedural_state_dict
        import torch.distributed as dist
        world = dist.get_world_size() if dist.is_initialized() else 1
        mcfg = LargeConfig(embedding_dim=4096, num_heads=8, num_blocks=32, vocab_size=50304)
        sd = procedural_state_dict(mcfg, seed=0, dtype=torch.bfloat16, device=dev, gen_device=dev)
        model = LargeModel(mcfg, sd, dev, torch.bfloat16, tp_rank=rank if world > 1 else 0, tp_world=world,
                           fused_adjacent=os.environ.get("XL_FUSED_ADJACENT", "1") != "0")
        del sd
        torch.cuda.empty_cache()
        B, S, GEN = 8, 8192, 512
        tok_host = torch.randint(0, mcfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(5)).pin_memory()
        tok_dev = tok_host.to(dev)
        out_host = torch.empty(B, GEN, dtype=torch.long).pin_memory()

        # the decode loop replays a CUDA graph (with tensor parallelism the NCCL all-reduces are part of it)
        graphed = os.environ.get("XL_DECODE_GRAPH", "1") == "1"

        def step():
            return model.generate(tok_dev, GEN, use_cuda_graph=graphed)[0]

        def e2e_step():
            out_host.copy_(model.generate(tok_host.to(dev, non_blocking=True), GEN, use_cuda_graph=graphed)[0], non_blocking=True)

        cfg = dict(model="xLSTM-7B-shaped (random init)", embedding_dim=4096, num_heads=8, num_blocks=32, vocab_size=50304,
                   global_batch=B, seq_len=S, decode_tokens=GEN)
        return dict(step=step, e2e_step=e2e_step, teardown=model.release_graph, units=B * (S + GEN), unit="tokens/s", metric="xlstm7b_prefill_decode_tokens_per_s",
                    workload="xlstm7b_prefill8x8192_decode512", cfg=cfg,
                    # algorithmic bytes of one step per rank: the weights once per decoded token (and once for the prefill)
                    # plus the cell's prefill traffic; the decode loop is what the time goes to
                    bytes=(GEN + 1) * sum(t.numel() * t.element_size() for t in model.parameters_on_device() if t is not model.embedding)
                    + 32 * chunkwise_bytes(B, 8 // world, S, 256, 512),
                    flops=0, kernel="whole step: prefill (32 chunkwise launches + library GEMMs) and 512 graph replays", h2d=tok_host.numel() * 8, d2h=out_host.numel() * 8,
                    l2="weights (13.7 GB) and activations exceed the 126 MB L2", launches=32 + 32 * GEN, scaling="strong",
                    parallelism="tp", heavy=True)
    raise SystemExit(f"unknown case {name}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--case", default="chunkwise", choices=["chunkwise", "chunkwise_b1", "step", "slstm", "layer_ops", "model7b", "continuous7b"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="profiling runs: device-resident loop only")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    args.warmup = max(args.warmup, 3)

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

    case = build_case(args.case, dev, rank)
    step = case["step"]
    sampler = ClockSampler(local)
    if rank == 0 and not args.no_e2e:
        sampler.start()
    for _ in range(args.warmup):
        step()
    xlstm_b200.check_device_status(dev)

    # ---- device-resident throughput: exactly K steps between barriers, one CUDA event per step
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    ev[0].record()
    for s in range(args.steps):
        step()
        ev[s + 1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    kernel_ms = sum(ev[s].elapsed_time(ev[s + 1]) for s in range(args.steps)) / args.steps

    e2e_ms, e2e_steps = float("nan"), 0
    if not args.no_e2e:
        # the clock record needs a few hundred ms under load: keep the same step running, untimed, until it has samples
        # (not when the step holds collectives, as the tensor-parallel model step does: rank 0 alone would wait for
        # its peers for ever -- and those steps run for seconds anyway, the record is long enough)
        if rank == 0 and sampler.proc is not None and case.get("parallelism") != "tp":
            t_end = time.time() + 3.0
            base = sampler.count()
            while sampler.count() < base + 8 and time.time() < t_end:
                for _ in range(1 if case.get("heavy") else 20):
                    step()
                torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
        # ---- end to end through the public call with HOST buffers (pinned H2D of the inputs, kernel, D2H of the result)
        e2e_steps = 1 if case.get("heavy") else max(3, min(args.steps, 10))
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
    else:
        clocks = None

    t = torch.tensor([total_ms, e2e_ms, kernel_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, kernel_ms = t.tolist()
    xlstm_b200.check_device_status(dev)

    if rank == 0:
        strong = case.get("scaling") == "strong"
        nrep = 1 if strong else world   # weak scaling: every rank processes its own units
        value = nrep * case["units"] * args.steps / (total_ms * 1e-3)
        peak, peak_kind = measured_peak_hbm()
        achieved = case["bytes"] / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": case["metric"], "value": value, "unit": case["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": case["workload"], **case["cfg"], "parallelism": f"{case.get('parallelism', 'dp')}{world}", "l2": case["l2"]},
            "gpu_launches": args.steps * case["launches"],
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": case.get("traffic"), "traffic_source": "ncu dram__bytes_read+write of one launch, see profiles/",
                         "peak_source": peak_kind, "kernel": case["kernel"], "kernel_ms": kernel_ms,
                         "algorithmic_bytes": case["bytes"], "tensor_tflops": case["flops"] / (kernel_ms * 1e-3) / 1e12},
        }
        if not args.no_e2e:
            line["e2e"] = {"value": nrep * case["units"] * e2e_steps / (e2e_ms * 1e-3), "unit": case["unit"],
                           "h2d_bytes_per_step": case["h2d"], "d2h_bytes_per_step": case["d2h"], "steps": e2e_steps}
        if args.case == "chunkwise" and not args.no_cpu_baseline and world == 1 and not args.no_e2e:
            threads = os.cpu_count() or 1
            dt = cpu_chunkwise_seconds(threads)
            line["cpu_baseline"] = {"value": CFG["S"] / dt, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": CPU_SAMPLE}
        print(json.dumps(line))
    if case.get("teardown"):
        case["teardown"]()   # a live CUDA graph with NCCL kernels keeps the communicator from shutting down
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
