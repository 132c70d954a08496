#!/usr/bin/env python
"""Benchmark of the low-precision attention path (and the block quantizers).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one causal attention forward + backward over one batch of synthetic
input of the Llama-3-8B attention shape (B=2, Hq=32, Hkv=8, S=8192, D=128;
bf16 N(0,1) Q/K with RoPE theta=5e5, V ~ N(0,1), dO ~ N(0,1e-2)).  With N > 1
(torchrun, one rank per GPU) that ONE problem is partitioned by (batch, kv head):
16 units, 16 / N per rank, no collective on the data path ("strong" scaling;
value = the problem's FLOPs over the slowest rank's time).  Rank 0 prints one JSON line.

value   : algorithmic TFLOP/s (6 causal matmuls: 2 forward, 4 backward), inputs resident in HBM
e2e     : same metric through FA4AttentionWrapper + autograd with q, k, v, dO copied from pinned host
          memory every step and O, dQ, dK, dV copied back to pinned host memory every step (uploads of
          the next step and downloads of the previous one overlap the kernels on two more streams);
          the returned tensors are compared with the resident-input run's
roofline: the backward kernel against the FP4/FP8 tensor peaks measured in the same run by an
          MMA-only kernel of the library (all SMs, operands resident in shared memory)
With N > 1 the line also carries `weak_scaling` (every rank the whole shape) and `long_context_c5`
(S = 131072 sharded over the ranks through the context-parallel NCCL ring).
--impl reference times the CPU emulation (oracle/) of the same path on the host cores.

--workload picks other measurements, each printing one JSON line of its own and none of them the headline:
c3 (D = 64), c5 (S = 131072 forward through the context-parallel ring, strong scaling over the ranks), noncausal,
quant (block quantizers), project / project_small (NVFP4 projection GEMM), module / module_small (attention block
from hidden states to hidden states, forward and forward + backward; --no-fused for separate passes), small (profiler
case of the headline kernels: one eighth of the benchmark configuration, what one of eight GPUs holds of it).
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
for _p in (ROOT / "fp4-fa4_b200", ROOT / "oracle"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402

WORKLOADS = {
    "c2": dict(B=2, Hq=32, Hkv=8, S=8192, D=128),     # the benchmark configuration
    "small": dict(B=1, Hq=8, Hkv=2, S=8192, D=128),  # same tiles and sequence, 1/8 of the heads: profiler captures only
    "c3": dict(B=16, Hq=32, Hkv=8, S=4096, D=64),    # the D = 64 configuration (same FLOPs as c2)
    "c5": dict(B=1, Hq=32, Hkv=8, S=131072, D=128),  # long context: forward only, MXFP4 P.V, sequence sharded over the ranks
    "noncausal": dict(B=1, Hq=32, Hkv=32, S=32768, D=128),  # the reference's historical inference shape: unmasked forward only
    # NVFP4 projection GEMMs (rows = tokens): the Llama-3-8B QKV projection, and a quarter of its rows for profiler captures
    "project": dict(M=16384, N=6144, K=4096),
    "project_small": dict(M=4096, N=6144, K=4096),
    # the block quantizers alone at the C4 shape [16384, 4096] (also a leg of the default run)
    "quant": dict(M=16384, K=4096),
    # module-level forward of one Llama-3-8B attention block (hidden 4096): projections + rotation + attention core
    "module": dict(B=2, Hq=32, Hkv=8, S=8192, D=128, hidden=4096),
    "module_small": dict(B=1, Hq=16, Hkv=4, S=4096, D=128, hidden=2048),  # profiler captures only
}
WORKLOAD = dict(WORKLOADS["c2"])
METRIC = "causal_attn_fwd_bwd_tflops"
UNIT = "TFLOP/s"


def causal_matmul_flops(B, Hq, S, D):
    return 2.0 * B * Hq * D * (S * (S + 1) / 2.0)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """SM clock and throttle-reason samples during the timed region (read-only NVML queries every
    10 ms from a host thread; nvidia-smi every 100 ms when the NVML binding is missing)."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.nvml, self.stop_flag = index, [], None, None, threading.Event()

    def _nvml_handle(self):
        import pynvml as N

        N.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(self.index).uuid)
        uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        return N, N.nvmlDeviceGetHandleByUUID(uuid)

    def start(self):
        try:
            self.nvml = self._nvml_handle()
            self.nvml[0].nvmlDeviceGetClockInfo(self.nvml[1], self.nvml[0].NVML_CLOCK_SM)
            threading.Thread(target=self._poll, daemon=True).start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _poll(self):
        N, h = self.nvml
        bits = (N.nvmlClocksEventReasonHwSlowdown, N.nvmlClocksEventReasonHwThermalSlowdown,
                N.nvmlClocksEventReasonSwThermalSlowdown, N.nvmlClocksEventReasonSwPowerCap)
        top = N.nvmlDeviceGetMaxClockInfo(h, N.NVML_CLOCK_SM)
        while not self.stop_flag.is_set():
            try:
                mask = N.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.rows.append([str(N.nvmlDeviceGetClockInfo(h, N.NVML_CLOCK_SM)), str(top)] +
                                 ["active" if mask & b else "not active" for b in bits])
            except Exception:
                pass
            time.sleep(0.01)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.nvml is None and self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"]}
        if self.nvml is not None:
            self.stop_flag.set()
        else:
            time.sleep(0.15)
            self.proc.terminate()
        rows = [r for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(int(r[0]) for r in rows)
        reasons = [n for i, n in enumerate(self.NAMES) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows),
                "source": "nvml, 10 ms" if self.nvml is not None else "nvidia-smi, 100 ms"}


def make_inputs(seed, device, pin=False):
    """Synthetic C2 inputs, generated on the CPU so that every rank/arm sees the same values."""
    import fa4b_oracle as O

    q, k, v, do = O.make_attention_inputs(WORKLOAD["B"], WORKLOAD["Hq"], WORKLOAD["Hkv"], WORKLOAD["S"], WORKLOAD["D"],
                                          seed=seed, rope=True, do_std=0.01)
    host = [t.pin_memory() if pin else t for t in (q, k, v, do)]
    return host, [t.to(device) for t in host]


def cpu_emulation_rate(seconds_budget=12.0, S=4096):
    """The oracle's forward + backward of one (batch, kv-head) unit (4 query heads) at a reduced
    sequence length, as algorithmic TFLOP/s on the host cores."""
    import fa4b_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    D = WORKLOAD["D"]
    q, k, v, do = O.make_attention_inputs(1, 4, 1, S, D, seed=1, rope=True, do_std=0.01)
    flops = 6.0 * causal_matmul_flops(1, 4, S, D)
    reps, t_total = 0, 0.0
    while reps < 1 or (t_total < seconds_budget and reps < 256):
        t0 = time.perf_counter()
        fwd = O.attn_forward(q, k, v)
        O.attn_backward(q, k, v, fwd.o, fwd.lse, do)
        t_total += time.perf_counter() - t0
        reps += 1
    sec = t_total / reps
    return dict(value=flops / sec / 1e12, unit=UNIT, cores=torch.get_num_threads(), kind="port",
                sample=f"oracle fwd+bwd of 1 batch x 1 kv-head group (4 query heads) at S={S}, D={D}; {reps} reps, "
                       f"{sec:.2f} s each"), sec


def run_reference(args, rank, world):
    if rank != 0:
        return
    rates = []
    for _ in range(max(1, args.warmup and 1)):
        cpu_emulation_rate(seconds_budget=0.0, S=1024)
    t_steps = []
    for _ in range(args.steps):
        r, sec = cpu_emulation_rate(seconds_budget=0.0, S=4096)
        rates.append(r)
        t_steps.append(sec)
    best = rates[len(rates) // 2]
    value = sorted(x["value"] for x in rates)[len(rates) // 2]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * sum(t_steps) / len(t_steps), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 emulation of fp4_e2m1 x fp8_e4m3", "data": "synthetic",
        "config": {"workload": "C2 Llama-3-8B attention B2 Hq32 Hkv8 S8192 D128 causal fwd+bwd", "timed_sample": best["sample"]},
        "cpu_baseline": dict(best, value=value),
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def other_configurations(device):
    """The other configurations of the path on this GPU, for the record beside the headline (rank 0, one GPU each):
    C3 (D = 64, B16, S4096) forward + backward and C5's forward (S = 131072, MXFP4 P.V) as one rank's three block calls."""
    from fa4b import attention
    from fa4b import context_parallel as cp

    out = {}
    g = torch.Generator(device=device).manual_seed(7)
    B, Hq, Hkv, S, D = (WORKLOADS["c3"][k] for k in ("B", "Hq", "Hkv", "S", "D"))
    q, k, v = (torch.randn(B, h, S, D, device=device, generator=g).bfloat16() for h in (Hq, Hkv, Hkv))
    do = (torch.randn(B, Hq, S, D, device=device, generator=g) * 0.01).bfloat16()
    ws = attention.alloc_workspace(attention.make_dims(q, k, None, "e4m3_fp8"), device)

    def c3_step():
        o, lse, _ = attention.attn_forward(q, k, v, workspace=ws)
        attention.attn_backward(o, lse, do, ws)

    def timed(fn, warm, reps):
        for _ in range(warm):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        b.synchronize()
        return a.elapsed_time(b) / reps

    ms = timed(c3_step, 3, 5)
    ws.check_status()
    out["c3_B16_Hq32_Hkv8_S4096_D64_fwd_bwd"] = {"ms_per_step": ms, "tflops": 6.0 * causal_matmul_flops(B, Hq, S, D) / (ms * 1e-3) / 1e12}
    del q, k, v, do, ws
    B, Hq, Hkv, S, D = (WORKLOADS["c5"][k] for k in ("B", "Hq", "Hkv", "S", "D"))
    q, k, v = (torch.randn(B, h, S, D, device=device, generator=g).bfloat16() for h in (Hq, Hkv, Hkv))
    engine = cp.KernelEngine(pv_format="mxfp4_e8m0_block32")
    ms = timed(lambda: cp.ring_attention_forward(q, k, v, engine), 2, 3)
    out["c5_B1_Hq32_Hkv8_S131072_D128_fwd_mxfp4_pv_one_rank"] = {"ms_per_step": ms, "tflops": 2.0 * causal_matmul_flops(B, Hq, S, D) / (ms * 1e-3) / 1e12}
    return out


def quantizer_rates(device, reps=10):
    """C4: fused RMSNorm + NVFP4 (row + transposed) and MXFP4 of [16384, 4096] bf16, algorithmic GB/s."""
    import fa4b
    import fa4b_oracle as O

    M, K = 16384, 4096
    x, gamma = O.make_quantizer_inputs(M, K, seed=20260825)
    x, gamma = x.to(device), gamma.to(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    out = {}
    cases = {
        "rmsnorm_nvfp4_row_col": (lambda: fa4b.tk_fused_norm_quantize(x, gamma, 1e-6, encode_centric=False), 2 * M * K + 2 * K + 2 * (M * K // 2) + 2 * (M * K // 16) + 4 * M + 4),
        "nvfp4_row_col": (lambda: fa4b.tk_quantize_for_gemm(x, encode_centric=False), 2 * M * K + 2 * (M * K // 2) + 2 * (M * K // 16)),
        # the TK quantiser's own default recipe (one multiplication per element instead of an exact division)
        "nvfp4_row_col_encode_centric": (lambda: fa4b.tk_quantize_for_gemm(x, encode_centric=True), 2 * M * K + 2 * (M * K // 2) + 2 * (M * K // 16)),
        "mxfp4": (lambda: fa4b.mxfp4_quantize_for_gemm(x), 2 * M * K + M * K // 2 + M * K // 32),
        # learned-weight recipe (one scale per 16 x 16 tile), both orientations, on the same matrix
        "nvfp4_weight_dual": (lambda: fa4b.prepare_nvfp4_projection_weight_dual(x), 2 * M * K + 2 * (M * K // 2) + 2 * (M * K // 16)),
    }
    for name, (fn, nbytes) in cases.items():
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            flush.zero_()  # evict the 126 MB L2
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b))
        ms = sorted(ts)[len(ts) // 2]
        out[name] = {"gbs": nbytes / ms / 1e6, "ms": ms, "algorithmic_bytes": nbytes}
    # Llama-3-8B QKV projection [16384, 4096] x [6144, 4096]^T on prepared NVFP4 operands (tensor-bound: TFLOP/s)
    N = 6144
    w = (torch.randn(N, K, device=device) * 0.02).bfloat16()
    fr, sr, _, _, sg, _ = fa4b.tk_quantize_for_gemm(x, return_transpose=False, encode_centric=False)
    wq = fa4b.prepare_nvfp4_projection_weight(w)
    y = torch.empty(M, N, dtype=torch.bfloat16, device=device)
    st = torch.zeros(4, dtype=torch.int32, device=device)
    for _ in range(3):
        fa4b.project_nvfp4((fr, sr, sg), wq, out=y, status=st)
    ts = []
    for _ in range(reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fa4b.project_nvfp4((fr, sr, sg), wq, out=y, status=st)
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    if int(st[0]) != 0:
        raise RuntimeError(f"project_nvfp4: device-side wait gave up: {st.tolist()}")
    ms = sorted(ts)[len(ts) // 2]
    out["project_nvfp4_qkv_16384x6144x4096"] = {"tflops": 2.0 * M * N * K / ms / 1e9, "ms": ms}
    return out


def init_nccl(device):
    """Process group for the ranks torchrun started.  NCCL may print its version banner on standard output when the
    first communicator is built; standard output carries the one JSON line, so the banner goes to standard error."""
    import torch.distributed as dist

    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        dist.init_process_group("nccl", device_id=device)
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


def dram_traffic_from_profile(kernel: str, workload: str):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of `kernel` at `workload`, as recorded by the last ncu
    capture whose summary is committed under profiles/ (a line `dram_bytes_per_launch <kernel> <workload> <bytes>`);
    (None, None) when no such record exists.  Never measured inside a benchmark run: ncu replays the kernel."""
    import re

    for path in sorted((ROOT / "profiles").glob("*.md")):
        m = re.search(rf"^dram_bytes_per_launch\s+{re.escape(kernel)}\s+{re.escape(workload)}\s+(\d+)\s*$", path.read_text(), re.M)
        if m:
            return int(m.group(1)), f"profiles/{path.name}"
    return None, None


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist

    from fa4b import attention, fa4_attention, parallel

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        init_nccl(device)
    B, Hq, Hkv, S, D = (WORKLOAD[k] for k in ("B", "Hq", "Hkv", "S", "D"))
    G = Hq // Hkv
    # the launcher pins every rank to one host thread; generating the inputs may use this rank's share of the cores
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    # ONE problem of the configured shape for the whole job, partitioned by (batch, kv head): every rank generates the
    # same global tensors from the same seed and keeps its own units; no collective on the data path
    host_global, _ = make_inputs(20260825, "cpu", pin=False)
    n_units = B * Hkv
    if world > n_units:
        raise SystemExit(f"{world} ranks for {n_units} (batch, kv-head) units")
    mine = parallel.shard_attention_inputs(host_global[0], host_global[1], host_global[2], rank, world, host_global[3])
    host = [t.contiguous().pin_memory() for t in (mine[0], mine[1], mine[2], mine[3])]  # q [U,G,S,D], k, v [U,1,S,D], dO
    del host_global, mine
    q, k, v, do = (t.to(device) for t in host)
    U = q.shape[0]
    # L2 hygiene: when a rank's inputs are smaller than twice the 126 MB L2 (a shard of the problem on many GPUs),
    # consecutive timed steps read different copies of them, enough copies to exceed 2x L2 together
    in_bytes = sum(t.numel() * t.element_size() for t in (q, k, v, do))
    n_rot = max(1, -(-(2 * (126 << 20)) // in_bytes))
    rot = [(q, k, v, do)] + [tuple(t.clone() for t in (q, k, v, do)) for _ in range(n_rot - 1)]
    flops_job = 6.0 * causal_matmul_flops(B, Hq, S, D)       # the whole job
    flops_rank = 6.0 * causal_matmul_flops(U, G, S, D)
    dims = attention.make_dims(q, k, None, "e4m3_fp8")
    ws = attention.alloc_workspace(dims, device)

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        e.record()  # creates the underlying handle
        return e

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed_steps(step_fn, n_warm, n_steps, sampler=None):
        for _ in range(n_warm):
            step_fn(None)
        sync()
        if sampler is not None:
            sampler.start()
        pairs = [[ev() for _ in range(4)] for _ in range(n_steps)]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        t0.record()
        for i in range(n_steps):
            step_fn(pairs[i])
        t1.record()
        sync()
        return t0.elapsed_time(t1), pairs

    result = {"n": 0}

    def step(events=None):
        e = events or [None] * 4
        q_, k_, v_, do_ = rot[result["n"] % n_rot]
        result["n"] += 1
        o, lse, _ = attention.attn_forward(q_, k_, v_, workspace=ws, events=(e[0], e[1]))
        result["o"] = o
        result["grads"] = attention.attn_backward(o, lse, do_, ws, events=(e[2], e[3]))

    sampler = ClockSampler(local_rank)
    ms_total, pairs = timed_steps(step, max(args.warmup, 3), args.steps, sampler if rank == 0 else None)
    clocks = sampler.stop() if rank == 0 else None
    ws.check_status()
    fwd_all = sorted(p[0].elapsed_time(p[1]) for p in pairs)
    bwd_all = sorted(p[2].elapsed_time(p[3]) for p in pairs)
    fwd_ms, bwd_ms = sum(fwd_all) / args.steps, sum(bwd_all) / args.steps
    resident = [result["o"].float().cpu()] + [t.float().cpu() for t in result["grads"]]
    plan = attention.backward_plan(dims)
    # This library's kernels per step: per-head amax, K/V publication, forward (quantises Q itself), dO publication,
    # backward, FP32-sum conversion. The driver's memset nodes are not counted.
    n_launches = 6

    def pct(v):  # p10 / median / p90 of the per-step kernel times
        n = len(v)
        return {"p10": v[int(0.1 * (n - 1))], "p50": v[n // 2], "p90": v[int(round(0.9 * (n - 1)))]}

    extras = not args.no_extras
    # ---- end to end through the public operator: host buffers, copies both ways inside the timed region
    wrapper = fa4_attention.FA4AttentionWrapper(fa4_attention.resolve_fa4_config(fa4_attention.FA4()), head_dim=D)
    # Two sets of device buffers: the copy stream uploads step i + 1's inputs from pinned host memory while step i
    # computes (the prefetch a training loop does), and step i's results (O, dQ, dK, dV) go back to pinned host memory
    # on a third stream while step i + 1 computes; every step's inputs and results cross PCIe inside the timed region.
    bufs = [tuple(torch.empty_like(t) for t in (q, k, v, do)) for _ in range(2)]
    out_host = [tuple(torch.empty(t.shape, dtype=torch.bfloat16).pin_memory() for t in (q, q, k, v)) for _ in range(2)]
    up_stream, down_stream = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    ready = [torch.cuda.Event() for _ in range(2)]
    free = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    drained = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]  # results stay referenced until their download has been issued

    def upload(i):
        with torch.cuda.stream(up_stream):
            up_stream.wait_event(free[i % 2])  # the step that last used this set has finished with it
            for dst, src in zip(bufs[i % 2], host):
                dst.copy_(src, non_blocking=True)
            ready[i % 2].record(up_stream)

    def e2e_step(i, last):
        if not last:
            upload(i + 1)
        main = torch.cuda.current_stream(device)
        main.wait_event(ready[i % 2])
        dq_, dk_, dv_, ddo = bufs[i % 2]
        qq, kk, vv = dq_.requires_grad_(True), dk_.requires_grad_(True), dv_.requires_grad_(True)
        out = wrapper(qq, kk, vv)
        out.backward(ddo)
        res = (out.detach(), qq.grad, kk.grad, vv.grad)
        computed[i % 2].record(main)
        free[i % 2].record(main)
        keep[i % 2] = res
        with torch.cuda.stream(down_stream):
            down_stream.wait_event(computed[i % 2])
            for dst, src in zip(out_host[i % 2], res):
                dst.copy_(src, non_blocking=True)
                src.record_stream(down_stream)
            drained[i % 2].record(down_stream)
        for t in (qq, kk, vv):
            t.grad = None
            t.requires_grad_(False)

    e2e_ms, e2e_check = float("nan"), None
    if extras:
        def e2e_run(n_steps, e0=None):
            for ev_ in free:
                ev_.record()
            if e0 is not None:
                up_stream.wait_event(e0)  # the first upload starts inside the timed region
            upload(0)
            for i in range(n_steps):
                e2e_step(i, last=(i == n_steps - 1))
            torch.cuda.current_stream(device).wait_stream(down_stream)  # the last results have landed on the host

        e2e_run(2)
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_run(args.steps, e0)
        e1.record()
        sync()
        e2e_ms = e0.elapsed_time(e1)
        # what came back over PCIe against the resident-input run of the same problem (dQ sums in another order)
        got = [t.float() for t in out_host[(args.steps - 1) % 2]]
        import fa4b_oracle as O
        diffs = {n: O.rel_l2(a, b) for n, a, b in zip(("o", "dq", "dk", "dv"), resident, got)}
        # dQ: its partial sums meet as f16 pairs in another order (7.5e-4 measured between two runs)
        e2e_check = {"rel_l2_vs_resident_run": diffs, "ok": bool(diffs["o"] == 0.0 and max(diffs.values()) < 4e-3)}
        if not e2e_check["ok"]:
            raise SystemExit(f"end-to-end results differ from the resident-input run: {diffs}")
        del bufs, keep

    # ---- secondary: every rank runs the whole configured shape on its own ("weak" scaling, global batch B * world)
    weak_ms = None
    if world > 1 and extras:
        host_w, (qw, kw, vw, dow) = make_inputs(20260825 + rank, device, pin=False)
        ws_w = attention.alloc_workspace(attention.make_dims(qw, kw, None, "e4m3_fp8"), device)

        def step_w(events=None):
            o, lse, _ = attention.attn_forward(qw, kw, vw, workspace=ws_w)
            attention.attn_backward(o, lse, dow, ws_w)

        weak_ms, _ = timed_steps(step_w, 3, args.steps)
        ws_w.check_status()
        del host_w, qw, kw, vw, dow, ws_w

    # ---- long-context configuration (C5) on the same ranks: the only part of the path with a collective
    c5 = run_c5_leg(device, rank, world) if (world > 1 and extras and args.workload == "c2") else None

    times = torch.tensor([ms_total, e2e_ms, weak_ms if weak_ms is not None else 0.0], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, weak_ms_max = (float(x) for x in times.cpu())
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    f1 = causal_matmul_flops(U, G, S, D)  # this rank's share: what its kernels were timed on
    # backward kernel: 4 algorithmic matmuls; 1 FP4 (score recompute) + 4 FP8 executed
    # tensor denominators: measured on this GPU by the library's own MMA-only run (all SMs, operands in shared
    # memory); the cuBLAS bf16 figure x2 / x4 is kept beside them for comparison
    from fa4b import microgate
    tp8, tp4 = microgate.tensor_peak("fp8"), microgate.tensor_peak("nvfp4")
    p8, p4 = tp8, tp4
    bwd_peak = 4.0 * f1 / (f1 / (p4 * 1e12) + 4.0 * f1 / (p8 * 1e12)) / 1e12
    bwd_ach = 4.0 * f1 / (bwd_ms * 1e-3) / 1e12
    fwd_peak = 2.0 * f1 / (f1 / (p4 * 1e12) + f1 / (p8 * 1e12)) / 1e12
    fwd_ach = 2.0 * f1 / (fwd_ms * 1e-3) / 1e12
    cpu = cpu_emulation_rate()[0] if (extras and world == 1) else None
    quant = quantizer_rates(device) if (extras and world == 1) else {}
    # one-GPU side measurements (C3, one rank's C5 block calls)
    others = other_configurations(device) if (extras and args.workload == "c2" and world == 1) else {}
    for qv in quant.values():
        if "gbs" in qv:
            qv["frac_of_hbm"] = qv["gbs"] / peaks["hbm_gbs"]
        else:
            qv["frac_of_nvfp4_peak"] = qv["tflops"] / p4
    nbytes_in = sum(t.numel() * t.element_size() for t in host)
    nbytes_out = sum(t.numel() * t.element_size() for t in out_host[0])
    traffic, traffic_source = dram_traffic_from_profile(f"attn_bwd_kernel<{D}>", args.workload) if world == 1 else (None, None)
    names = {"c2": "C2 Llama-3-8B attention B2 Hq32 Hkv8 S8192 D128 causal fwd+bwd",
             "c3": "C3 B16 Hq32 Hkv8 S4096 D64 causal fwd+bwd (not the headline configuration)",
             "small": "PROFILER CASE (not a benchmark result): B1 Hq8 Hkv2 S8192 D128 causal fwd+bwd"}
    line = {
        "metric": METRIC, "value": flops_job * args.steps / (ms_total * 1e-3) / 1e12, "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp4_e2m1 (QK^T) x fp8_e4m3/e5m2 (PV, gradients), f32 accumulate", "data": "synthetic",
        "config": {"workload": names[args.workload] + (f", ONE problem partitioned by (batch, kv head) over {world} GPUs: {U} of {n_units} units per GPU, no collective" if world > 1 else ""),
                   "global_batch": B, "units_per_gpu": U,
                   "l2": (f"a rank's inputs ({in_bytes >> 20} MiB bf16) exceed twice the 126 MB L2" if n_rot == 1 else
                          f"a rank's inputs are {in_bytes >> 20} MiB: consecutive steps read different copies ({n_rot} copies, {n_rot * in_bytes >> 20} MiB > 2x L2)"),
                   "flops": "6 causal matmuls = 12*B*Hq*D*S(S+1)/2", "includes": "Q/K/V quantisation and dO/statistics publication"},
        "clocks": clocks,
        "e2e": {"value": (flops_job * args.steps / (e2e_ms * 1e-3) / 1e12) if e2e_ms == e2e_ms else None, "unit": UNIT,
                "h2d_bytes_per_step": nbytes_in, "d2h_bytes_per_step": nbytes_out,
                "returns": "O, dQ, dK, dV to pinned host memory every step (third stream, overlapped with the next step)",
                "check": e2e_check},
        "gpu_launches": n_launches * args.steps,
        "roofline": {"bound": "tensor", "kernel": f"attn_bwd_kernel<{D}>", "achieved": bwd_ach, "peak": bwd_peak, "unit": UNIT,
                     "frac": bwd_ach / bwd_peak,
                     "traffic": traffic, "traffic_source": traffic_source, "ms_per_launch": bwd_ms,
                     "work_list": {"chunk_query_tiles": plan.chunk, "ctas": plan.grid, "split_key_rows_per_head": plan.split_rows},
                     "peak_source": (f"measured here: tcgen05 MMA-only run on all SMs, FP8 {tp8:.0f} TF/s, NVFP4 {tp4:.0f} TF/s, combined over the "
                                     f"kernel's FP4/FP8 mix ({peaks['source']} cuBLAS bf16 burst {peaks['bf16']} TF/s x2 / x4 would give "
                                     f"{2 * peaks['bf16']:.0f} / {4 * peaks['bf16']:.0f})"),
                     "tensor_peaks": {"fp8_tflops": tp8, "nvfp4_tflops": tp4},
                     "ms_per_launch_percentiles": pct(bwd_all),
                     "forward": {"achieved": fwd_ach, "peak": fwd_peak, "frac": fwd_ach / fwd_peak, "ms_per_launch": fwd_ms,
                                 "ms_per_launch_percentiles": pct(fwd_all)},
                     "whole_step": {"achieved": flops_rank / (ms_total / args.steps * 1e-3) / 1e12,
                                    "peak": 6.0 * f1 / (2.0 * f1 / (p4 * 1e12) + 5.0 * f1 / (p8 * 1e12)) / 1e12}},
        "cpu_baseline": cpu,
        "quantizers": quant,
        "other_configurations": others,
    }
    line["roofline"]["whole_step"]["frac"] = line["roofline"]["whole_step"]["achieved"] / line["roofline"]["whole_step"]["peak"]
    if world > 1 and extras:
        line["weak_scaling"] = {"value": world * 6.0 * causal_matmul_flops(B, Hq, S, D) * args.steps / (weak_ms_max * 1e-3) / 1e12, "unit": UNIT,
                                "ms_per_step": weak_ms_max / args.steps, "global_batch": B * world,
                                "note": "every rank runs the whole configured shape on inputs of its own"}
    if c5 is not None:
        line["long_context_c5"] = c5
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def c5_inputs(device, rank, Sl, B, Hq, Hkv, D):
    g = torch.Generator(device=device).manual_seed(20260825 + rank)

    def student_t(*shape):
        z = torch.randn(*shape, device=device, generator=g)
        chi = sum(torch.randn(*shape[:-1], 1, device=device, generator=g) ** 2 for _ in range(3)) / 3.0
        return (z / chi.sqrt()).bfloat16()

    q, k = student_t(B, Hq, Sl, D), student_t(B, Hkv, Sl, D)
    v = torch.randn(B, Hkv, Sl, D, device=device, generator=g).bfloat16()
    return q, k, v, g


def run_c5_leg(device, rank, world):
    """The long-context configuration as an extra of the default line when the job has several ranks: ONE sequence of
    131072 tokens sharded zig-zag over the ranks, quantised K/V shards round an NCCL ring.  Forward on the MXFP4 P.V
    route (the configuration's route; forward only, as the reference's diagnostic route is), and forward + backward
    on the FP8 P.V route, for which the backward exists.  Times are the slowest rank's."""
    import torch.distributed as dist

    from fa4b import context_parallel as cp

    B, Hq, Hkv, S, D = (WORKLOADS["c5"][k] for k in ("B", "Hq", "Hkv", "S", "D"))
    Sl = S // world
    q, k, v, g = c5_inputs(device, rank, Sl, B, Hq, Hkv, D)
    out = {"n_gpus": world, "scaling": "strong", "unit": UNIT,
           "workload": f"C5 B1 Hq32 Hkv8 S131072 D128 causal, one sequence over {world} ranks (zig-zag), Student-t(3) Q and K",
           "exchange": "NCCL ring (NVLS off) of quantised K/V chunks: 17.3 MB per chunk and hop forward; one all_reduce(MAX) of 40 amax words"}

    def timed(fn, warm, reps):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(reps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([t0.elapsed_time(t1) / reps], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    f1 = causal_matmul_flops(B, Hq, S, D)
    engine = cp.KernelEngine(pv_format="mxfp4_e8m0_block32")
    ms = timed(lambda: cp.ring_attention_forward(q, k, v, engine), 2, 3)
    out["forward_mxfp4_pv"] = {"ms_per_step": ms, "value": 2.0 * f1 / (ms * 1e-3) / 1e12}
    del engine
    engine8 = cp.KernelEngine()
    do = (torch.randn(B, Hq, Sl, D, device=device, generator=g) * 0.01).bfloat16()

    def fwd_bwd():
        o, lse, state = cp.ring_attention_forward(q, k, v, engine8, return_state=True)
        cp.ring_attention_backward(o, lse, do, state, engine8)

    ms = timed(fwd_bwd, 1, 2)
    out["forward_backward_fp8_pv"] = {"ms_per_step": ms, "value": 6.0 * f1 / (ms * 1e-3) / 1e12}
    return out


def run_c5(args, rank, world, local_rank):
    """Long-context forward (C5): the whole job is ONE sequence of 131072 tokens, sharded zig-zag over the ranks
    ("strong" scaling); quantised K/V shards travel round an NCCL ring.  Heavy-tailed (Student-t, 3 degrees of
    freedom) q and k, MXFP4 P.V route.  value = forward TFLOP/s of the whole job, max over ranks."""
    import torch.distributed as dist

    from fa4b import context_parallel as cp

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        init_nccl(device)
    B, Hq, Hkv, S, D = (WORKLOAD[k] for k in ("B", "Hq", "Hkv", "S", "D"))
    Sl = S // world
    q, k, v, _ = c5_inputs(device, rank, Sl, B, Hq, Hkv, D)
    engine = cp.KernelEngine(pv_format="mxfp4_e8m0_block32")
    sampler = ClockSampler(local_rank)
    for _ in range(max(args.warmup, 3)):
        cp.ring_attention_forward(q, k, v, engine)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        o, lse = cp.ring_attention_forward(q, k, v, engine)
    t1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    if world > 1:
        dist.barrier()
    times = torch.tensor([t0.elapsed_time(t1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms = float(times.item())
    if rank == 0:
        flops = 2.0 * causal_matmul_flops(B, Hq, S, D)
        print(json.dumps({
            "metric": "causal_attn_fwd_tflops_long_context", "value": flops * args.steps / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp4_e2m1 (QK^T) x mxfp4 (P.V), f32 accumulate", "data": "synthetic",
            "config": {"workload": f"C5 B1 Hq32 Hkv8 S131072 D128 causal forward, MXFP4 P.V, context parallel over {world} rank(s)",
                       "exchange": "NCCL ring of quantised K/V shards (17.3 MB per chunk per hop), one all_reduce(MAX) of 40 amax words",
                       "l2": "operands exceed L2", "includes": "amax, quantisation, ring, merges"},
            "clocks": clocks, "gpu_launches": None}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_noncausal(args, rank, world, local_rank):
    """Unmasked forward at the reference's non-causal inference shape (B1, S32768, H32, D128), both P.V formats,
    operands published beforehand as in the reference's measurement; FLOPs = 4*B*H*S^2*D."""
    from fa4b import attention

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    B, Hq, Hkv, S, D = (WORKLOAD[k] for k in ("B", "Hq", "Hkv", "S", "D"))
    g = torch.Generator(device=device).manual_seed(20260825)
    q, k, v = (torch.randn(B, h, S, D, device=device, generator=g).bfloat16() for h in (Hq, Hkv, Hkv))
    out = {}
    for pv in ("e4m3_fp8", "mxfp4_e8m0_block32"):
        dims = attention.make_dims(q, k, None, pv, causal=False)
        ws = attention.alloc_workspace(dims, device)
        attention.attn_prepare(q, k, v, ws)
        for _ in range(max(args.warmup, 3)):
            attention.attn_forward_prepared(ws, causal=False)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            attention.attn_forward_prepared(ws, causal=False)
        t1.record()
        torch.cuda.synchronize()
        ws.check_status()
        ms = t0.elapsed_time(t1) / args.steps
        out[pv] = {"ms": ms, "tflops": 4.0 * B * Hq * S * S * D / (ms * 1e-3) / 1e12}
    print(json.dumps({"metric": "noncausal_attn_fwd_tflops", "value": out["e4m3_fp8"]["tflops"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "ms_per_step": out["e4m3_fp8"]["ms"], "higher_is_better": True, "data": "synthetic",
                      "config": {"workload": "unmasked forward B1 H32 S32768 D128, operands published beforehand (not the headline configuration)"},
                      "by_pv_format": out}), flush=True)


def run_project(args, rank, world, local_rank):
    """y = x . w^T on prepared NVFP4 operands (activation 1x16 blocks, weight 16x16 tiles), the kernel alone."""
    import fa4b

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    M, N, K = (WORKLOAD[k] for k in ("M", "N", "K"))
    g = torch.Generator(device=device).manual_seed(20260825)
    x = torch.randn(M, K, device=device, generator=g).bfloat16()
    w = (torch.randn(N, K, device=device, generator=g) * 0.02).bfloat16()
    fr, sr, _, _, sg, _ = fa4b.tk_quantize_for_gemm(x, return_transpose=False, encode_centric=False)
    wq = fa4b.prepare_nvfp4_projection_weight(w)
    y = torch.empty(M, N, dtype=torch.bfloat16, device=device)
    st = torch.zeros(4, dtype=torch.int32, device=device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    for _ in range(max(args.warmup, 1)):
        fa4b.project_nvfp4((fr, sr, sg), wq, out=y, status=st)
    ts = []
    for _ in range(args.steps):
        flush.zero_()  # evict the 126 MB L2
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fa4b.project_nvfp4((fr, sr, sg), wq, out=y, status=st)
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    if int(st[0]) != 0:
        raise RuntimeError(f"project_nvfp4: device-side wait gave up: {st.tolist()}")
    ms = sorted(ts)[len(ts) // 2]
    from fa4b import microgate

    p4 = microgate.tensor_peak("nvfp4") if not args.no_extras else None
    print(json.dumps({"metric": "nvfp4_projection_tflops", "value": 2.0 * M * N * K / ms / 1e9, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True, "data": "synthetic",
                      "config": {"workload": f"NVFP4 projection [{M}, {K}] x [{N}, {K}]^T -> bf16, operands prepared beforehand (not the headline configuration)",
                                 "l2": "flushed between timed launches"},
                      "roofline": None if p4 is None else {"bound": "tensor", "achieved": 2.0 * M * N * K / ms / 1e9, "peak": p4, "unit": UNIT,
                                                           "frac": 2.0 * M * N * K / ms / 1e9 / p4,
                                                           "peak_source": "measured here: tcgen05 NVFP4 MMA-only run on all SMs"},
                      "gpu_launches": args.steps}), flush=True)


def run_module(args, rank, world, local_rank):
    """Forward of the attention block from hidden states to hidden states, per-step and per-stage times."""
    import fa4b
    from fa4b import attention
    from fa4b.lowp_module import LowpFA4AttentionBlock

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    B, Hq, Hkv, S, D, hidden = (WORKLOAD[k] for k in ("B", "Hq", "Hkv", "S", "D", "hidden"))
    g = torch.Generator(device=device).manual_seed(20260825)
    mk = lambda r, c: (torch.randn(r, c, device=device, generator=g) / c ** 0.5).bfloat16()
    # the QKV projection publishes the attention operands from its epilogue (no BF16 Q/K/V round trip)
    blk = LowpFA4AttentionBlock(mk(Hq * D, hidden), mk(Hkv * D, hidden), mk(Hkv * D, hidden), mk(hidden, Hq * D), Hq, Hkv, D,
                                fused_publish=not args.no_fused)
    x = torch.randn(B, S, hidden, device=device, generator=g).bfloat16()
    inv = 1.0 / (500000.0 ** (torch.arange(0, D, 2, device=device, dtype=torch.float64) / D))
    ang = torch.arange(S, device=device, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().bfloat16(), ang.sin().bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    for _ in range(max(args.warmup, 3)):
        blk(x, cos, sin)
    ts = []
    for _ in range(args.steps):
        flush.zero_()  # evict the 126 MB L2
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        blk(x, cos, sin)  # inference form: nothing kept for a backward
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    ms = sorted(ts)[len(ts) // 2]
    # forward + backward (input and weight gradients of both projections, attention backward, inverse rotation)
    dy = (torch.randn(B, S, hidden, device=device, generator=g) * 0.05).bfloat16()
    tb = []
    for i in range(args.steps + 1):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        y, mid = blk.forward(x, cos, sin, return_intermediates=True)
        blk.backward(dy, mid, cos, sin)
        b.record()
        b.synchronize()
        mid["workspace"].check_status()
        if i:
            tb.append(a.elapsed_time(b))
    ms_fb = sorted(tb)[len(tb) // 2]
    M = B * S
    flops = 2.0 * M * hidden * (Hq + 2 * Hkv) * D + 2.0 * M * hidden * Hq * D + 2.0 * causal_matmul_flops(B, Hq, S, D)
    flops_fb = 3.0 * (2.0 * M * hidden * (Hq + 2 * Hkv) * D + 2.0 * M * hidden * Hq * D) + 6.0 * causal_matmul_flops(B, Hq, S, D)
    print(json.dumps({"metric": "attention_block_fwd_tflops", "value": flops / ms / 1e9, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "data": "synthetic",
                      "config": {"workload": f"attention block forward B{B} S{S} hidden {hidden} Hq{Hq} Hkv{Hkv} D{D}: NVFP4 QKV projection, "
                                             "pair-native RoPE, NVFP4/FP8 causal attention, NVFP4 output projection (not the headline configuration)",
                                 "flops": "2*M*hidden*(Hq+2Hkv)*D + 2*M*hidden*Hq*D + 2 causal matmuls", "l2": "flushed between timed steps"},
                      "forward_backward": {"ms_per_step": ms_fb, "tflops": flops_fb / ms_fb / 1e9,
                                           "flops": "3x the projection matmuls + 6 causal matmuls"},
                      "fused_publication": not args.no_fused, "gpu_launches": (10 if not args.no_fused else 13) * args.steps}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=tuple(WORKLOADS), default="c2",
                    help="'small' is for profiler captures; its line is not a benchmark result")
    ap.add_argument("--no-extras", action="store_true", help="skip the CPU baseline, quantizer and end-to-end legs")
    ap.add_argument("--no-fused", action="store_true", help="module workload: separate projection, rotation and publication passes")
    args = ap.parse_args()
    WORKLOAD.update(WORKLOADS[args.workload])
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU fallback (use --impl reference for the CPU emulation)")
    if args.workload == "c5":
        run_c5(args, rank, world, local_rank)
        return
    if args.workload == "noncausal":
        if rank == 0:
            run_noncausal(args, rank, world, local_rank)
        return
    if args.workload.startswith("module"):
        if rank == 0:
            run_module(args, rank, world, local_rank)
        return
    if args.workload == "quant":
        if rank == 0:
            torch.cuda.set_device(local_rank)
            rates = quantizer_rates(torch.device("cuda", local_rank), reps=max(args.steps, 1))
            print(json.dumps({"metric": "block_quantizer_rates", "unit": "GB/s (algorithmic bytes) or TFLOP/s", "n_gpus": 1, "data": "synthetic",
                              "config": {"workload": "C4 [16384, 4096] bf16 (not the headline configuration)", "l2": "flushed between timed launches"},
                              "quantizers": rates}), flush=True)
        return
    if args.workload.startswith("project"):
        if rank == 0:
            run_project(args, rank, world, local_rank)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
