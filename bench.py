"""Benchmark of the factored-LSTM basecaller stack on B200 (sm_100a), one JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--quick]

Workload (the configuration the headline metric is quoted on): 5 factored-LSTM layers of
alternating direction, hidden 768, factor rank 128, T = 1000 timesteps, 1024 chunks PER GPU
(weak scaling: chunks are independent, every rank runs its own batch, no collective on the data
path). One "step" = one pass of the whole stack over one [T, B, 768] int8 batch.

    value            chunk-timesteps per second per layer, summed over GPUs
                     = n_gpus * B * T * layers / step_time   (inputs resident in HBM). The K steps
                     are independent passes over 1024-chunk batches; they run two at a time, side
                     by side in one [T, 2048, H] layer launch (chunks are independent: the bytes are
                     those of separate passes, tested), because the recurrence is a latency chain
                     whose step time barely depends on the rows in flight and one launch holds 16
                     row tiles; an odd last step runs alone. `one_pass_per_launch` beside it is
                     the same measurement with every step in a launch of its own.
    e2e              the same through the library's C streaming handle (fluke_flstm_stream_*, bound by
                     fluke_b200.lstm.StackPipeline) with HOST buffers: every step copies its input
                     from pinned host memory and its output back, all inside the timed region; the
                     handle overlaps the copies of neighbouring steps with the layers of the
                     current one and runs two consecutive steps side by side in one layer launch;
                     pipeline fill and drain included. `copy_only` beside it is the same copies
                     with no kernels (all ranks at once): the ceiling the host link sets.
    strong           the north star's own wording: 1024 chunks IN TOTAL sharded over the GPUs
                     (fluke_b200.shard.shard_range), same timing rule; at N = 1 it is `value`
    saturation       (N = 1) recurrence time per step of one layer against the batch size
    roofline         the persistent LSTM recurrence kernel of the timed region (tensor bound):
                     algorithmic FLOPs per launch / its launch duration, measured with CUDA events
                     on the launching stream, against the measured bf16 GEMM peak of this pool;
                     `traffic` from the ncu capture recorded in profiles/lstm_recurrence_traffic.json
    cpu_baseline     the CPU oracle (oracle/fluke_oracle.c, a port: the reference has no CPU
                     implementation of the LSTM contraction) on a bounded sample, all host cores;
                     the rate is extrapolated to the full workload
    ops              (N = 1) the other configurations of the path (rotary, RMSNorm(+quant), QKV
                     GEMM + rotary, dual GEMM + SiLU, fp8 twins, base GEMM, dequant-transposes) timed with
                     rotating buffers larger than L2, each with its CPU baseline timed in the same
                     run (the reference's own nn_cpu.c from oracle/_ref where it has the function,
                     else torch-CPU restatements of the reference tests' references, else the
                     oracle port) and an end-to-end figure with host buffers

`--impl reference` times the CPU oracle of the same workload on the host cores (bounded sample
per step) and prints the same line with "impl": "reference".
Synthetic seeded data throughout (weights N(0, 1/sqrt(fan_in)), inputs N(0,1)).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

T_STEPS, HIDDEN, RANK, LAYERS, CHUNKS_PER_GPU = 1000, 768, 128, 5, 1024
METRIC = "lstm_chunk_timesteps_per_sec_per_layer"
UNIT = "chunk-timesteps/s (per layer, summed over GPUs)"


# ---- helpers shared with the CPU tests -----------------------------------------------------------

def local_units(chunks, timesteps, layers):
    """Work units one rank processes per step (chunk-timesteps x layers)."""
    return chunks * timesteps * layers


def reduce_step_time(ms):
    """Max over ranks of a per-rank step time (identity without torch.distributed)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return ms
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def strong_scaling_record(total_chunks, world, ms, timesteps=T_STEPS, layers=LAYERS):
    """The strong-scaling sub-record: `total_chunks` in all, sharded over `world` ranks, one pass in
    `ms` milliseconds (max over ranks)."""
    from fluke_b200.shard import shard_range
    sizes = [e - b for b, e in (shard_range(total_chunks, r, world) for r in range(world))]
    return {"chunks_total": total_chunks, "chunks_per_gpu": max(sizes), "ms_per_step": ms,
            "value": total_chunks * timesteps * layers / (ms * 1e-3), "unit": UNIT}


def roofline_fractions(us, ops, bytes_, tensor_tops, hbm_gbs):
    """(frac_tensor, frac_hbm, frac_of_floor) of a kernel that needs `ops` operations and `bytes_`
    algorithmic bytes and ran `us` microseconds: achieved over the tensor peak, over the HBM copy
    bandwidth, and the larger of the two floors over the measured time."""
    t_tensor = ops / (tensor_tops * 1e12) * 1e6 if tensor_tops else 0.0
    t_hbm = bytes_ / (hbm_gbs * 1e9) * 1e6
    return (round(t_tensor / us, 3) if tensor_tops else None, round(t_hbm / us, 3), round(max(t_tensor, t_hbm) / us, 3))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        d = json.load(open(path))
        return dict(hbm_gbs=d["hbm_gbs"], tf_burst=d["bf16_tflops"], tf_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


def recurrence_traffic(kernel_name, row_tiles):
    """DRAM bytes per step of the recurrence kernel launched over `row_tiles` tiles of 128 chunks, from
    the ncu capture recorded under profiles/."""
    path = os.path.join(ROOT, "profiles", "lstm_recurrence_traffic.json")
    try:
        rec = json.load(open(path))
    except (OSError, ValueError):
        return None
    for k in rec.get("kernels", []):
        if k["kernel"] == kernel_name and k.get("row_tiles") == row_tiles:
            return k
    return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index, period_ms=200):
        self.idx, self.rows, self.proc, self.period = gpu_index, [], None, period_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        self.thread.join(2)
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 9 for i in range(4) if r[5 + i].lower() == "active"})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ---- CPU arm (oracle port) -------------------------------------------------------------------------

def host_cores():
    return os.cpu_count() or 1


def cpu_lstm_sample(seconds_target=15.0):
    """Times the CPU oracle on a bounded sample of the workload (1 layer, B chunks, T steps of
    the same shapes); returns (chunk-timesteps/s per layer, cores, description)."""
    import torch
    from fluke_b200 import prep
    from oracle import port
    cores = port.set_threads(host_cores())   # torchrun exports OMP_NUM_THREADS=1
    g = torch.Generator().manual_seed(42)
    H, R = HIDDEN, RANK

    def run(B, T):
        dn_ih, s_ih = prep.quantize_int8_rows(torch.randn(R, H, generator=g) / H ** 0.5)
        dn_hh, s_hh = prep.quantize_int8_rows(torch.randn(R, H, generator=g) / H ** 0.5)
        w_up = (torch.randn(4 * H, 2 * R, generator=g) / (2 * R) ** 0.5).half()
        bias = torch.randn(4 * H, generator=g) * 0.05
        x, xs = prep.quantize_int8_rows(torch.randn(T * B, H, generator=g))
        t0 = time.perf_counter()
        port.lstm_layer(x.view(T, B, H).numpy(), xs.numpy(), dn_ih.numpy(), s_ih.numpy(), dn_hh.numpy(), s_hh.numpy(),
                        w_up.numpy(), bias.numpy(), np.zeros((B, H), np.float32), np.zeros((B, H), np.int8))
        return time.perf_counter() - t0

    B = max(128, 8 * cores)
    probe = run(B, 4)
    T = int(max(4, min(1000, seconds_target / max(probe / 4, 1e-6))))
    sec = run(B, T)
    return B * T / sec, cores, f"1 layer, {B} chunks x {T} timesteps, H={H}, R={R}, OpenMP over chunks"


def cpu_gate_epilogue_reference():
    """The reference's own fluke_flstm_step_cpu (src/nn_cpu.c:247-285, compiled into oracle/_ref) on
    [1024, 768]: the gate epilogue of one timestep, in chunk-timesteps/s. None when oracle/_ref
    was not built."""
    from oracle import ref
    lib = ref.cpu()
    if lib is None:
        return None
    cores = host_cores()
    rng = np.random.default_rng(0)
    B, H = 1024, HIDDEN
    scratch = rng.standard_normal((B, 4 * H)).astype(np.float32)
    ih = rng.standard_normal((B, 4 * H)).astype(np.float32)
    cell = np.zeros((B, H), np.float32)
    hh = np.zeros((B, H), np.float32)
    P = ctypes.c_void_p
    args = [a.ctypes.data_as(P) for a in (scratch, ih, cell, hh)]
    lib.fluke_flstm_step_cpu(*args, B, H, cores)
    reps, t0 = 20, time.perf_counter()
    for _ in range(reps):
        lib.fluke_flstm_step_cpu(*args, B, H, cores)
    sec = (time.perf_counter() - t0) / reps
    return {"value": B / sec, "unit": "chunk-timesteps/s (gate epilogue only: fluke_flstm_step_cpu)", "cores": cores,
            "kind": "reference", "sample": f"[{B}, {H}] fp32, {reps} calls"}


# ---- GPU arm ----------------------------------------------------------------------------------------

def time_rotating(calls, iters, torch, sustain_s=0.0, gpu_index=0):
    """calls: list of zero-arg launchers on disjoint buffers (total footprint > L2); returns the
    mean milliseconds per call over `iters` rounds. The rounds are captured into one CUDA graph and
    the replay is timed with CUDA events, so the figure is the GPU's time for back-to-back
    launches, free of the Python/ctypes cost per call (which is of the order of these kernels'
    own 10-20 us). Falls back to timing the Python loop if the capture fails.
    With sustain_s > 0 the graph is also replayed back to back for that long with the SM clock
    sampled, and (ms, sustained_ms, clocks) is returned: the figure under the clock the kernel
    itself pulls; clocks["burst_sm_mhz"] is the clock during one more replay of the timed burst,
    measured from inside the GPU (GpuClockProbe)."""
    from fluke_b200 import lib as flib
    L = flib.load()
    for c in calls:
        c()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        prev = L.fluke_get_stream()
        with torch.cuda.stream(side):
            L.fluke_set_stream(side.cuda_stream)
            try:
                g.capture_begin()
                for _ in range(iters):
                    for c in calls:
                        c()
                g.capture_end()
            finally:
                L.fluke_set_stream(prev)
        graph = g
    except Exception:
        torch.cuda.synchronize()
        graph = None
    n = iters * len(calls)
    if graph is None:
        e0.record()
        for _ in range(iters):
            for c in calls:
                c()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        return (ms, None, None) if sustain_s > 0 else ms
    torch.cuda.synchronize()
    graph.replay()          # warm replay
    torch.cuda.synchronize()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    if sustain_s <= 0:
        return ms
    burst_mhz = None
    try:
        probe = GpuClockProbe(torch, ms * n).start()
        graph.replay()
        torch.cuda.synchronize()
        burst_mhz = probe.median_mhz(0.1 * ms * n, 0.9 * ms * n)
    except Exception:
        torch.cuda.synchronize()
    reps = max(1, int(sustain_s * 1e3 / max(ms * n, 1e-3)))
    sampler = ClockSampler(gpu_index, period_ms=100).start()
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["burst_sm_mhz"] = burst_mhz
    return ms, e0.elapsed_time(e1) / (n * reps), clocks


class GpuClockProbe:
    """The SM clock seen from inside the GPU while a burst of kernels runs: one thread on a side
    stream records (cycle counter, nanosecond timer) every 20 us (fluke_sm100_clock_samples of
    lib/libfluke_probe.so). nvidia-smi's samples are 100 ms apart; a dense tcgen05 kernel pulls the
    clock from its idle maximum down to the power limit's level within a few tens of microseconds,
    so a burst of a few milliseconds runs at a clock nvidia-smi never shows."""
    GAP_NS = 20000

    def __init__(self, torch, expected_ms):
        from fluke_b200 import lib as flib
        self.torch, self.fn = torch, flib.load_probe().fluke_sm100_clock_samples
        self.n = int(min(1 << 16, max(64, expected_ms * 1e6 / self.GAP_NS + 64)))
        self.buf = torch.zeros(2 * self.n, dtype=torch.int64, device="cuda")
        self.stream = torch.cuda.Stream()

    def start(self):
        rc = self.fn(self.buf.data_ptr(), self.n, self.GAP_NS, self.stream.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"fluke_sm100_clock_samples: CUDA error {rc}")
        return self

    def median_mhz(self, from_ms, to_ms):
        """Median clock over the samples taken between from_ms and to_ms after the first one."""
        v = self.buf.cpu().view(self.n, 2).double()
        t = (v[:, 1] - v[0, 1]) / 1e6
        mhz = (v[1:, 0] - v[:-1, 0]) / (v[1:, 1] - v[:-1, 1]).clamp_min(1.0) * 1e3
        sel = (t[1:] >= from_ms) & (t[1:] <= to_ms)
        return float(mhz[sel].median()) if bool(sel.any()) else None


def measure_tensor_peaks(torch):
    """tcgen05.mma issue-rate probe on every SM (operands resident in shared memory, no global
    traffic): the measured tensor-pipe ceilings for int8 / e4m3 / f16. MEASURED_PEAKS.json only has
    bf16 through cuBLAS, so the int8/fp8 fractions of the GEMM-class kernels are quoted against
    these. Two figures per type: with ZERO operands (nothing toggles, the clock stays at its
    maximum: the issue rate) and with pseudo-random operands for a few milliseconds (the board's
    power limit pulls the clock down: what the tensor pipe sustains on real data), each with the SM
    clock the probe itself measured (cycles / nanoseconds)."""
    from fluke_b200 import lib as flib
    fn = flib.load_probe().fluke_sm100_mma_peak
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    cyc = torch.zeros(2 * sms, dtype=torch.int64, device="cuda")
    out = {}
    for kind, name, kelems in ((0, "int8", 32), (1, "e4m3", 32), (2, "f16", 16)):
        rec = {}
        for pattern, iters, key in ((0, 16384, ""), (1, 49152, "_random_operands")):
            fn(kind, 256, iters, pattern, cyc.data_ptr(), sms, None)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(kind, 256, iters, pattern, cyc.data_ptr(), sms, None)
            e1.record()
            torch.cuda.synchronize()
            if rc != 0:
                continue
            v = cyc.view(sms, 2).double()
            ops = 2.0 * 128 * 256 * kelems * iters * sms
            rec["TOPs" + key] = round(ops / e0.elapsed_time(e1) / 1e9, 1)
            rec["ops_per_clk_per_sm" + key] = round(2.0 * 128 * 256 * kelems * iters / v[:, 0].mean().item(), 1)
            rec["sm_mhz" + key] = round(float((v[:, 0] / v[:, 1].clamp_min(1.0)).median()) * 1e3, 0)
        if rec:
            out[name] = rec
    return out


def _cpu_time(fn, min_reps=2, budget_s=2.0):
    fn()
    reps, t0 = 0, time.perf_counter()
    while reps < min_reps or (time.perf_counter() - t0 < budget_s and reps < 20):
        fn()
        reps += 1
    return (time.perf_counter() - t0) / reps


def _rotate_half_torch(c, sin, cos, seqlen, heads=8, hd=64, qk_cols=1024):
    """Rotate-half on the q and k heads of c [M, 1536] f32, position = row % seqlen (restates the
    torch reference of cute/test_rotary.py:95-107)."""
    import torch
    m = c.shape[0]
    pos = torch.arange(m) % seqlen
    s, co = sin[pos][:, None, :], cos[pos][:, None, :]
    qk = c[:, :qk_cols].reshape(m, 2 * heads, hd)
    x0, x1 = qk[..., :hd // 2], qk[..., hd // 2:]
    rot = torch.cat([x0 * co - x1 * s, x0 * s + x1 * co], dim=-1).reshape(m, qk_cols)
    return torch.cat([rot, c[:, qk_cols:]], dim=1).half()


def bench_ops(torch, peaks, tensor_peaks, gpu_index):
    """Configs 1-4 of the path and the other entry points of the library; each entry reports the
    kernel time, achieved GB/s or TOP/s, fractions of the measured HBM copy bandwidth and (GEMMs) of
    the measured tensor peak, the CPU baseline of the same operation timed now on the host cores,
    and an end-to-end time through the C ABI with pinned host buffers (copies inside)."""
    from fluke_b200 import ops, prep
    from oracle import port, ref
    dev = "cuda"
    out = {}
    g = torch.Generator().manual_seed(0)
    hbm = peaks["hbm_gbs"]
    cores = host_cores()
    sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    torch.set_num_threads(cores)
    port.set_threads(cores)
    refcpu = ref.cpu()
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

    def entry(ms, bytes_, ops_=None, kind=None, sustained=None):
        us = ms * 1e3
        e = {"us": round(us, 2), "GBps": round(bytes_ / ms / 1e6, 1), "frac_hbm": round(bytes_ / ms / 1e6 / hbm, 3)}
        tp = tensor_peaks.get(kind) or {}
        if ops_:
            e["TOPs"] = round(ops_ / ms / 1e9, 1)
            peak = tp.get("TOPs")
            ft, _, ff = roofline_fractions(us, ops_, bytes_, peak, hbm)
            e["frac_tensor"], e["frac_of_floor"], e["tensor_peak_TOPs"] = ft, ff, peak
            if tp.get("TOPs_random_operands"):
                # against what the tensor pipe sustains on toggling operands under the power limit
                e["frac_tensor_powered"] = round(e["TOPs"] / tp["TOPs_random_operands"], 3)
        if sustained and sustained[0] is not None:
            sus_ms, clk = sustained
            e["sustained"] = {"us": round(sus_ms * 1e3, 2), "sm_mhz": clk.get("sm_mhz"), "reasons": clk.get("reasons"),
                              "us_x_mhz": round(sus_ms * 1e3 * clk["sm_mhz"], 0) if clk.get("sm_mhz") else None}
            if clk.get("burst_sm_mhz"):
                # the timed burst in SM cycles, and (GEMMs) the MMA issue cycles of the same work
                # on all SMs as a fraction of them: the structural figure, free of the clock
                cyc = us * clk["burst_sm_mhz"]
                e["burst"] = {"sm_mhz": round(clk["burst_sm_mhz"], 0), "us_x_mhz": round(cyc, 0)}
                if ops_ and tp.get("ops_per_clk_per_sm"):
                    e["burst"]["frac_tensor_cycles"] = round(ops_ / (tp["ops_per_clk_per_sm"] * sm_count) / cyc, 3)
        return e

    def cpu(seconds, kind, what):
        return {"ms": round(seconds * 1e3, 3), "cores": cores, "kind": kind, "what": what}

    def e2e(fn, h2d, d2h, reps=3):
        """fn() does host -> device copies, the call, device -> host copies; timed with a sync on both sides."""
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) / reps * 1e3
        return {"ms": round(ms, 3), "h2d_bytes": int(h2d), "d2h_bytes": int(d2h)}

    pin = lambda t: t.contiguous().pin_memory()

    # ---- config 1: rotary on q,k of [32,1000,3,8,64] ------------------------------------------------
    sin, cos = prep.rotary_tables(1000, 64, device=dev)
    q_host = [torch.randn(32, 1000, 3, 8, 64, generator=g).half() for _ in range(4)]
    qs = [q.to(dev) for q in q_host]
    ms = time_rotating([lambda q=q: ops.rotary_qkv_(q, sin, cos, 32) for q in qs], 20, torch)
    out["rotary_cfg1"] = entry(ms, 131.33e6)
    x32 = q_host[0].float().numpy().copy()
    sin_h, cos_h = sin.cpu().numpy(), cos.cpu().numpy()
    if refcpu is not None:
        def rot_cpu():
            for chunk in (0, 1):
                base = x32.ctypes.data + chunk * 8 * 64 * 4
                refcpu.fluke_rotary_emb_cpu(P(base), sin_h.ctypes.data_as(P), cos_h.ctypes.data_as(P), 32, 1000, 8, 64, 32,
                                            3 * 512 * 1000, 3 * 512, 64, cores)
        out["rotary_cfg1"]["cpu_baseline"] = cpu(_cpu_time(rot_cpu), "reference", "fluke_rotary_emb_cpu fp32, q and k")
    else:
        out["rotary_cfg1"]["cpu_baseline"] = cpu(_cpu_time(lambda: [port.rotary_f32(x32.reshape(-1)[c * 512:], sin_h, cos_h, 32, 1000, 8, 32,
                                                                                     3 * 512 * 1000, 3 * 512, 64) for c in (0, 1)]),
                                                 "port", "oracle rotary fp32, q and k, 1 thread")
    qp, qd = pin(q_host[0]), qs[0]

    def rot_e2e():
        qd.copy_(qp, non_blocking=True)
        ops.rotary_qkv_(qd, sin, cos, 32)
        qp.copy_(qd, non_blocking=True)
    out["rotary_cfg1"]["e2e"] = e2e(rot_e2e, qp.numel() * 2, qp.numel() * 2)
    del qs, q_host

    # ---- config 2: rmsnorm (+quant) [32000,512] -------------------------------------------------------
    n, h = 32000, 512
    w = (1 + 0.1 * torch.randn(h, generator=g)).half().to(dev)
    x_host = [torch.randn(n, h, generator=g).half() for _ in range(6)]
    xs_ = [t.to(dev) for t in x_host]
    rs = [torch.randn(n, h, generator=g).half().to(dev) for _ in range(2)]
    outs = [torch.empty(n, h, dtype=torch.float16, device=dev) for _ in range(2)]
    ms = time_rotating([lambda i=i: ops.rmsnorm(xs_[i], rs[i % 2], w, 2.0, 1e-5, out=outs[i % 2]) for i in range(6)], 20, torch)
    out["rmsnorm_cfg2"] = entry(ms, 98.31e6)
    xf, rf, wf, of = x_host[0].float().numpy(), rs[0].float().cpu().numpy(), w.float().cpu().numpy(), np.empty((n, h), np.float32)
    if refcpu is not None:
        out["rmsnorm_cfg2"]["cpu_baseline"] = cpu(_cpu_time(lambda: refcpu.fluke_rmsnorm_cpu(
            xf.ctypes.data_as(P), rf.ctypes.data_as(P), wf.ctypes.data_as(P), of.ctypes.data_as(P), n, h, F(2.0), F(1e-5), cores)),
            "reference", "fluke_rmsnorm_cpu fp32")
    else:
        out["rmsnorm_cfg2"]["cpu_baseline"] = cpu(_cpu_time(lambda: port.rmsnorm_f32(xf, rf, wf, 2.0, 1e-5)), "port", "oracle rmsnorm fp32")
    xp, rp, op_ = pin(x_host[0]), pin(rs[0].cpu()), pin(torch.empty(n, h, dtype=torch.float16))

    def rms_e2e():
        xs_[0].copy_(xp, non_blocking=True); rs[0].copy_(rp, non_blocking=True)
        ops.rmsnorm(xs_[0], rs[0], w, 2.0, 1e-5, out=outs[0])
        op_.copy_(outs[0], non_blocking=True)
    out["rmsnorm_cfg2"]["e2e"] = e2e(rms_e2e, 2 * n * h * 2, n * h * 2)

    q8 = [torch.zeros(n, h, dtype=torch.int8, device=dev) for _ in range(6)]
    s8 = [torch.ones(n, device=dev) for _ in range(6)]
    ms = time_rotating([lambda i=i: ops.rmsnorm_quant_int8(xs_[i], w, q8[i], s8[i], 0.0, 1e-5) for i in range(6)], 20, torch)
    out["rmsnorm_quant_int8_cfg2"] = entry(ms, 65.79e6)
    x16, w16 = x_host[0].numpy(), w.cpu().numpy()
    zres, ones = np.zeros((n, h), np.int8), np.ones(n, np.float32)
    out["rmsnorm_quant_int8_cfg2"]["cpu_baseline"] = cpu(_cpu_time(lambda: port.rmsnorm_quant(x16, w16, zres, ones, 0.0, 1e-5)),
                                                         "port", "oracle restatement of rmsnorm_quant_int8 (the reference has no CPU twin)")
    q8p, s8p = pin(torch.zeros(n, h, dtype=torch.int8)), pin(torch.ones(n))

    def rmsq_e2e():
        xs_[0].copy_(xp, non_blocking=True); q8[0].copy_(q8p, non_blocking=True); s8[0].copy_(s8p, non_blocking=True)
        ops.rmsnorm_quant_int8(xs_[0], w, q8[0], s8[0], 0.0, 1e-5)
        q8p.copy_(q8[0], non_blocking=True); s8p.copy_(s8[0], non_blocking=True)
    out["rmsnorm_quant_int8_cfg2"]["e2e"] = e2e(rmsq_e2e, n * h * 3 + n * 4, n * h + n * 4)
    u8 = [torch.zeros(n, h, dtype=torch.uint8, device=dev) for _ in range(6)]
    ms = time_rotating([lambda i=i: ops.rmsnorm_quant_fp8(xs_[i], w, u8[i], s8[i], 0.0, 1e-5) for i in range(6)], 20, torch)
    out["rmsnorm_quant_fp8_cfg2"] = entry(ms, 65.79e6)
    out["rmsnorm_quant_fp8_cfg2"]["cpu_baseline"] = cpu(_cpu_time(lambda: port.rmsnorm_quant(x16, w16, zres.view(np.uint8), ones, 0.0, 1e-5, fp8=True)),
                                                        "port", "oracle restatement of rmsnorm_quant_fp8")
    # per-row quantisers on the same [32000,512] f16 input: read 2 B, write 1 B per element + scales
    ms = time_rotating([lambda i=i: ops.quant_int8(xs_[i], out=q8[i], scale=s8[i]) for i in range(6)], 20, torch)
    out["quant_int8_cfg2"] = entry(ms, n * h * 3 + n * 4)
    out["quant_int8_cfg2"]["cpu_baseline"] = cpu(_cpu_time(lambda: port.quant(x16)), "port", "oracle restatement of quant_int8")
    ms = time_rotating([lambda i=i: ops.quant_fp8(xs_[i], out=u8[i], scale=s8[i]) for i in range(6)], 20, torch)
    out["quant_fp8_cfg2"] = entry(ms, n * h * 3 + n * 4)
    out["quant_fp8_cfg2"]["cpu_baseline"] = cpu(_cpu_time(lambda: port.quant(x16, fp8=True)), "port", "oracle restatement of quant_fp8")
    # LSTM -> decoder hand-off: [T,N,C] int8 / e4m3 -> f16 [N,T,C]
    tq = [torch.randint(-127, 128, (1000, 64, 512), generator=g, dtype=torch.int8).to(dev) for _ in range(4)]
    for name, fp8 in (("dequant_int8_transpose", False), ("dequant_fp8_transpose", True)):
        src = [t.view(torch.uint8) if fp8 else t for t in tq]
        ms = time_rotating([lambda s=s: ops.dequant_transpose(s, 0.01, fp8=fp8) for s in src], 10, torch)
        out[name] = entry(ms, 1000 * 64 * 512 * 3)
        hsrc = src[0].cpu().numpy()
        out[name]["cpu_baseline"] = cpu(_cpu_time(lambda: port.dequant_transpose(hsrc, 0.01, fp8=fp8)), "port", "oracle restatement")
    del tq, xs_, rs, outs, u8

    # ---- config 3: QKV GEMM + rotary, M=32000 -----------------------------------------------------------
    be = ops.int8_select(0)
    a_host = [prep.quantize_int8_rows(torch.randn(n, 512, generator=g)) for _ in range(3)]
    a8 = [(a.to(dev), s.to(dev)) for a, s in a_host]
    wq_h, sq_h = prep.quantize_int8_rows(torch.randn(1536, 512, generator=g) * 0.02)
    wq, sq = wq_h.to(dev), sq_h.to(dev)
    o3 = [torch.empty(n, 1536, dtype=torch.float16, device=dev) for _ in range(3)]
    qkv_bytes, qkv_ops = 115.87e6, 2.0 * n * 1536 * 512
    ms, sus, clk = time_rotating([lambda i=i: ops.qkv_rotary_i8(be, a8[i][0], wq, a8[i][1], sq, sin, cos, 1000, out=o3[i]) for i in range(3)],
                                 20, torch, sustain_s=0.6, gpu_index=gpu_index)
    out["qkv_rotary_i8_cfg3"] = entry(ms, qkv_bytes, qkv_ops, "int8", (sus, clk))
    sin_c, cos_c = sin.cpu(), cos.cpu()
    a0, sa0 = a_host[0]

    def qkv_cpu():
        c = (a0.float() * sa0[:, None]) @ (wq_h.float() * sq_h[:, None]).T
        return _rotate_half_torch(c, sin_c, cos_c, 1000)
    out["qkv_rotary_i8_cfg3"]["cpu_baseline"] = cpu(_cpu_time(qkv_cpu), "port", "torch-CPU restatement of the reference test's torch reference (dequantised fp32 GEMM + rotate-half)")
    ap, sap, o3p = pin(a0), pin(sa0), pin(torch.empty(n, 1536, dtype=torch.float16))

    def qkv_e2e():
        a8[0][0].copy_(ap, non_blocking=True); a8[0][1].copy_(sap, non_blocking=True)
        ops.qkv_rotary_i8(be, a8[0][0], wq, a8[0][1], sq, sin, cos, 1000, out=o3[0])
        o3p.copy_(o3[0], non_blocking=True)
    out["qkv_rotary_i8_cfg3"]["e2e"] = e2e(qkv_e2e, n * 512 + n * 4, n * 1536 * 2)
    # the chain of a transformer block: RMSNorm + int8 quantisation, then the QKV GEMM on what it
    # wrote (three rotating buffer sets, 147 MB each): per (norm, GEMM) pair
    xc = [torch.randn(n, h, generator=g).half().to(dev) for _ in range(3)]
    qc = [torch.zeros(n, h, dtype=torch.int8, device=dev) for _ in range(3)]
    sc_ = [torch.ones(n, device=dev) for _ in range(3)]
    chain = []
    for i in range(3):
        chain += [lambda i=i: ops.rmsnorm_quant_int8(xc[i], w, qc[i], sc_[i], 0.0, 1e-5),
                  lambda i=i: ops.qkv_rotary_i8(be, qc[i], wq, sc_[i], sq, sin, cos, 1000, out=o3[i])]
    ms_pair = time_rotating(chain, 10, torch) * 2
    out["rmsnorm_quant_then_qkv_chain"] = {"us": round(ms_pair * 1e3, 2),
                                           "sum_of_the_two_alone_us": round(out["rmsnorm_quant_int8_cfg2"]["us"] + out["qkv_rotary_i8_cfg3"]["us"], 2),
                                           "note": "the GEMM's int8 activations come from L2 (profiles/rmsnorm_quant_qkv_chain_ncu_summary.md)"}
    del xc, qc, sc_

    # ---- config 4: dual GEMM + SiLU ------------------------------------------------------------------------
    wg_h, sg_h = prep.quantize_int8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wu_h, su_h = prep.quantize_int8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wg, sg, wu, su = wg_h.to(dev), sg_h.to(dev), wu_h.to(dev), su_h.to(dev)
    o4 = [torch.empty(n, 2048, dtype=torch.float16, device=dev) for _ in range(3)]
    mlp_bytes, mlp_ops = 149.7e6, 4.0 * n * 2048 * 512
    ms, sus, clk = time_rotating([lambda i=i: ops.gated_mlp_i8(be, a8[i][0], wg, wu, a8[i][1], sg, su, out=o4[i]) for i in range(3)],
                                 20, torch, sustain_s=0.6, gpu_index=gpu_index)
    out["gated_mlp_i8_cfg4"] = entry(ms, mlp_bytes, mlp_ops, "int8", (sus, clk))

    def mlp_cpu():
        ad = a0.float() * sa0[:, None]
        gate = ad @ (wg_h.float() * sg_h[:, None]).T
        up = ad @ (wu_h.float() * su_h[:, None]).T
        return (torch.nn.functional.silu(gate) * up).half()
    out["gated_mlp_i8_cfg4"]["cpu_baseline"] = cpu(_cpu_time(mlp_cpu), "port", "torch-CPU restatement of the reference test's torch reference (two dequantised fp32 GEMMs, silu(g)*u)")
    o4p = pin(torch.empty(n, 2048, dtype=torch.float16))

    def mlp_e2e():
        a8[0][0].copy_(ap, non_blocking=True); a8[0][1].copy_(sap, non_blocking=True)
        ops.gated_mlp_i8(be, a8[0][0], wg, wu, a8[0][1], sg, su, out=o4[0])
        o4p.copy_(o4[0], non_blocking=True)
    out["gated_mlp_i8_cfg4"]["e2e"] = e2e(mlp_e2e, n * 512 + n * 4, n * 2048 * 2)

    # ---- base int8 GEMM at the LSTM's x_down shape: M = 131072 rows of the [T*B, 768] input, N = 128 ---
    mx = 131072
    ax = [torch.randint(-127, 128, (mx, 768), generator=g, dtype=torch.int8).to(dev) for _ in range(2)]
    sax = (torch.rand(mx, generator=g) * 0.02 + 0.001).to(dev)
    wd_h, sd_h = prep.quantize_int8_rows(torch.randn(128, 768, generator=g) / 768 ** 0.5)
    wd, sd = wd_h.to(dev), sd_h.to(dev)
    od = [torch.empty(mx, 128, dtype=torch.float16, device=dev) for _ in range(2)]
    ms = time_rotating([lambda i=i: ops.down_proj_i8(ax[i], wd, sax, sd, out=od[i]) for i in range(2)], 10, torch)
    out["down_proj_i8_x_down"] = entry(ms, mx * 768 + mx * 128 * 2 + mx * 4, 2.0 * mx * 128 * 768, "int8")
    axh, saxh = ax[0][:16384].cpu(), sax[:16384].cpu()
    sec = _cpu_time(lambda: ((axh.float() * saxh[:, None]) @ (wd_h.float() * sd_h[:, None]).T).half())
    out["down_proj_i8_x_down"]["cpu_baseline"] = cpu(sec * (mx / 16384), "port", "torch-CPU dequantised fp32 GEMM on 16384 of the 131072 rows, scaled")
    del ax, od

    # ---- fp8 variants of 3 and 4 (plain [N,K] weights) ---------------------------------------------------
    be8 = ops.fp8_select(0)
    f_host = [prep.quantize_fp8_rows(torch.randn(n, 512, generator=g)) for _ in range(3)]
    f8 = [(a.view(torch.uint8).to(dev), s.to(dev)) for a, s in f_host]
    wq8_h, sq8_h = prep.quantize_fp8_rows(torch.randn(1536, 512, generator=g) * 0.02)
    wq8, sq8 = wq8_h.view(torch.uint8).to(dev), sq8_h.to(dev)
    ms, sus, clk = time_rotating([lambda i=i: ops.qkv_rotary_fp8(be8, f8[i][0], wq8, f8[i][1], sq8, sin, cos, 1000, plain=True, out=o3[i]) for i in range(3)],
                                 20, torch, sustain_s=0.6, gpu_index=gpu_index)
    out["qkv_rotary_fp8_cfg3"] = entry(ms, qkv_bytes, qkv_ops, "e4m3", (sus, clk))
    f0, sf0 = f_host[0]

    def qkv8_cpu():
        c = (f0.float() * sf0[:, None]) @ (wq8_h.float() * sq8_h[:, None]).T
        return _rotate_half_torch(c, sin_c, cos_c, 1000)
    out["qkv_rotary_fp8_cfg3"]["cpu_baseline"] = cpu(_cpu_time(qkv8_cpu), "port", "torch-CPU restatement of fly/test_rotary.py's reference")
    wg8_h, sg8_h = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wu8_h, su8_h = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wg8, sg8, wu8, su8 = wg8_h.view(torch.uint8).to(dev), sg8_h.to(dev), wu8_h.view(torch.uint8).to(dev), su8_h.to(dev)
    ms, sus, clk = time_rotating([lambda i=i: ops.gated_mlp_fp8(be8, f8[i][0], wg8, wu8, f8[i][1], sg8, su8, plain=True, out=o4[i]) for i in range(3)],
                                 20, torch, sustain_s=0.6, gpu_index=gpu_index)
    out["gated_mlp_fp8_cfg4"] = entry(ms, mlp_bytes, mlp_ops, "e4m3", (sus, clk))

    def mlp8_cpu():
        ad = f0.float() * sf0[:, None]
        gate = ad @ (wg8_h.float() * sg8_h[:, None]).T
        up = ad @ (wu8_h.float() * su8_h[:, None]).T
        return (torch.nn.functional.silu(gate) * up).half()
    out["gated_mlp_fp8_cfg4"]["cpu_baseline"] = cpu(_cpu_time(mlp8_cpu), "port", "torch-CPU restatement of fly/test_dual_gemm_silu.py's reference")
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from fluke_b200 import lib as flib, ops, prep
    from fluke_b200.lstm import FactoredLstmLayer, StackPipeline, run_stack
    from fluke_b200.shard import shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the library has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))
    L = flib.load()
    peaks = measured_peaks()

    T, B, H, R, NL = T_STEPS, CHUNKS_PER_GPU, HIDDEN, RANK, LAYERS
    gw = torch.Generator().manual_seed(42)                       # weights: identical on every rank
    layers = [FactoredLstmLayer.random(H, R, bool(i % 2), gw, dev) for i in range(NL)]
    gx = torch.Generator().manual_seed(1000 + rank)              # each rank's own chunks
    x_host = torch.empty(T, B, H, dtype=torch.int8).pin_memory()
    xs_host = torch.empty(T * B, dtype=torch.float32).pin_memory()
    slab = 100                                                   # N(0,1) rows quantised per row (amax/127);
    q, s = prep.quantize_int8_rows(torch.randn(slab * B, H, generator=gx))   # one slab of timesteps, tiled over T
    for t0 in range(0, T, slab):
        x_host[t0:t0 + slab] = q.view(slab, B, H)
        xs_host[t0 * B:(t0 + slab) * B] = s
    x_dev, xs_dev = x_host.to(dev), xs_host.to(dev)
    bufs = [torch.empty(T, B, H, dtype=torch.int8, device=dev) for _ in range(2)]
    ws = torch.empty(L.fluke_factored_lstm_layer_workspace(T, B, H, R), dtype=torch.uint8, device=dev)
    out_host = torch.empty(T, B, H, dtype=torch.int8).pin_memory()

    def fresh_state(b=B):
        return [(torch.zeros(b, H, dtype=torch.float32, device=dev), torch.zeros(b, H, dtype=torch.int8, device=dev))
                for _ in range(NL)]

    def step_resident():
        return run_stack(layers, x_dev, xs_dev, state=fresh_state(), workspace=ws, buffers=bufs)[0]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, after=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if after is not None:
            after()
        e1.record()
        barrier()
        return reduce_step_time(e0.elapsed_time(e1) / steps)

    # two batches side by side: what a launch of the timed region works on
    x2, xs2 = torch.cat([x_dev, x_dev], dim=1), torch.cat([xs_dev.view(T, B)] * 2, dim=1).reshape(-1)
    bufs2 = [torch.empty(T, 2 * B, H, dtype=torch.int8, device=dev) for _ in range(2)]
    ws2 = torch.empty(L.fluke_factored_lstm_layer_workspace(T, 2 * B, H, R), dtype=torch.uint8, device=dev)

    def step_pair():
        return run_stack(layers, x2, xs2, state=fresh_state(2 * B), workspace=ws2, buffers=bufs2)[0]

    def run_steps(k):
        """k independent passes: two per layer launch, an odd last one alone."""
        for _ in range(k // 2):
            step_pair()
        if k % 2:
            step_resident()

    # ---- headline: weak scaling, inputs resident ------------------------------------------------------
    run_steps(max(args.warmup, 3))
    step_resident()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = timed(lambda: run_steps(args.steps), 1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    ms_single = timed(step_resident, min(args.steps, 8))           # every step in a launch of its own

    # ---- strong scaling: 1024 chunks in total, sharded ------------------------------------------------
    if world > 1:
        b0, b1 = shard_range(CHUNKS_PER_GPU, rank, world)
        bs = b1 - b0
        xs_sh = x_dev[:, b0:b1].contiguous()
        ss_sh = xs_dev.view(T, B)[:, b0:b1].contiguous().view(-1)
        bufs_sh = [torch.empty(T, bs, H, dtype=torch.int8, device=dev) for _ in range(2)]

        def step_strong():
            return run_stack(layers, xs_sh, ss_sh, state=fresh_state(bs), workspace=ws, buffers=bufs_sh)[0]
        for _ in range(3):
            step_strong()
        ms_strong = timed(step_strong, args.steps)
        del xs_sh, ss_sh, bufs_sh
    else:
        ms_strong = ms_single

    # ---- end to end: host buffers in the timed region, through the C streaming handle --------------------
    pipe = StackPipeline(layers, T, B, dev, passes_per_launch=2, time_chunks=4)

    def step_e2e():
        return pipe.submit(x_host, xs_host, out_host)

    for _ in range(3):      # a full group and a single pass: both paths of the driver warmed up
        step_e2e()
    pipe.drain()
    ms_e2e = timed(step_e2e, args.steps, after=pipe.drain)   # fill and drain of the pipeline included
    pipe.close()
    del pipe
    # the same copies with no kernels, all ranks at once: what the host link allows
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def copy_only():
        with torch.cuda.stream(s_in):
            x_dev.copy_(x_host, non_blocking=True)
            xs_dev.copy_(xs_host, non_blocking=True)
        with torch.cuda.stream(s_out):
            out_host.copy_(bufs[0], non_blocking=True)

    def copy_done():
        torch.cuda.current_stream().wait_stream(s_in)
        torch.cuda.current_stream().wait_stream(s_out)
    copy_only(); copy_done()
    ms_copy = timed(copy_only, args.steps, after=copy_done)
    torch.cuda.empty_cache()

    # the recurrence kernel of the timed region (the wide configuration: 16 row tiles in one launch):
    # layer minus x_down GEMM, both from CUDA events
    lay0 = layers[0]
    st2 = (torch.zeros(2 * B, H, dtype=torch.float32, device=dev), torch.zeros(2 * B, H, dtype=torch.int8, device=dev))

    def layer2(mask):
        ops.factored_lstm_layer_i8(x2, xs2, lay0.dn_ih, lay0.dn_ih_scale, lay0.dn_hh, lay0.dn_hh_scale, lay0.w_up,
                                   lay0.bias, st2[0], st2[1], h_out=bufs2[0], workspace=ws2, phase_mask=mask)
    us_pair = {}
    for mask in (7, 1):
        layer2(mask)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        layer2(mask); layer2(mask)
        e1.record()
        torch.cuda.synchronize()
        us_pair[mask] = e0.elapsed_time(e1) / 2 * 1e3
        if mask == 7:
            form_pair = L.fluke_sm100_lstm_last_form()
    del x2, xs2, bufs2, ws2, st2
    status = flib.read_status()
    if status != 0:
        raise SystemExit(f"bench.py: device status word {status:#x}: a bounded device wait gave up")

    units = local_units(B, T, NL) * world
    value = units / (ms * 1e-3)
    e2e_value = units / (ms_e2e * 1e-3)

    line = None
    if rank == 0:
        # dominant kernel: the persistent recurrence launch of one layer. Its duration is the
        # layer's time minus the x_down GEMM's (phase mask 1), both from CUDA events on the
        # launching stream.
        lay = layers[0]

        def layer_us(x, xs, b, mask, reps=3):
            st = fresh_state(b)[0]
            hout = bufs[0].view(-1)[:x.numel()].view(x.shape)

            def only():
                ops.factored_lstm_layer_i8(x, xs, lay.dn_ih, lay.dn_ih_scale, lay.dn_hh, lay.dn_hh_scale, lay.w_up,
                                           lay.bias, st[0], st[1], h_out=hout, workspace=ws, phase_mask=mask)
            only()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                only()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps * 1e3   # microseconds
        flops = T * (2.0 * B * (2 * R) * (4 * H) + 2.0 * B * R * H)   # per 1024-chunk layer: f16 gate contraction + int8 hh projection

        def roofline_of(us_layer, us_xdown, form, batches):
            kname = {1: "lstm_cluster_kernel", 2: "lstm_persist_kernel"}.get(form, "lstm_step_kernel")
            us_k = us_layer - us_xdown
            achieved = batches * flops / (us_k * 1e-6) / 1e12
            tr = recurrence_traffic(kname, batches * ((B + 127) // 128))
            return {"kernel": kname, "bound": "tensor", "achieved": round(achieved, 2),
                    "peak": peaks["tf_sustained"], "unit": "TFLOP/s", "frac": round(achieved / peaks["tf_sustained"], 4),
                    "peak_source": f"{peaks['source']} bf16 GEMM, sustained",
                    "chunks_per_launch": batches * B,
                    "traffic": None if tr is None else tr["dram_read_bytes_per_step"] * T + float(T) * batches * B * H,
                    "traffic_source": None if tr is None else
                    f"profiles/lstm_recurrence_traffic.json: {tr['dram_read_bytes_per_step']:.0f} B read per step (ncu, T={tr['T_captured']}) "
                    "x T, plus the h_out the launch writes (larger than L2)",
                    "flops_per_launch": batches * flops,
                    "us_per_launch": {"layer_total": round(us_layer, 3), "x_down_gemm": round(us_xdown, 3), kname: round(us_k, 3)},
                    "cycles_per_step": round(us_k / T * (clocks["sm_mhz"] or 0), 0) if clocks else None}
        roofline = roofline_of(us_pair[7], us_pair[1], form_pair, 2)
        us_layer, us_xdown = layer_us(x_dev, xs_dev, B, 7), layer_us(x_dev, xs_dev, B, 1)
        roofline_single = roofline_of(us_layer, us_xdown, L.fluke_sm100_lstm_last_form(), 1)
        cpu_v, cores, sample = cpu_lstm_sample()
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8+f16",
            "data": "synthetic",
            "config": {"workload": "factored int8 LSTM stack: 5 layers alternating direction, T=1000, H=768, rank=128, "
                                   f"{B} chunks per GPU per step", "l2": "inputs larger than L2 (786 MB per layer input)",
                       "parallelism": f"dp{world} (independent chunks, no collective)",
                       "steps_per_launch": "2: the K independent steps run two at a time, side by side in one [T, 2048, H] "
                                           "layer launch (16 row tiles); one_pass_per_launch is the figure with one step per launch"},
            "timesteps_per_sec_per_gpu_per_layer": T * NL / (ms * 1e-3),
            "one_pass_per_launch": {"value": units / (ms_single * 1e-3), "unit": UNIT, "ms_per_step": ms_single,
                                    "roofline": roofline_single},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": x_host.numel() + xs_host.numel() * 4, "d2h_bytes_per_step": out_host.numel(),
                    "passes_per_launch": 2, "time_chunks": 4, "api": "fluke_flstm_stream_* (C handle)",
                    "copy_only": {"ms_per_step": ms_copy, "value": units / (ms_copy * 1e-3),
                                  "GBps_per_gpu_h2d": (x_host.numel() + xs_host.numel() * 4) / ms_copy / 1e6,
                                  "GBps_per_gpu_d2h": out_host.numel() / ms_copy / 1e6,
                                  "note": "the step's copies alone, both directions at once, all ranks at once, no kernels"},
                    "frac_of_copy_ceiling": ms_copy / ms_e2e},
            "strong": strong_scaling_record(CHUNKS_PER_GPU, world, ms_strong),
            "gpu_launches": (args.steps // 2 + args.steps % 2) * NL * 2,   # per layer call: x_down GEMM + persistent recurrence
            "clocks": clocks, "roofline": roofline,
            "cpu_baseline": {"value": cpu_v, "unit": "chunk-timesteps/s (per layer)", "cores": cores, "kind": "port",
                             "sample": sample, "extrapolated": True,
                             "gate_epilogue_reference": cpu_gate_epilogue_reference()},
        }
        if world == 1 and not args.quick:
            # per-GPU saturation: recurrence time per step of one layer against the batch
            sat, Ts = {}, 250
            for b in (128, 256, 512, 896, 1024, 2048):
                xb = x_dev[:Ts].repeat(1, 2, 1)[:, :b].contiguous() if b > B else x_dev[:Ts, :b].contiguous()
                sb = (xs_dev.view(T, B)[:Ts].repeat(1, 2)[:, :b] if b > B else xs_dev.view(T, B)[:Ts, :b]).contiguous().view(-1)
                us = (layer_us(xb, sb, b, 7) - layer_us(xb, sb, b, 1)) / Ts
                sat[str(b)] = {"us_per_step": round(us, 3), "form": L.fluke_sm100_lstm_last_form(),
                               "chunk_timesteps_per_s": round(b / (us * 1e-6), 0)}
                del xb, sb
            line["saturation"] = {"note": "one layer, T=250, recurrence launch only; form 1 = cluster exchange, 2 = L2 exchange", "by_chunks": sat}
            del x_dev, xs_dev, bufs
            torch.cuda.empty_cache()
            tensor_peaks = measure_tensor_peaks(torch)
            ops_sampler = ClockSampler(local_rank).start()
            line["ops"] = bench_ops(torch, peaks, tensor_peaks, local_rank)
            line["ops_clocks"] = ops_sampler.stop()
            line["tensor_peaks_measured"] = tensor_peaks
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    per_step = max(3.0, min(20.0, 60.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        v, cores, sample = cpu_lstm_sample(per_step)
        if i >= args.warmup:
            vals.append(v)
    value = float(np.mean(vals))
    B, T, NL = CHUNKS_PER_GPU, T_STEPS, LAYERS
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": local_units(B, T, NL) / value * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8+f16", "data": "synthetic",
        "config": {"workload": "factored int8 LSTM stack: 5 layers alternating direction, T=1000, H=768, rank=128, "
                               f"{B} chunks per GPU", "note": "CPU arm: bounded sample per step, rate extrapolated"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                         "extrapolated": True, "gate_epilogue_reference": cpu_gate_epilogue_reference()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--quick", action="store_true", help="skip the saturation curve and the ops section")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
