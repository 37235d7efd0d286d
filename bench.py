"""Benchmark of the Waypoint-1.5 DiT hot path: 720p fp8 generated frames per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one ``gen_frame`` at 720p with linear, kv_cache and attn_compute all fp8: 5 network
evaluations (4 denoise + 1 commit) of the 24-layer DiT on 512 tokens, every layer's KV cache
holding 16 buckets of seeded e4m3 K/V, replayed from one CUDA graph.  Weights and inputs are
synthetic (seeded random init, no checkpoint exists on the box).  ``value`` is latent frames per
second with the noise latent already on the device; ``e2e`` is the same through
``Engine.gen_frame`` with the noise coming from pinned host memory and the latent copied back
every frame.  With N > 1 every rank runs its own independent session on its own GPU (the
reference has no multi-GPU mode; sessions do not communicate), and ``value`` is the sum; the same
ranks then run ONE session sharded by KV-head group, reported as the ``tp`` record of the line.

Beside the headline the line carries: per-kernel times with the same-box cuBLASLt figure for each GEMM shape, the
e4m3 tensor throughput measured in this run (the roofline's denominator), the same frame with scaled e4m3 (``scaled``),
and the CPU oracle of the path timed on the host cores (``cpu_baseline``).

``--impl reference`` times the CPU oracle of the same path on the host cores, on a bounded sample
(one local and one global transformer block per step), scaled to a full frame.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

# The CPU arm runs numpy's BLAS on the host cores.  Launchers such as torch.distributed.run export
# OMP_NUM_THREADS=1 to their workers, which would make the same arm 16 times slower at N = 8 than at N = 1: the
# thread count of that arm is pinned here, before numpy loads its BLAS, to the same number at every N.
CPU_ARM_THREADS = min(16, os.cpu_count() or 1)
if "reference" in sys.argv:
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(CPU_ARM_THREADS)

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_LATENT_FPS_720P_FP8 = 20.0  # RTX 4090, from the table in the reference project's README
HEIGHT, WIDTH = 32, 16  # 720p token grid: 32 rows x 16 columns = 512 tokens per frame
FRAME_T0 = 128  # caches pre-filled as if 128 frames had been appended
NOMINAL_E4M3_TFLOPS = 4500.0  # dense e4m3 tensor throughput of one B200 as published (context beside the measured figure)


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    except Exception:
        return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def measure_e4m3_peak_own(qb, n: int = 8192, sustained_s: float = 2.0):
    """Dense e4m3 tensor throughput of this GPU as this library's own GEMM reaches it: C[n, n] = A[n, n] . B[n, n]^T,
    e4m3 operands, bf16 output, 2 n^3 flops.  `burst`: the best of 10 launches, each timed alone; `sustained`: launches
    back to back for about `sustained_s` seconds (the power cap settles the clocks lower)."""
    r = np.random.default_rng(5)
    blk = r.standard_normal((n, 256), dtype=np.float32)
    a = qb.qf.quantize_e4m3(qb.QuarkTensor.from_numpy(np.tile(blk, (1, n // 256))))
    b = qb.qf.quantize_e4m3(qb.QuarkTensor.from_numpy(np.tile(blk[::-1].copy(), (1, n // 256))))
    c = qb.QuarkTensor.empty(n, n, dtype="bf16")
    call = lambda: qb.qf.gemm(a, b, out_dtype="bf16", compute_dtype="e4m3", out=c)  # noqa: E731
    for _ in range(3):
        call()
    flops = 2.0 * n * n * n
    best = 1e30
    for _ in range(10):
        e0, e1 = qb.runtime.Event(), qb.runtime.Event()
        e0.record()
        call()
        e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_ms(e1))
    reps = max(10, int(sustained_s * 1e3 / best))
    e0, e1 = qb.runtime.Event(), qb.runtime.Event()
    e0.record()
    for _ in range(reps):
        call()
    e1.record()
    e1.synchronize()
    sus = e0.elapsed_ms(e1) / reps
    return {"burst_tflops": round(flops / best / 1e9, 1), "sustained_tflops": round(flops / sus / 1e9, 1), "shape": f"{n}^3 e4m3 -> bf16"}


# --------------------------------------------------------------------------- cuBLASLt on the same box (a mode of its own: it imports torch)


def run_cublaslt_baseline(args):
    """The reference's production GEMM path on CUDA is cublasLtMatmul with e4m3 A and B, f32 accumulation, unit
    scales and a bf16 result (src/quark/runtime/cublas.py:296-459 through kernels/gemm/cublas_dispatch.py:46-68).
    torch reaches the same library call through torch._scaled_mm (e4m3) and torch.matmul (bf16).  Prints one JSON
    line: the four projection shapes at M = 512 (and 128 with --all-m), plain GEMM without epilogue, timed like
    this file's own per-kernel figures (CUDA events around a CUDA graph of 72 launches over 24 weight matrices),
    and the 8192^3 e4m3 and bf16 throughput as a burst (best of 10) and sustained for two seconds."""
    import torch

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    one = torch.ones((), device=dev, dtype=torch.float32)

    def timed(fns, reps=3):
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                for f in fns:
                    f()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * len(fns))

    rows = []
    for M in (512, 128) if args.all_m else (512,):
        for name, N, K in (("gemm_qkv", 4096, 2048), ("gemm_out", 2048, 2048), ("gemm_fc1", 8192, 2048), ("gemm_fc2", 2048, 8192)):
            A = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            Ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(24)]
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            us_bf16 = timed([(lambda W=W: torch.matmul(A, W.t(), out=out)) for W in Ws])
            A8, W8 = A.to(torch.float8_e4m3fn), [W.to(torch.float8_e4m3fn) for W in Ws]
            us_fp8 = timed([(lambda W=W: torch._scaled_mm(A8, W.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)) for W in W8])
            rows.append({"M": M, "kernel": name, "N": N, "K": K, "cublaslt_bf16_us": round(us_bf16, 2), "cublaslt_e4m3_us": round(us_fp8, 2)})
            del Ws, W8
    n = 8192
    flops = 2.0 * n**3
    peak = {}
    for tag, mk in (("e4m3", lambda t: t.to(torch.float8_e4m3fn)), ("bf16", lambda t: t)):
        a, b = mk(torch.randn(n, n, device=dev, dtype=torch.bfloat16)), mk(torch.randn(n, n, device=dev, dtype=torch.bfloat16))
        if tag == "e4m3":
            call = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
        else:
            call = lambda: torch.matmul(a, b.t())  # noqa: E731
        for _ in range(3):
            call()
        best = 1e30
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            call()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(10, int(2000.0 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            call()
        e1.record()
        torch.cuda.synchronize()
        peak[tag] = {"burst_tflops": round(flops / best / 1e9, 1), "sustained_tflops": round(flops / (e0.elapsed_time(e1) / reps) / 1e9, 1)}
    print(json.dumps({"cublaslt_baseline": rows, "peak_8192": peak, "torch": torch.__version__}), flush=True)


def cublaslt_baseline_subprocess(timeout_s: float = 240.0):
    """Runs the mode above in a process of its own (torch stays out of this one); None with a reason on failure."""
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--cublaslt-baseline"], capture_output=True, text=True, timeout=timeout_s)
        for line in reversed(r.stdout.strip().splitlines()):
            if line.startswith("{"):
                return json.loads(line), None
        return None, f"exit {r.returncode}: {(r.stderr or r.stdout)[-300:]}"
    except Exception as e:  # a timeout, a missing torch: the bench line is printed without these figures
        return None, f"{type(e).__name__}: {e}"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, device: int):
        self.device, self.rows, self.proc = device, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )  # fmt: skip
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=mx or None, reasons=sorted(reasons), samples=len(sm))


# --------------------------------------------------------------------------- algorithmic work per launch


def attn_flops(tpf, S, Hq=32, Dh=64):
    return 4.0 * Hq * tpf * S * Dh


def gemm_flops(M, N, K):
    return 2.0 * M * N * K


# --------------------------------------------------------------------------- our arm


def bench_config(n_layers: int = 24, *, tp_rank: int = 0, tp_world: int = 1, fp8_scales: bool = False):
    from quark_b200.models import QuantConfig, Waypoint15Config

    return Waypoint15Config(height=HEIGHT, width=WIDTH, n_layers=n_layers, quant=QuantConfig.all_fp8(), tp_rank=tp_rank, tp_world=tp_world,
                            fp8_scales=fp8_scales)  # fmt: skip


def build_engine(seed: int, device: int, n_layers: int = 24, *, tp_rank: int = 0, tp_world: int = 1, comm=None, params=None, fp8_scales: bool = False):
    import quark_b200 as qb

    cfg = bench_config(n_layers, tp_rank=tp_rank, tp_world=tp_world, fp8_scales=fp8_scales)
    eng = qb.Engine(cfg=cfg, quant=cfg.quant, seed=seed, device=device, comm=comm, params=params)
    # pre-fill every layer's cache with seeded N(0,1) -> e4m3 K/V, as after 128 appended frames.  A tensor-parallel
    # rank holds the rows of its own KV heads of the very caches the single-GPU session holds (both caches are
    # head-major, so a rank's share is one contiguous block), so that the two can be compared.  With cache scales
    # the stored bytes are those of value / scale[head].
    r = np.random.default_rng([seed, 99])
    for blk in eng.model.blocks:
        kc = blk.kv_cache
        for t, sc in ((kc.K_cache, kc.k_scale), (kc.Vt_cache, kc.v_scale)):
            a = r.standard_normal(t.numel * tp_world, dtype=np.float32)[tp_rank * t.numel : (tp_rank + 1) * t.numel]
            if sc is not None:
                a = (a.reshape(cfg.n_kv_heads_local, -1) * (np.float32(1.0) / sc.to_numpy())[:, None]).reshape(-1)
            src = qb.QuarkTensor.from_numpy(a)
            qb.qf.quantize_e4m3(src, out=t)
    eng.set_frame_t(FRAME_T0)
    qb.runtime.synchronize()
    return qb, eng


def scaled_record(args, qb, device, params):
    """The same frame with scaled e4m3 (the wording of the benchmark configuration): every linear weight narrowed with
    one scale per output channel (amax / 448), both caches with one scale per KV head, attention undoing the cache scales.
    The reference has no scales, so this is reported beside the headline, not as it."""
    try:
        _, eng = build_engine(seed=0, device=device, params=params, fp8_scales=True)
        noise = np.random.default_rng([1234, 0]).standard_normal(eng.cfg.latent_numel, dtype=np.float32)
        for _ in range(3):
            eng.gen_frame(noise=noise)
        eng.set_frame_t(FRAME_T0 + 1)
        qb.runtime.synchronize()
        steps = max(5, min(args.steps, 10))
        ms, per = timed_steps(qb, steps, lambda i: eng.gen(eng._noise_dev))
        rec = {"value": round(steps * 1000.0 / ms, 3), "unit": "frames/s", "ms_per_step": round(ms / steps, 4), "ms_per_nfe": round(ms / steps / 5.0, 4),
               "steps": steps, "ms_per_step_spread": spread(per), "launches_per_frame": int(eng.launches_per_frame),
               "quant": "e4m3 with per-output-channel weight scales (amax / 448) and per-KV-head cache scales",
               "device_status": qb._lib.device_status()}  # fmt: skip
        eng.close()
        return rec
    except Exception as e:
        return {"error": f"{type(e).__name__}: {e}"[:300]}


def time_kernels(qb, eng, peaks):
    """Per-launch device time of the hot kernels, each timed alone with CUDA events around a graph of
    launches over the 24 layers' own buffers (24 distinct weight / cache sets, far larger than L2 together).
    Launches of one kernel back to back overlap each other's set-up the way they do inside a frame."""
    blocks = list(eng.model.blocks)
    cfg = eng.cfg
    tpf = cfg.tpf
    ft = eng.gen.frame_t
    res = {}

    def timed(fn, reps=3):
        for b in blocks:  # warm-up pass: every cached buffer exists before the capture
            fn(b)
        # one CUDA graph of reps x 24 launches, so that the host's launch rate cannot bound the figure
        with qb.runtime.capture_graph() as cap:
            for _ in range(reps):
                for b in blocks:
                    fn(b)
        cap.graph.launch()
        e0, e1 = qb.runtime.Event(), qb.runtime.Event()
        e0.record()
        cap.graph.launch()
        e1.record()
        e1.synchronize()
        return e0.elapsed_ms(e1) * 1e3 / (reps * len(blocks))  # us per launch

    xq = qb.QuarkTensor.zeros(tpf, cfg.d_model, dtype="e4m3")
    hq = qb.QuarkTensor.zeros(tpf, cfg.mlp_dim, dtype="e4m3")
    xr = qb.QuarkTensor.zeros(tpf, cfg.d_model, dtype="bf16")
    aq = qb.QuarkTensor.zeros(tpf, cfg.d_model, dtype="e4m3")  # the e4m3 copy of its output that attention emits
    g = eng.model.blocks[0]._cond_lut[0][2]
    qkv = qb.QuarkTensor.zeros(tpf, cfg.qkv_dim, dtype="bf16")
    fp8_peak = peaks["e4m3_tflops"]
    shapes = {
        "gemm_qkv": (lambda b: b.qkv_proj(xq), gemm_flops(tpf, cfg.qkv_dim, cfg.d_model)),
        "gemm_out": (lambda b: b.out_proj(aq, gate=g, residual=xr), gemm_flops(tpf, cfg.d_model, cfg.d_model)),
        "gemm_fc1": (lambda b: b.mlp.fc1(xq, activation="silu", out_dtype="e4m3"), gemm_flops(tpf, cfg.mlp_dim, cfg.d_model)),
        "gemm_fc2": (lambda b: b.mlp.fc2(hq, gate=g, residual=xr), gemm_flops(tpf, cfg.d_model, cfg.mlp_dim)),
        "owl_attn": (lambda b: b.attn(qkv, b.kv_cache, ft), None),
        "kv_cache_update": (lambda b: b.kv_cache(qkv, ft, frozen=True), None),
    }
    # the QKV projection as the frame launches it: head norm, value residual, RoPE(K) and the cache append in its epilogue
    # (frozen: the ring slot is left alone, as in the four denoising passes)
    def qkv_fused(b):
        kc = b.kv_cache
        mix = hasattr(b, "v_residual")
        return qb.qf.gemm_qkv_post(
            xq, b.qkv_proj.weight.data, qkv if mix else None, b.v_residual.lamb.data if mix else None, ft, kc._frozen[1], kc.Vt_cache,
            kc.segments, kc.n_segments, kc.K_cache, n_q_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, H_spatial=cfg.height, W_spatial=cfg.width,
            num_buckets=kc._kw["num_buckets"], pinned_dilation=kc._kw["pinned_dilation"], out=qkv_out, w_scale=b.qkv_proj.w_scale,
            k_scale=kc.k_scale, v_scale=kc.v_scale)  # fmt: skip

    qkv_out = qb.QuarkTensor.zeros(tpf, cfg.qkv_dim, dtype="bf16")
    if cfg.fuse_qkv_gemm and cfg.quilt_factor == 1:
        shapes["gemm_qkv_fused_epilogue"] = (qkv_fused, gemm_flops(tpf, cfg.qkv_dim, cfg.d_model))
    # the norm that follows out-proj and fc2, alone
    s1, b1 = eng.model.blocks[0]._cond_lut[0][3], eng.model.blocks[0]._cond_lut[0][4]
    shapes["ada_rmsnorm"] = (lambda b: b.pre_mlp_norm(xr, s1, b1, emit_e4m3=True), None)
    for name, (fn, flops) in shapes.items():
        us = timed(fn)
        entry = dict(us_per_launch=round(us, 2))
        if name == "owl_attn":
            # keys attended per layer at this frame: local layers 16 buckets, global layers 17 (non-write frame)
            S = np.mean([sum(b.kv_cache.segments.to_numpy()[1::2][: int(b.kv_cache.n_segments.to_numpy()[0])]) for b in blocks])
            flops = attn_flops(tpf, float(S))
            entry["keys_attended_mean"] = float(S)
        if flops is not None:
            entry.update(tflops=round(flops / us / 1e6, 1), frac_of_peak=round(flops / us / 1e6 / fp8_peak, 3))
        elif name == "ada_rmsnorm":
            bytes_ = tpf * cfg.d_model * (2 + 2 + 1)  # x in, bf16 and e4m3 out
            entry.update(gbs=round(bytes_ / us / 1e3, 1), frac_of_peak=round(bytes_ / us / 1e3 / peaks["hbm_gbs"], 3))
        else:
            bytes_ = 2 * tpf * 1024 * 2 + 2 * tpf * 1024 * 1 + 28
            entry.update(gbs=round(bytes_ / us / 1e3, 1), frac_of_peak=round(bytes_ / us / 1e3 / peaks["hbm_gbs"], 3))
        res[name] = entry
    return res


def dram_traffic_from_profiles():
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the hot kernels at this workload's
    shapes, read from the table of the ncu summary that is kept beside this file (its header names the commit
    the capture was taken at).  Returns ({kernel: bytes}, source) or ({}, reason)."""
    path = os.path.join(ROOT, "profiles", "dram_traffic_720p_fp8.md")
    out, commit = {}, None
    try:
        with open(path) as f:
            for line in f:
                if line.lower().startswith("captured at commit"):
                    commit = line.split(":", 1)[1].strip()
                cells = [c.strip() for c in line.strip().strip("|").split("|")]
                if len(cells) >= 2 and cells[0] in ("owl_attn", "gemm_qkv", "gemm_out", "gemm_fc1", "gemm_fc2"):
                    out[cells[0]] = float(cells[1]) * 1e6
    except OSError as e:
        return {}, f"no ncu summary: {e}"
    return out, f"profiles/dram_traffic_720p_fp8.md (ncu capture at commit {commit})"


SFU_EXP_PER_CLK_PER_SM = 16  # ex2.approx.f32: one warp instruction per 8 cycles and scheduler (measured)
N_SMS = 148


def max_over_ranks(values, dist, device="cpu"):
    """Element-wise maximum of a list of floats over all ranks (identity without a process group)."""
    if dist is None:
        return [float(v) for v in values]
    import torch

    t = torch.tensor(list(values), device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.cpu()]


def aggregate_fps(world: int, steps: int, elapsed_ms_max: float) -> float:
    """Whole-job frames per second: every rank generated `steps` frames in the slowest rank's time."""
    return world * steps * 1000.0 / elapsed_ms_max


def timed_steps(qb, steps, step_fn):
    """CUDA events around every step on the launching stream; returns (total ms, list of per-step ms)."""
    ev = [qb.runtime.Event() for _ in range(steps + 1)]
    ev[0].record()
    for i in range(steps):
        step_fn(i)
        ev[i + 1].record()
    ev[-1].synchronize()
    per = [ev[i].elapsed_ms(ev[i + 1]) for i in range(steps)]
    return ev[0].elapsed_ms(ev[-1]), per


def spread(per_step_ms):
    a = np.asarray(per_step_ms, dtype=np.float64)
    return {"min": round(float(a.min()), 4), "median": round(float(np.median(a)), 4), "max": round(float(a.max()), 4)}


def tp_record(args, qb, rank, world, local, dist, ref_latent, noise0):
    """The same frame as ONE session sharded by KV-head group over all ranks (QKV / fc1 column-parallel, out-proj / fc2
    row-parallel, the partial outputs summed over the ranks), measured on the ranks of this run after the independent
    sessions: frames per second (device time, max over ranks), the all-reduce timed alone, and the generated latent
    against rank 0's single-GPU session on the same weights, cache contents and noise."""
    import torch

    from quark_b200.runtime.nccl import NcclComm, Watchdog

    rec = {"parallelism": f"tp{world} by KV-head group: {16 // world} KV heads per GPU, 2 sum all-reduces of [512, 2048] bf16 per block"}
    ok = torch.ones(1, device="cuda")
    comm = eng = None
    try:
        comm = NcclComm(rank, world, f"/tmp/qb_nccl_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}.id", fused=not args.tp_nccl_only)
        _, eng = build_engine(seed=0, device=local, tp_rank=rank, tp_world=world, comm=comm)  # rank 0's session weights on every rank
    except Exception as e:  # a rank that cannot join must not leave the others inside a collective
        ok.zero_()
        rec["error"] = f"{type(e).__name__}: {e}"[:300]
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if float(ok.item()) == 0.0:
        rec.setdefault("error", "another rank failed to build the sharded session")
        return rec
    rec["reduction"] = comm.reduction_name
    wd = Watchdog(comm, timeout_s=60.0)
    with wd.guard():
        out = eng.gen_frame(noise=noise0)  # captures the graph, then the first frame from the pre-filled state
    # a reduction whose wait ran out leaves a bit in the device status word: if any rank saw one, nothing is timed
    bad = torch.tensor([float(qb._lib.device_status())], device="cuda")
    dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    if float(bad.item()) != 0.0:
        rec["error"] = f"device status {int(bad.item())} after the first sharded frame (a bounded wait of the cross-GPU reduction ran out)"
        return rec
    if rank == 0 and ref_latent is not None:
        g = (out.reshape(-1).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        w = (ref_latent.reshape(-1).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        rec["latent_cos_vs_single_gpu"] = round(float(g @ w / (np.linalg.norm(g) * np.linalg.norm(w))), 6)
    with wd.guard():
        for i in range(max(args.warmup, 3)):
            eng.gen_frame(noise=noise0)
    eng.set_frame_t(FRAME_T0 + 1)
    dist.barrier()
    qb.runtime.synchronize()
    with wd.guard():
        dev_ms, per = timed_steps(qb, args.steps, lambda i: eng.gen(eng._noise_dev))
    dist.barrier()
    # the reduction alone: a graph of 48 (one NFE's worth) on the [512, 2048] bf16 partial
    def graph_of_48(fn):
        fn(-1)  # an odd call first: the 48 in the graph then go on alternating
        with qb.runtime.capture_graph() as cap:
            for i in range(48):
                fn(i)
        with wd.guard():
            cap.graph.launch()
            e0, e1 = qb.runtime.Event(), qb.runtime.Event()
            e0.record()
            cap.graph.launch()
            e1.record()
            e1.synchronize()
        us = e0.elapsed_ms(e1) * 1e3 / 48
        del cap
        return us

    y = qb.QuarkTensor.zeros(eng.cfg.tpf, eng.cfg.d_model, dtype="bf16")
    ar_us = graph_of_48(lambda i: comm.all_reduce_sum(y))  # ncclAllReduce alone (without the gate and norm kernels)
    fused_us = 0.0
    if comm.fused:  # sum + gate / residual + AdaRMSNorm (e4m3 out) in the one kernel
        arena = comm.arena(eng.cfg.tpf, eng.cfg.d_model)
        s0, b0, g0 = eng.model.blocks[0]._cond_lut[0][:3]
        sched = comm.tp_schedule  # the pushed schedule sums what is in the staging area (here: whatever the last frame left)
        fused_us = graph_of_48(lambda i: arena.reduce(y, g0, s0, b0, x_slot=i & 1, emit_e4m3=True, schedule=sched))  # alternating slots, as the blocks do
        rec["reduction_schedule"] = {0: "chosen by rank count", 1: "one-shot", 2: "two-shot", 3: "pushed by the GEMM, two-shot"}.get(sched, str(sched))
    dev_ms, ar_us, fused_us = max_over_ranks([dev_ms, ar_us, fused_us], dist, "cuda")
    rec.update(fps=round(args.steps * 1000.0 / dev_ms, 3), ms_per_step=round(dev_ms / args.steps, 4), ms_per_nfe=round(dev_ms / args.steps / 5.0, 4),
               allreduce_us=round(ar_us, 2), launches_per_frame=int(eng.launches_per_frame), device_status=qb._lib.device_status(),
               ms_per_step_spread=spread(per), scaling="strong")  # fmt: skip
    if comm.fused:
        rec["fused_reduction_us"] = round(fused_us, 2)
    eng.close()  # the frame graph holds the communicator's collectives: it goes first
    comm.destroy()
    return rec


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    params = None
    want_scaled = rank == 0 and world == 1 and not args.no_scaled
    if want_scaled:  # one parameter set serves both engines (the scale-free one ignores the cache scales)
        from quark_b200.models import make_params

        params = make_params(bench_config(fp8_scales=True), seed=rank)
    qb, eng = build_engine(seed=rank, device=local, params=params)
    cfg = eng.cfg
    n = cfg.latent_numel
    rng = np.random.default_rng([1234, rank])
    noises = [rng.standard_normal(n, dtype=np.float32) for _ in range(4)]
    noise0 = np.random.default_rng([1234, 0]).standard_normal(n, dtype=np.float32)  # the same on every rank

    def barrier():
        if dist is not None:
            dist.barrier()
        qb.runtime.synchronize()

    # the first frame from the pre-filled state on rank 0's noise: what the sharded session is compared with (N > 1)
    ref_latent = eng.gen_frame(noise=noise0) if world > 1 else None  # captures the graph
    eng.set_frame_t(FRAME_T0)
    # warm-up (the first call also captures the graph), through the public API
    for i in range(max(args.warmup, 3)):
        eng.gen_frame(noise=noises[i % 4])
    launches_per_frame = eng.launches_per_frame
    h2d_d2h = (eng.h2d_bytes_per_frame, eng.d2h_bytes_per_frame)
    eng.set_frame_t(FRAME_T0 + 1)

    # ---- device-resident timing: graph replays, an event after every step
    peaks = measured_peaks()
    with ClockSampler(local) as clocks:
        barrier()
        dev_ms, dev_per = timed_steps(qb, args.steps, lambda i: eng.gen(eng._noise_dev))
        barrier()
        # ---- end to end: host noise -> pinned -> device, replay, latent back to the host, every step
        barrier()
        t0 = time.perf_counter()
        e2e_ev, e2e_per = timed_steps(qb, args.steps, lambda i: eng.gen_frame(noise=noises[i % 4]))
        e2e_ms = max(e2e_ev, (time.perf_counter() - t0) * 1e3)
        barrier()
    dev_ms, e2e_ms = max_over_ranks([dev_ms, e2e_ms], dist, "cuda")
    status = qb._lib.device_status()

    kernels = own_peak = kernel_clocks = None
    if rank == 0:
        eng.set_frame_t(FRAME_T0 + 1)  # every run times the same segment tables (17 buckets on the global layers)
        peaks["e4m3_tflops"] = 2.0 * peaks["bf16_tflops"]  # provisional: the fractions are recomputed below
        with ClockSampler(local) as kc:  # the kernels alone first, before the seconds-long peak measurement heats the GPU
            kernels = time_kernels(qb, eng, peaks)
        kernel_clocks = kc.summary()
        own_peak = measure_e4m3_peak_own(qb)
    cpu = cpu_baseline_sample() if (rank == 0 and world == 1 and not args.no_cpu_baseline) else None
    scaled = scaled_record(args, qb, local, params) if want_scaled else None

    tp = None
    if world > 1 and not args.no_tp:
        eng.close()
        del eng
        import gc

        gc.collect()
        try:
            tp = tp_record(args, qb, rank, world, local, dist, ref_latent, noise0)
        except Exception as e:  # the sessions measurement above stands whatever happens to the sharded one
            tp = {"error": f"{type(e).__name__}: {e}"[:300]}
    base, base_err = cublaslt_baseline_subprocess() if (rank == 0 and not args.no_cublaslt) else (None, "skipped")

    if rank == 0:
        ms_per_step = dev_ms / args.steps
        fps = aggregate_fps(world, args.steps, dev_ms)
        e2e_fps = aggregate_fps(world, args.steps, e2e_ms)
        # the roofline denominator: the best e4m3 8192^3 throughput measured in this run (this library's GEMM or
        # cuBLASLt), a burst figure, because each kernel is timed alone in a short graph
        e4m3_peak = {"own_gemm": own_peak, "nominal_dense_tflops": NOMINAL_E4M3_TFLOPS}
        peak_tflops, peak_src = own_peak["burst_tflops"], "this library's e4m3 GEMM, 8192^3, burst"
        if base is not None:
            e4m3_peak["cublaslt"] = base["peak_8192"]["e4m3"]
            e4m3_peak["cublaslt_bf16"] = base["peak_8192"]["bf16"]
            if base["peak_8192"]["e4m3"]["burst_tflops"] > peak_tflops:
                peak_tflops, peak_src = base["peak_8192"]["e4m3"]["burst_tflops"], "cuBLASLt e4m3 (torch._scaled_mm), 8192^3, burst"
            for row in base["cublaslt_baseline"]:
                if row["M"] == 512 and row["kernel"] in kernels:
                    kernels[row["kernel"]]["cublaslt_us"] = row["cublaslt_e4m3_us"]
        else:
            e4m3_peak["cublaslt_error"] = base_err
        for k in kernels.values():  # fractions against the final denominator
            if "tflops" in k:
                k["frac_of_peak"] = round(k["tflops"] / peak_tflops, 3)
        # every one of these runs once per layer: the dominant kernel is the slowest launch
        dom = max(("owl_attn", "gemm_qkv", "gemm_out", "gemm_fc1", "gemm_fc2"), key=lambda k: kernels[k]["us_per_launch"])
        gemm_us = sum(kernels[k]["us_per_launch"] for k in ("gemm_qkv", "gemm_out", "gemm_fc1", "gemm_fc2"))
        dk = kernels[dom]
        # head_dim 64 leaves 256 tensor flops per exponential: the attention kernel is bound by the
        # special-function unit long before the tensor pipe; report that roofline beside the contract's one
        exps = cfg.tpf * cfg.n_heads * kernels["owl_attn"]["keys_attended_mean"]
        sm_hz = (clocks.summary().get("sm_mhz") or 1965.0) * 1e6
        floor_us = exps / (SFU_EXP_PER_CLK_PER_SM * N_SMS * sm_hz) * 1e6
        sfu = {"exponentials_per_launch": int(exps), "floor_us": round(floor_us, 2),
               "frac": round(floor_us / kernels["owl_attn"]["us_per_launch"], 3)}
        traffic, traffic_src = dram_traffic_from_profiles()
        line = {
            "metric": "latent_fps_720p_fp8",
            "value": round(fps, 3),
            "unit": "frames/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 4),
            "ms_per_nfe": round(ms_per_step / 5.0, 4),
            "ms_per_step_spread": spread(dev_per),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": round(fps / PUBLISHED_LATENT_FPS_720P_FP8, 3),
            "dtype": "e4m3",
            "data": "synthetic",
            "impl": "ours",
            "config": {
                "workload": "gen_frame 720p fp8: 5 NFE x 24 layers, 512 tokens, d_model 2048, GQA 32/16 x 64, 16-bucket e4m3 KV per layer (BASELINE configs[2])",
                "grid": [HEIGHT, WIDTH],
                "frame_t": FRAME_T0 + 1,
                "quant": "linear=fp8 kv_cache=fp8 attn_compute=fp8 (unscaled e4m3, as the reference; the scaled variant is the `scaled` record)",
                "parallelism": "1 session per GPU, no collective (the sharded session is the `tp` record)" if world > 1 else "1 GPU",
                "l2": "inputs larger than L2: each NFE streams ~1.1 GB of e4m3 weights and ~0.4 GB of KV cache",
                "weights": "seeded random init N(0, 0.02)",
            },
            "e2e": {
                "value": round(e2e_fps, 3),
                "unit": "frames/s",
                "h2d_bytes_per_step": h2d_d2h[0],
                "d2h_bytes_per_step": h2d_d2h[1],
                "ms_per_step_spread": spread(e2e_per),
            },
            "gpu_launches": int(launches_per_frame * args.steps),
            "launches_per_frame": int(launches_per_frame),
            "roofline": {
                "kernel": dom,
                "bound": "tensor",
                "achieved": dk["tflops"],
                "peak": round(peak_tflops, 1),
                "unit": "TFLOP/s",
                "frac": round(dk["tflops"] / peak_tflops, 3),
                "traffic": traffic.get(dom),
                "traffic_source": traffic_src,
                "peak_source": f"measured in this run: {peak_src}",
            },
            "e4m3_peak": e4m3_peak,
            "kernels": kernels,
            "kernel_clocks": kernel_clocks,
            "owl_attn_sfu_bound": sfu,
            "gemm_us_per_layer": round(gemm_us, 2),
            "clocks": clocks.summary(),
            "device_status": status,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if scaled is not None:
            line["scaled"] = scaled
        if tp is not None:
            line["tp"] = tp
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- 360p bf16 NFE (BASELINE configs[1])


def run_nfe_360p_bf16(args):
    """The full 24-layer model at 360p (128 tokens, grid 16 x 8), all bf16, caches pre-filled with seeded
    N(0, 1) K / V as after 128 frames: ms per NFE from graph replays of gen_frame (5 NFE).  At M = 128 the
    GEMMs stream their weights (92 MB of bf16 per layer) and are HBM bound."""
    import quark_b200 as qb
    from quark_b200.models import QuantConfig, Waypoint15Config

    cfg = Waypoint15Config(height=16, width=8, quant=QuantConfig.all_bf16())
    eng = qb.Engine(cfg=cfg, quant=cfg.quant, seed=0, device=0)
    r = np.random.default_rng([0, 99])
    for blk in eng.model.blocks:
        for t in (blk.kv_cache.K_cache, blk.kv_cache.Vt_cache):
            t.copy_from(qb.QuarkTensor.from_numpy(r.standard_normal(t.numel, dtype=np.float32).reshape(t.shape), dtype="bf16"))
    eng.set_frame_t(FRAME_T0)
    noise = r.standard_normal(cfg.latent_numel, dtype=np.float32)
    for _ in range(max(args.warmup, 3)):
        eng.gen_frame(noise=noise)
    eng.set_frame_t(FRAME_T0 + 1)
    qb.runtime.synchronize()
    e0, e1 = qb.runtime.Event(), qb.runtime.Event()
    e0.record()
    for _ in range(args.steps):
        eng.gen(eng._noise_dev)
    e1.record()
    e1.synchronize()
    ms = e0.elapsed_ms(e1) / args.steps
    peaks = measured_peaks()
    weight_bytes = 24 * 46_137_344 * 2
    print(json.dumps({"workload": "gen_frame 360p bf16, 24 layers, 128 tokens (BASELINE configs[1])", "ms_per_frame": round(ms, 4),
                      "ms_per_nfe": round(ms / 5, 4), "latent_fps": round(1000.0 / ms, 2),
                      "weight_stream_gbs": round(weight_bytes / (ms / 5) / 1e6, 1), "hbm_frac": round(weight_bytes / (ms / 5) / 1e6 / peaks["hbm_gbs"], 3),
                      "launches_per_frame": eng.launches_per_frame, "device_status": qb._lib.device_status()}), flush=True)  # fmt: skip


# --------------------------------------------------------------------------- isolated attention sweep (BASELINE configs[3])


def run_attn_sweep(args):
    """owl_attn alone at 720p (512 queries, GQA 32/16 x 64) over KV histories of 16 / 64 / 128 / 256 buckets
    of 512 tokens, bf16 and e4m3, on a write frame (3 segments, one bucket masked) and the frame after
    (2 segments); prints one JSON line with a row per point.  K / V are seeded N(0, 1)."""
    import quark_b200 as qb

    qb._lib.require_device(0)
    peaks = measured_peaks()
    H, W, Hk, gqa, pd = HEIGHT, WIDTH, 16, 2, 8
    tpf = H * W
    r = np.random.default_rng(7)
    qkv = qb.QuarkTensor.from_numpy(r.standard_normal((tpf, 4096), dtype=np.float32), dtype="bf16")

    def randn_dev(shape, dt):
        a = r.standard_normal(shape, dtype=np.float32)
        if dt == "bf16":
            return qb.QuarkTensor.from_numpy(a, dtype="bf16")
        return qb.qf.quantize_e4m3(qb.QuarkTensor.from_numpy(a))

    def segment_table(ft, nb):
        """(start, length) pairs of the valid key ranges at frame ft: ring buckets plus the tail slot; on a
        write frame after the ring has wrapped, the bucket about to be overwritten is left out."""
        L = nb * tpf
        bucket = (ft + pd - 1) // pd
        slot = bucket % nb
        if ft % pd == 0 and bucket >= nb:
            return [0, slot * tpf, (slot + 1) * tpf, (nb - slot - 1) * tpf, L, tpf], 3
        return [0, min(bucket, nb) * tpf, L, tpf, 0, 0], 2

    rows = []
    for kv_dt in ("bf16", "e4m3"):
        es = 2 if kv_dt == "bf16" else 1
        for nb in (16, 64, 128, 256):
            cap = (nb + 1) * tpf
            Kc, Vc = randn_dev((Hk * cap, 64), kv_dt), randn_dev((Hk * 64, cap), kv_dt)
            out = qb.QuarkTensor.empty(tpf, 2048, dtype="bf16")
            for ft in (nb * pd, nb * pd + 1):
                segs, n = segment_table(ft, nb)
                S = int(sum(segs[1::2][:n]))
                sg = qb.QuarkTensor.from_numpy(np.asarray(segs, np.int32))
                ns = qb.QuarkTensor.from_numpy(np.array([n], np.int32))
                ftt = qb.QuarkTensor.from_numpy(np.array([ft], np.int32))
                call = lambda: qb.qf.owl_attn(qkv, Kc, Vc, sg, ns, 1, Hk, gqa, H, W, nb, pd, compute_dtype="e4m3" if kv_dt == "e4m3" else None,
                                              packed_qkv=True, frame_t=ftt, out=out)  # noqa: E731
                call()
                reps = max(3, min(20, int(2e5 / max(S, 1))))
                with qb.runtime.capture_graph() as cap_:
                    for _ in range(reps):
                        call()
                cap_.graph.launch()
                e0, e1 = qb.runtime.Event(), qb.runtime.Event()
                e0.record()
                cap_.graph.launch()
                e1.record()
                e1.synchronize()
                us = e0.elapsed_ms(e1) * 1e3 / reps
                del cap_  # the graph must be gone before the next capture begins (destroying it is not capturable)
                flops = attn_flops(tpf, float(S))
                byts = 2 * Hk * S * 64 * es + 2 * tpf * 32 * 64 * 2
                tensor_peak = peaks["bf16_tflops"] * (2.0 if kv_dt == "e4m3" else 1.0)
                rows.append({"kv": kv_dt, "buckets": nb, "frame_t": ft, "segments": int(n), "keys": S, "us": round(us, 1),
                             "tflops": round(flops / us / 1e6, 1), "tensor_frac": round(flops / us / 1e6 / tensor_peak, 3),
                             "gbs": round(byts / us / 1e3, 1), "hbm_frac": round(byts / us / 1e3 / peaks["hbm_gbs"], 3),
                             "sfu_frac": round(tpf * 32 * S / (SFU_EXP_PER_CLK_PER_SM * N_SMS * 1.965e9) * 1e6 / us, 3)})  # fmt: skip
            del Kc, Vc
    print(json.dumps({"attn_sweep_720p": rows, "device_status": qb._lib.device_status(), "peaks": peaks}), flush=True)


# --------------------------------------------------------------------------- one session sharded over the GPUs


def run_tp(args):
    """One 720p fp8 session sharded by KV-head group over all ranks (strong scaling): QKV / fc1 column-parallel,
    out-proj / fc2 row-parallel, an NCCL sum all-reduce of the [512, 2048] bf16 partial after each of the two.
    Every rank sees only its own GPU; no torch in the process."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    import quark_b200 as qb
    from quark_b200.runtime.nccl import LocalComm, NcclComm

    # every GPU of the job stays visible to every rank: the fused reduction maps the peers' buffers (CUDA IPC)
    qb._lib.require_device(local)
    qb._lib.check(qb._lib.load().qb_set_device(local))
    id_path = f"/tmp/qb_nccl_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}.id"
    comm = NcclComm(rank, world, id_path, fused=not args.tp_nccl_only) if world > 1 else LocalComm()
    _, eng = build_engine(seed=0, device=local, tp_rank=rank, tp_world=world, comm=comm)  # same weights and noise on every rank
    n = eng.cfg.latent_numel
    noises = [np.random.default_rng([1234, i]).standard_normal(n, dtype=np.float32) for i in range(4)]
    for i in range(max(args.warmup, 3)):
        eng.gen_frame(noise=noises[i % 4])
    eng.set_frame_t(FRAME_T0 + 1)
    flag = qb.QuarkTensor.zeros(1, dtype="f32")

    def barrier():
        comm.all_reduce_max(flag)
        qb.runtime.synchronize()

    with ClockSampler(local) as clocks:
        barrier()
        e0, e1 = qb.runtime.Event(), qb.runtime.Event()
        e0.record()
        for _ in range(args.steps):
            eng.gen(eng._noise_dev)
        e1.record()
        e1.synchronize()
        barrier()
        dev_ms = e0.elapsed_ms(e1)
        t0 = time.perf_counter()
        e2, e3 = qb.runtime.Event(), qb.runtime.Event()
        e2.record()
        for i in range(args.steps):
            eng.gen_frame(noise=noises[i % 4])
        e3.record()
        e3.synchronize()
        e2e_ms = max(e2.elapsed_ms(e3), (time.perf_counter() - t0) * 1e3)
        barrier()
    times = qb.QuarkTensor.from_numpy(np.array([dev_ms, e2e_ms], dtype=np.float32))
    comm.all_reduce_max(times)
    qb.runtime.synchronize()
    dev_ms, e2e_ms = (float(v) for v in times.to_numpy())
    status = qb._lib.device_status()
    launches_per_frame, h2d, d2h = eng.launches_per_frame, eng.h2d_bytes_per_frame, eng.d2h_bytes_per_frame
    eng.close()  # the frame graph holds the communicator's collectives: it goes first
    comm.destroy()
    if rank == 0:
        ms_per_step = dev_ms / args.steps
        fps = args.steps * 1000.0 / dev_ms
        print(json.dumps({
            "metric": "latent_fps_720p_fp8", "value": round(fps, 3), "unit": "frames/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "ms_per_nfe": round(ms_per_step / 5.0, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": round(fps / PUBLISHED_LATENT_FPS_720P_FP8, 3),
            "dtype": "e4m3", "data": "synthetic", "impl": "ours",
            "config": {"workload": "gen_frame 720p fp8, ONE session sharded over the GPUs (BASELINE configs[4])",
                       "parallelism": f"tp{world} by KV-head group: {16 // world} KV heads per GPU, QKV / fc1 column-parallel, out-proj / fc2 "
                                      f"row-parallel, 2 sums of [512, 2048] bf16 per block (48 per NFE) inside the CUDA graph: {comm.reduction_name}",
                       "frame_t": FRAME_T0 + 1, "l2": "inputs larger than L2"},
            "e2e": {"value": round(args.steps * 1000.0 / e2e_ms, 3), "unit": "frames/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches_per_frame * args.steps), "launches_per_frame": int(launches_per_frame),
            "clocks": clocks.summary(), "device_status": status,
        }), flush=True)  # fmt: skip


# --------------------------------------------------------------------------- CPU oracle arm


def blas_threads() -> int:
    try:
        from threadpoolctl import threadpool_info

        return max([int(i.get("num_threads", 1)) for i in threadpool_info()] or [1])
    except Exception:
        return int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))


class pinned_blas_threads:
    """The CPU arm's BLAS thread count, the same whatever the launcher exported (see CPU_ARM_THREADS)."""

    def __enter__(self):
        self._ctx = None
        try:
            from threadpoolctl import threadpool_limits

            self._ctx = threadpool_limits(limits=CPU_ARM_THREADS)
            self._ctx.__enter__()
        except Exception:
            self._ctx = None
        return self

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)
        return False


def oracle_block_seconds(seed=0, layer=0):
    """One 720p fp8 block through the chained CPU oracle (the bounded sample): `layer` 0 is a local block (16
    buckets of one frame each attended), layer 3 a global one (16 buckets of every 8th frame plus the tail: 17 buckets
    on the non-write frame timed here)."""
    from oracle import codec
    from oracle import model as om
    from quark_b200.models import QuantConfig, Waypoint15Config, make_params

    cfg = Waypoint15Config(n_layers=layer + 1, height=HEIGHT, width=WIDTH, quant=QuantConfig.all_fp8())
    params = make_params(cfg, seed)
    blk = params["blocks"][layer]
    for k in ("qkv.weight", "out.weight", "fc1.weight", "fc2.weight"):
        blk[k] = codec.f32_to_e4m3(codec.bf16_to_f32(blk[k]))
    q = om.Quant(linear="fp8", kv_cache="fp8", attn_compute="fp8")
    st = om.new_state(cfg, q)[layer]
    r = np.random.default_rng(seed)
    for name in ("K_cache", "Vt_cache"):
        st[name][...] = codec.f32_to_e4m3(r.standard_normal(st[name].shape).astype(np.float32))
    x = codec.f32_to_bf16(r.standard_normal((cfg.tpf, cfg.d_model)).astype(np.float32))
    with pinned_blas_threads():
        t0 = time.perf_counter()
        om.block_forward(cfg, layer, blk, st, x, 0, FRAME_T0 + 1, qkv_first=None, frozen=True, quant=q)
        return time.perf_counter() - t0


CPU_ARM_NOTE = ("numpy restatement of the reference's per-kernel oracles, chained as the model chains its kernels; it skips masked "
                "buckets and vectorises the e4m3 codec, which makes it several times faster than the reference's own 720p oracle (measured "
                "on the same 8 host cores: 28.3 s per bf16 block for the reference's, 3.7 s per fp8 block for this one); patchify, out-norm, "
                "unpatchify and the Euler steps are left out (under 1 % of the frame)")


def cpu_frame_seconds(local_s: float, global_s: float) -> float:
    """A frame = 5 NFE x (18 local + 6 global blocks)."""
    return 5.0 * (18.0 * local_s + 6.0 * global_s)


def cpu_baseline_sample(reps=2):
    with pinned_blas_threads():
        threads = blas_threads()
    loc = min(oracle_block_seconds(i, 0) for i in range(reps))
    glo = min(oracle_block_seconds(i, 3) for i in range(reps))
    frame_s = cpu_frame_seconds(loc, glo)
    return {
        "value": round(1.0 / frame_s, 5),
        "unit": "frames/s",
        "cores": threads,
        "kind": "port",
        "sample": f"one local ({loc:.2f} s) and one global ({glo:.2f} s) 720p fp8 transformer block through the chained numpy oracle, best of {reps}; "
                  f"frame = 5 NFE x (18 local + 6 global); {CPU_ARM_NOTE}",
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    for _ in range(min(args.warmup, 1)):
        oracle_block_seconds(0, 0)
    steps = max(1, min(args.steps, 4))
    loc = [oracle_block_seconds(i, 0) for i in range(steps)]
    glo = [oracle_block_seconds(i, 3) for i in range(steps)]
    frame_s = cpu_frame_seconds(float(np.mean(loc)), float(np.mean(glo)))
    fps = 1.0 / frame_s
    with pinned_blas_threads():
        threads = blas_threads()
    cpu = {
        "value": round(fps, 5),
        "unit": "frames/s",
        "cores": threads,
        "kind": "port",
        "sample": f"per step one local ({np.mean(loc):.2f} s) and one global ({np.mean(glo):.2f} s) 720p fp8 transformer block through the chained "
                  f"numpy oracle, mean of {steps}; frame = 5 NFE x (18 local + 6 global); {CPU_ARM_NOTE}",
    }
    print(json.dumps({
        "metric": "latent_fps_720p_fp8", "value": round(fps, 5), "unit": "frames/s", "n_gpus": world, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": round(frame_s * 1e3, 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(fps / PUBLISHED_LATENT_FPS_720P_FP8, 6), "dtype": "e4m3", "data": "synthetic", "impl": "reference",
        "config": {"workload": "gen_frame 720p fp8 (BASELINE configs[2]) on the host cores through the CPU oracle of the path",
                   "blas_threads": threads,
                   "note": "the reference's GPU path needs its Python tree, which is not present on the GPU box; its own CPU implementation of this path is the numpy oracle restated in oracle/"},
        "cpu_baseline": cpu,
        "e2e": {"value": round(fps, 5), "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)  # fmt: skip


def run_profile_nfe(args):
    """For profilers: build the engine, run eager (ungraphed) NFEs of the bench workload and exit.

    Prints how many kernels were launched before the last NFE and how many it has, so that a
    profiler can skip straight to it (`ncu -s <before> -c <per_nfe>`).
    """
    qb, eng = build_engine(seed=0, device=0, n_layers=args.layers)
    eng.set_frame_t(FRAME_T0 + 1)
    noise = qb.QuarkTensor.from_numpy(np.random.default_rng(0).standard_normal((1, eng.cfg.latent_numel), dtype=np.float32), dtype="bf16")
    for _ in range(2):  # the first pass allocates every cached buffer
        eng.model(noise, sigma_idx=0, frame_t=eng.gen.frame_t, frozen=True)
    qb.runtime.synchronize()
    before = qb._lib.kernel_launch_count()
    eng.model(noise, sigma_idx=0, frame_t=eng.gen.frame_t, frozen=True)
    qb.runtime.synchronize()
    per_nfe = qb._lib.kernel_launch_count() - before
    print(json.dumps({"launches_before": before, "launches_per_nfe": per_nfe, "device_status": qb._lib.device_status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile-nfe", action="store_true", help="run eager NFEs of the workload and exit (for ncu)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--attn-sweep", action="store_true", help="time owl_attn alone over KV histories of 16 .. 256 buckets and exit")
    ap.add_argument("--nfe-360p-bf16", action="store_true", help="time the 24-layer model at 360p in bf16 and exit")
    ap.add_argument("--mode", default="sessions", choices=["sessions", "tp"],
                    help="N > 1: 'sessions' = one independent session per GPU (weak scaling, the default); "
                         "'tp' = one session sharded by KV-head group with NCCL all-reduces (strong scaling)")
    ap.add_argument("--layers", type=int, default=24, help="model depth for --profile-nfe (smaller = less device memory under a profiler)")
    ap.add_argument("--cublaslt-baseline", action="store_true", help="time cuBLASLt (through torch) on the four projection shapes and at 8192^3, and exit")
    ap.add_argument("--all-m", action="store_true", help="--cublaslt-baseline: also M = 128")
    ap.add_argument("--no-cublaslt", action="store_true", help="leave the cuBLASLt figures out of the main line")
    ap.add_argument("--no-scaled", action="store_true", help="leave the scaled-e4m3 frame out of the main line")
    ap.add_argument("--no-tp", action="store_true", help="N > 1: leave the sharded session out of the main line")
    ap.add_argument("--tp-nccl-only", action="store_true", help="the sharded session sums with ncclAllReduce + a gate kernel instead of the fused reduction")
    args = ap.parse_args()
    if args.cublaslt_baseline:
        run_cublaslt_baseline(args)
    elif args.profile_nfe:
        run_profile_nfe(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.attn_sweep:
        run_attn_sweep(args)
    elif args.nfe_360p_bf16:
        run_nfe_360p_bf16(args)
    elif args.mode == "tp":
        run_tp(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
