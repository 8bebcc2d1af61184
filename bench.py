#!/usr/bin/env python
"""Headline benchmark: greedy decode of the seeded random-init 27B-shape W6 model at batch 1 (the 27B benchmark configuration):
prefill of 2048 seeded tokens in 512-token chunks, then decode steps.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 27b|4b|tiny]

One "step" is one decoded token.  `value` is decode tok/s with the step replayed as a CUDA graph and the token fed back
on the device (inputs resident in HBM); `e2e` is the same loop driven like the reference drives its backend
(crates/det/src/model.rs:439-547): host embedding row -> H2D, forward, argmax, 4-byte D2H per token.  The roofline object
covers the decode GEMV (k_gemv_stream) timed alone with CUDA events on the library's queue; `cpu_baseline` is the CPU
reference port timed on a bounded slice of the same model.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SEED = 20261125
PROMPT_SEED = 1


def _peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class Events:
    """CUDA events on the library's own queue (torch.cuda.Event would only see torch's stream)."""

    def __init__(self, stream):
        self.rt = C.CDLL("libcudart.so.12")
        self.stream = C.c_void_p(stream)

    def record(self):
        e = C.c_void_p()
        assert self.rt.cudaEventCreate(C.byref(e)) == 0
        assert self.rt.cudaEventRecord(e, self.stream) == 0
        return e

    def ms(self, a, b) -> float:
        assert self.rt.cudaEventSynchronize(b) == 0
        out = C.c_float()
        assert self.rt.cudaEventElapsedTime(C.byref(out), a, b) == 0
        return out.value


class ClockSampler:
    """Samples the SM clock, power and throttle reasons through NVML from a thread of this process while the timed
    regions run (read-only queries; a polling nvidia-smi process disturbs a latency-bound decode loop measurably)."""

    def __init__(self, index: int, period_s: float = 0.2):
        self.rows, self.index, self.period, self._stop, self.thread = [], index, period_s, threading.Event(), None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        except Exception:
            self.nv = None
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                sm = nv.nvmlDeviceGetClockInfo(self.dev, nv.NVML_CLOCK_SM)
                mx = nv.nvmlDeviceGetMaxClockInfo(self.dev, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev)
                self.rows.append((time.time(), sm, mx, reasons))
            except Exception:
                pass
            self._stop.wait(self.period)

    def stop(self):
        self._stop.set()
        if self.thread:
            self.thread.join(timeout=2)

    def summary(self, windows) -> dict:
        if not getattr(self, "nv", None):
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "note": "NVML unavailable"}
        nv = self.nv
        flags = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        sm, mx, reasons = [], 0, set()
        for ts, s_, m_, r in self.rows:
            if not any(a <= ts <= b for a, b in windows):
                continue
            sm.append(s_)
            mx = max(mx, m_)
            for name, bit in flags.items():
                if r & bit:
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------------
SHAPES = {   # layers, hidden, ffn, attention (q heads, kv heads, head dim), GDN (k heads, v heads), vocab
    "tiny": dict(layers=8, hidden=1024, ffn=3072, n_h=8, n_kv=2, hd=256, n_k=8, n_v=16, vocab=32768),
    "4b": dict(layers=32, hidden=2560, ffn=9216, n_h=16, n_kv=4, hd=256, n_k=16, n_v=32, vocab=248320),
    "27b": dict(layers=64, hidden=5120, ffn=17408, n_h=24, n_kv=4, hd=256, n_k=16, n_v=48, vocab=248320),
}


def launches_per_token(cfg: str, fused: bool = True) -> int:
    """Kernels of one device-resident decode step.  Fused (default): a Gated DeltaNet layer is 5 launches (qkv|z + a|b
    GEMV with the RMSNorm prologue, the mixer step, output GEMV with the quantization prologue, gate|up GEMV with the
    RMSNorm prologue and the SwiGLU epilogue, down GEMV with the quantization prologue), an attention layer 6 (q|k|v GEMV,
    prep, attention, output GEMV, gate|up, down), plus embed, head GEMV, argmax and token feedback.  Unfused: every op on
    its own (11 / 10 per layer, plus the final norm)."""
    layers = SHAPES[cfg]["layers"]
    n_attn = layers // 4
    if fused:
        return (layers - n_attn) * 5 + n_attn * 6 + 4
    return (layers - n_attn) * 11 + n_attn * 10 + 5


def _prompt(h, n, vocab):
    import numpy as np
    ids = np.zeros(n, np.int32)
    h.dh_synth_prompt(PROMPT_SEED, n, vocab, ids.ctypes.data)
    return ids


def _check(rc, h):
    if rc != 0:
        raise RuntimeError(h.dh_last_error().decode())


def _mem_available_gb() -> float:
    try:
        for line in open("/proc/meminfo"):
            if line.startswith("MemAvailable:"):
                return int(line.split()[1]) / 1e6
    except OSError:
        pass
    return 0.0


def _weights_gb(cfg: str) -> float:
    """Packed linear weights of a configuration (W6 body, W8 head and GDN a|b) as the CPU port keeps them."""
    s = SHAPES[cfg]
    h, f, hd, nh, nkv, nk, nv = s["hidden"], s["ffn"], s["hd"], s["n_h"], s["n_kv"], s["n_k"], s["n_v"]
    row = lambda k, bits: k * bits // 8 + 4 + k // 128 * 2
    attn = (nh * 2 * hd + 2 * nkv * hd) * row(h, 6) + h * row(nh * hd, 6)
    gdn = (2 * nk * 128 + 2 * nv * 128) * row(h, 6) + 2 * nv * row(h, 8) + h * row(nv * 128, 6)
    ffn = 2 * f * row(h, 6) + h * row(f, 6)
    n_attn = s["layers"] // 4
    return (n_attn * attn + (s["layers"] - n_attn) * gdn + s["layers"] * ffn + s["vocab"] * row(h, 8)) / 1e9


def cpu_baseline(h, cfg: str, threads: int, tokens: int = 8, warmup: int = 1, context: int = 2048, chunk: int = 256):
    """The CPU port of the reference's x86 backend (oracle/x86_backend.hpp: strip-repacked packed weights, K-blocked
    vpdpbusd / vpmaddubsw GEMM, SIMD glue, attention and Gated DeltaNet, OpenMP where the reference uses rayon) on the
    same model at full depth: prefill `context` tokens of the benchmark prompt in `chunk`-token batches (the reference's
    `det bench` default, crates/det-cli/src/main.rs:297), then `warmup` untimed and `tokens` timed greedy decode steps
    (forward + argmax, wall clock).  When the host has too little memory for the full model the first 4 and 8 layers
    are timed instead and the line says "extrapolated"."""
    import importlib.util
    import numpy as np
    spec = importlib.util.spec_from_file_location("oracle_build", ROOT / "oracle" / "build.py")
    ob = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ob)
    os.environ["OMP_NUM_THREADS"] = str(threads)   # a launcher (torchrun) exports 1; the baseline uses every host core
    o = C.CDLL(str(ob.build()))
    o.orc_set_threads(threads)                     # also when the OpenMP runtime was loaded before the variable changed
    threads = o.orc_max_threads()
    o.orc_cpu_backend_new.restype = C.c_void_p
    o.orc_cpu_backend_new.argtypes = [C.c_int]
    o.orc_ref_backend_free.argtypes = [C.c_void_p]
    level = o.orc_cpu_simd_level()
    if level == 0:
        raise RuntimeError("the CPU port needs AVX2")
    rb = o.orc_cpu_backend_new(-1)
    simd = {2: "AVX-VNNI vpdpbusd", 1: "AVX2 vpmaddubsw"}[level]
    vocab = SHAPES[cfg]["vocab"]
    need_gb, have_gb = _weights_gb(cfg) * 2.2 + 4, _mem_available_gb()   # det rows of one linear + strips + working set
    ids = _prompt(h, max(context, 8), vocab)

    def run(layers: int, ctx: int):
        m = h.dh_model_new_synth(rb, cfg.encode(), layers, SEED, ctx + tokens + warmup + 8, chunk)
        if not m:
            raise RuntimeError(h.dh_last_error().decode())
        t0 = time.perf_counter()
        _check(h.dh_model_prefill(m, ids.ctypes.data, ctx), h)
        t_prefill = time.perf_counter() - t0
        tok, rng = C.c_int32(0), C.c_uint64(0)
        _check(h.dh_model_pick(m, 1, 1.0, 0, 1.0, C.byref(rng), C.byref(tok)), h)
        toks = [tok.value]
        t_dec = 0.0
        for i in range(warmup + tokens):
            t0 = time.perf_counter()
            one = np.array([tok.value], np.int32)
            _check(h.dh_model_forward(m, one.ctypes.data, 1), h)
            _check(h.dh_model_pick(m, 1, 1.0, 0, 1.0, C.byref(rng), C.byref(tok)), h)
            if i >= warmup:
                t_dec += time.perf_counter() - t0
            toks.append(tok.value)
        h.dh_model_free(m)
        return t_dec / tokens, t_prefill, toks

    full = SHAPES[cfg]["layers"]
    base = {"unit": "tok/s", "cores": threads, "kind": "port", "ram_gb": round(have_gb, 1)}
    if have_gb >= need_gb:
        per_token, t_prefill, toks = run(0, context)
        base.update({"value": 1.0 / per_token, "extrapolated": False, "steps_timed": tokens, "ms_per_step": per_token * 1e3,
                     "context": context, "prefill": {"value": context / t_prefill, "unit": "tok/s", "tokens": context, "chunk": chunk},
                     "tokens": toks,
                     "sample": f"{cfg} shape at full depth ({full} layers + W8 head): prefill {context} tokens of the benchmark "
                               f"prompt in {chunk}-token chunks, {warmup} untimed + {tokens} timed greedy decode tokens; restated "
                               f"x86 backend of the reference ({simd}, packed strip weights), {threads} OpenMP threads"})
    else:
        times = {}
        for layers in (4, 8):
            times[layers], _, _ = run(layers, 8)
        per_token = times[4] + (times[8] - times[4]) * (full // 4 - 1)
        base.update({"value": 1.0 / per_token, "extrapolated": True, "steps_timed": tokens, "ms_per_step": per_token * 1e3,
                     "context": 8,
                     "sample": f"{cfg} shape, first 4 and 8 layers + W8 head ({have_gb:.0f} GB of host memory available, "
                               f"{need_gb:.0f} GB needed for the full depth), {tokens} decode tokens each at position 8, "
                               f"extrapolated linearly to {full} layers; restated x86 backend of the reference ({simd}), "
                               f"{threads} OpenMP threads"})
    o.orc_ref_backend_free(rb)
    return base


# dram bytes / algorithmic bytes of the decode GEMV in the committed profiler capture (68.62 - 68.94 MB for 68.38 MB)
GEMV_TRAFFIC_RATIO = 1.006


def _tensor_parallel(args, h, rank: int, world: int, shape: dict, rows: int):
    """N > 1: tensor parallel over NVLink.  torch.distributed (gloo, CPU) only carries the NCCL id, the IPC handles, the
    barriers and the max-over-ranks of the timings; the data path uses the library's own exchange on its queue.  `rows` is
    the largest batch whose exchanges should fit the peer staging.  Returns (dist, comm handle, saved stdout fd)."""
    import numpy as np
    if world == 1:
        return None, None, None
    # libraries loaded for the exchange (NCCL) may print banners on stdout; the contract is ONE JSON line there
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo")
    nid = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = np.zeros(128, np.uint8)
        h.dh_nccl_unique_id(buf.ctypes.data)
        nid = torch.from_numpy(buf)
    dist.broadcast(nid, 0)
    nid_np = nid.numpy().copy()
    if args.exchange == "nccl":
        comm = h.dh_nccl_comm_new(nid_np.ctypes.data, rank, world)
        if not comm:
            raise RuntimeError(h.dh_last_error().decode())
        return dist, comm, saved_stdout
    # decode-sized exchanges: one kernel per rank storing packets into every peer's staging (CUDA IPC mapped);
    # prefill chunks (megabytes) stay on NCCL.  16 staging bytes per gathered value of the largest exchange.
    mixw = shape["n_h"] * shape["hd"]
    staging = 16 * max(rows * max(mixw, shape["ffn"], shape["hidden"]), shape["vocab"]) + 4096
    comm = h.dh_peer_comm_new(nid_np.ctypes.data, rank, world, staging)
    if not comm:
        raise RuntimeError(h.dh_last_error().decode())
    mine = np.zeros(64, np.uint8)
    h.dh_peer_comm_handle(comm, mine.ctypes.data)
    every = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(every, torch.from_numpy(mine))
    handles = np.concatenate([e.numpy() for e in every]).copy()
    h.dh_peer_comm_open(comm, handles.ctypes.data)
    if args.exchange == "peer-unfused":
        h.dh_peer_comm_set_fuse(comm, 0)
    elif args.exchange == "peer-rows":
        h.dh_peer_comm_set_fuse(comm, 1)     # exchanges fused with their row kernels, not with the GEMVs
    dist.barrier()
    return dist, comm, saved_stdout


def run_ours(args, rank: int, world: int, local_rank: int):
    import numpy as np
    from det_b200 import capi
    rt = C.CDLL("libcudart.so.12")
    assert rt.cudaSetDevice(local_rank) == 0
    h, d = capi.host(), capi.cuda()
    if args.no_pdl:
        d.det_debug_set_pdl(0)
    cfg = args.config
    shape = SHAPES[cfg]
    K, W, P, chunk = args.steps, args.warmup, args.prefill, args.chunk
    max_ctx = P + 2 * (K + W) + 16
    bk = h.dh_cuda_backend_new(1, 1)
    if not bk:
        raise RuntimeError(h.dh_last_error().decode())
    if args.no_fuse:
        h.dh_cuda_debug(bk, 0, 0)
    elif args.no_swiglu_amax:
        h.dh_cuda_debug(bk, 0, 3)
    if args.gemv_flags:
        d.det_debug_set_gemv(args.gemv_flags)
    if args.rows_wide_min >= 0:
        d.det_debug_set_rows(args.rows_wide_min)
    if args.tc_splitk:
        d.det_debug_set_tc_variant(0x100)
    dist, comm, saved_stdout = _tensor_parallel(args, h, rank, world, shape, rows=8)
    if world == 1 and args.emulate_tp > 1:
        # timing aid: this process runs the launch sequence of rank 0 of an N-way shard with every exchange looped back
        # to its own memory (no peer latency, meaningless values): what one rank costs without waiting for the others
        mixw = shape["n_h"] * shape["hd"]
        staging = 16 * max(chunk * max(mixw, shape["ffn"], shape["hidden"]), shape["vocab"]) + 4096
        comm = h.dh_peer_comm_new(None, 0, args.emulate_tp, staging)
        if not comm:
            raise RuntimeError(h.dh_last_error().decode())
        h.dh_peer_comm_open_loopback(comm)
    t_load = time.perf_counter()
    model = h.dh_model_new_synth_tp(bk, cfg.encode(), args.layers, SEED, max_ctx, chunk, comm)
    if not model:
        raise RuntimeError(h.dh_last_error().decode())
    d.det_sync()
    t_load = time.perf_counter() - t_load
    ev = Events(d.det_cuda_stream())
    sampler = ClockSampler(local_rank)
    sampler.start()
    windows = []

    def barrier():
        d.det_sync()
        if dist:
            dist.barrier()

    def max_over_ranks(ms: float) -> float:
        if not dist:
            return ms
        import torch
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- prefill (P tokens in `chunk`-token batches), timed for the secondary metric
    ids = _prompt(h, P, shape["vocab"])
    # warm-up: one chunk through every prefill kernel and exchange (first-use set-up of descriptors and of the NCCL
    # channels is not part of the rate), then back to an empty context
    _check(h.dh_model_prefill(model, ids.ctypes.data, min(P, chunk)), h)
    _check(h.dh_model_reset(model), h)
    barrier()
    w0 = time.time()
    a = ev.record()
    _check(h.dh_model_prefill(model, ids.ctypes.data, P), h)
    b = ev.record()
    prefill_ms = max_over_ranks(ev.ms(a, b))
    windows.append((w0, time.time()))
    tok = C.c_int32(0)
    rng = C.c_uint64(0)
    _check(h.dh_model_pick(model, 1, 1.0, 0, 1.0, C.byref(rng), C.byref(tok)), h)
    first_token = tok.value
    prompt_logits = None
    if world > 1 and rank == 0:
        prompt_logits = np.zeros(shape["vocab"], np.float32)
        h.dh_model_logits(model, prompt_logits.ctypes.data, prompt_logits.size)

    # ---- decode, device-resident (value): W warm-up steps (the first one captures the graph), then exactly K
    dec = h.dh_graph_decoder_new(model)
    if not dec:
        raise RuntimeError(h.dh_last_error().decode())
    out = np.zeros(max(K, W), np.int32)
    _check(h.dh_graph_decoder_enqueue(dec, tok.value, W, 1), h)
    n = h.dh_graph_decoder_finish(dec, out.ctypes.data, out.size)
    last = int(out[n - 1])
    stream_head = [first_token] + [int(x) for x in out[:n]]     # greedy tokens from the end of the prompt on
    barrier()
    rt.cudaProfilerStart()      # a profiler started with "--profile-from-start off" sees the timed decode steps only
    w0 = time.time()
    a = ev.record()
    _check(h.dh_graph_decoder_enqueue(dec, last, K, 1), h)
    b = ev.record()
    decode_ms = max_over_ranks(ev.ms(a, b))
    windows.append((w0, time.time()))
    n = h.dh_graph_decoder_finish(dec, out.ctypes.data, out.size)
    rt.cudaProfilerStop()
    graph_tokens = out[:n].copy()
    stream_head += [int(x) for x in graph_tokens]
    last = int(graph_tokens[-1])

    # ---- decode end to end through the plugin calls (host embedding -> H2D, forward, argmax, D2H) as model.rs drives it
    def eager_steps(count, tok_id):
        one = np.zeros(1, np.int32)
        t = C.c_int32(tok_id)
        for _ in range(count):
            one[0] = t.value
            _check(h.dh_model_forward(model, one.ctypes.data, 1), h)
            _check(h.dh_model_pick(model, 1, 1.0, 0, 1.0, C.byref(rng), C.byref(t)), h)
        return t.value

    last = eager_steps(W, last)
    barrier()
    w0 = time.time()
    a = ev.record()
    t_wall = time.perf_counter()
    last = eager_steps(K, last)
    b = ev.record()
    e2e_ms = max_over_ranks(max(ev.ms(a, b), (time.perf_counter() - t_wall) * 1e3))
    windows.append((w0, time.time()))

    # ---- the decode GEMV alone: every linear of the model at M = 1 (one token's GEMVs), weights 20 GB >> L2
    nbytes, nlaunch, sweep_ms = C.c_size_t(0), C.c_size_t(0), None
    if world == 1 and args.emulate_tp <= 1:
        _check(h.dh_gemv_sweep(model, 1, C.byref(nbytes), C.byref(nlaunch)), h)
        reps = 3
        barrier()
        w0 = time.time()
        a = ev.record()
        _check(h.dh_gemv_sweep(model, reps, C.byref(nbytes), C.byref(nlaunch)), h)
        b = ev.record()
        sweep_ms = ev.ms(a, b)
        windows.append((w0, time.time()))
    time.sleep(0.3)
    sampler.stop()
    err = d.det_last_error()
    if err:
        raise RuntimeError(f"device-side wait reported error {err}")
    # N > 1: rank 0 also runs the same prompt through an UNSHARDED copy of the model on its own GPU and compares the
    # last-position logits with the sharded run's, bit for bit (after every timed region; the other ranks are done)
    logits_equal = None
    if prompt_logits is not None and args.emulate_tp <= 1:
        solo = h.dh_model_new_synth(bk, cfg.encode(), args.layers, SEED, P + 16, chunk)
        if not solo:
            raise RuntimeError(h.dh_last_error().decode())
        _check(h.dh_model_prefill(solo, ids.ctypes.data, P), h)
        solo_logits = np.zeros(shape["vocab"], np.float32)
        h.dh_model_logits(solo, solo_logits.ctypes.data, solo_logits.size)
        h.dh_model_free(solo)
        logits_equal = bool(np.array_equal(solo_logits.view(np.uint32), prompt_logits.view(np.uint32)))

    if saved_stdout is not None:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)
    if rank != 0:
        return
    peak, peak_kind = _peaks()
    achieved = nbytes.value / (sweep_ms * 1e-3) / 1e9 if sweep_ms else None
    line = {
        "metric": "27B W6 decode tok/s bs1" if cfg == "27b" else f"{cfg} W6 decode tok/s bs1",
        "value": K / (decode_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": decode_ms / K, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None,
        "dtype": "int8 x W6 -> int64 (fp32 glue)", "data": "synthetic",
        "config": {"workload": f"{cfg}-shape seeded random-init W6 model (W8 head and GDN a/b), batch 1: prefill {P} tokens in "
                               f"{chunk}-token chunks, then greedy decode", "context_at_timing": P + W,
                   **({"layers_built": args.layers, "note": "reduced depth: not a result"} if args.layers else {}),
                   "parallelism": (f"EMULATED rank 0 of tp{args.emulate_tp}, exchanges looped back: not a result"
                                   if args.emulate_tp > 1 else "1 GPU") if world == 1 else
                   f"tp{world}: output-row / head tensor parallel, one batch-1 sequence; fp32 slices all-gathered " +
                   ("by NCCL" if args.exchange == "nccl" else
                    "by one peer-store kernel per rank over NVLink in decode, by NCCL in prefill"),
                   "l2": "weights streamed per token (20 GB at 27B) exceed the 126 MB L2", "seed": SEED,
                   "rot_dim": 64, "rope_theta": 1e7, "eps": 1e-6, "v_scale": 2 ** -10},
        "e2e": {"value": K / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": shape["hidden"] * 4,
                "d2h_bytes_per_step": 4},
        # tensor parallel: three of a layer's four exchanges run as prologues of the GEMVs they feed, so a Gated DeltaNet
        # layer is 6 launches (qkv|z + a|b, mixer step, out, gate|up, SwiGLU exchange + quantization, down) and an attention
        # layer 7, plus embed, head GEMV, logits gather, argmax and token feedback; "peer-rows" keeps every exchange in a
        # row kernel of its own (10 per layer), stand-alone exchanges add 4 exchange kernels, 2 residual adds and 1 quant
        "gpu_launches": K * (launches_per_token(cfg, fused=not args.no_fuse) if world == 1 else
                             (SHAPES[cfg]["layers"] * 6 + SHAPES[cfg]["layers"] // 4 + 5) if args.exchange == "peer" and not args.no_fuse else
                             SHAPES[cfg]["layers"] * (10 if args.exchange in ("peer", "peer-rows") else 17) + 6),
        "prefill": {"value": P / (prefill_ms * 1e-3), "unit": "tok/s", "tokens": P, "chunk": chunk},
        "roofline": None if achieved is None else
                    {"bound": "hbm", "kernel": "k_gemv_stream", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                     # DRAM traffic needs a profiler capture, which never runs inside a timed benchmark: the committed
                     # capture of the K = 5120 x N = 17408 launch read and wrote 1.004 - 1.008 x its algorithmic bytes
                     # (68.38 MB), and the traffic of this kernel grows with the bytes it streams, so the mean launch
                     # of the sweep is scaled by the middle of that range
                     "traffic": GEMV_TRAFFIC_RATIO * nbytes.value / max(1, nlaunch.value),
                     "traffic_how": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one K=5120 x N=17408 launch "
                                    "(profiles/k_gemv_stream_w6_k5120_n17408.md: 1.004-1.008 x algorithmic) scaled to "
                                    "the mean launch of this sweep, bytes per launch",
                     "launches": nlaunch.value, "bytes": nbytes.value, "ms": sweep_ms,
                     "how": "every linear of the model at M=1, 3 passes back to back, CUDA events on the launch queue"},
        "clocks": sampler.summary(windows),
        "load_s": t_load,
        "tokens_head": [int(x) for x in graph_tokens[:8]],
    }
    if logits_equal is not None:
        line["logits_equal_1gpu"] = logits_equal     # sharded vs unsharded last-position logits after the prompt
    if world == 1 and not args.no_cpu:
        base = cpu_baseline(h, cfg, os.cpu_count() or 1, tokens=args.cpu_tokens, context=min(P, args.cpu_context))
        if base.get("context") == P and "tokens" in base:
            # the same prompt through the CPU port: its greedy tokens must be the GPU's (27B parity at the full config)
            cpu_toks = base["tokens"]
            k = min(len(cpu_toks), len(stream_head))
            base["tokens_equal_gpu"] = cpu_toks[:k] == stream_head[:k]
            base["tokens_compared"] = k
        line["cpu_baseline"] = base
    print(json.dumps(line), flush=True)


def run_reference(args, rank: int, world: int):
    """`--impl reference`: the reference's own CPU path for the same metric.  The reference is Rust and cannot be built
    here (no cargo / rustc), so this arm times the CPU port under oracle/ — its reference backend with the restated x86
    integer GEMM of `--backend cpu` for the linears — with every host thread on a bounded slice of the same workload;
    rank 0 alone runs."""
    if rank != 0:
        return
    from det_b200 import capi
    h = capi.host()
    # build the CPU-side weights with the device generator when a GPU is present (identical rows, seconds instead of
    # minutes of f64 scale search on the host)
    if capi.cuda().det_init() == 0:
        h.dh_use_cuda_synth_rows(1)
    threads = os.cpu_count() or 1
    K, W = args.steps, args.warmup
    K = max(1, min(K, args.cpu_tokens))     # a bounded sample: the CPU needs 0.1 - 0.3 s per 27B token
    base = cpu_baseline(h, args.config, threads, tokens=K, warmup=min(W, 3), context=min(args.prefill, args.cpu_context))
    cfg = args.config
    line = {
        "impl": "reference",
        "metric": "27B W6 decode tok/s bs1" if cfg == "27b" else f"{cfg} W6 decode tok/s bs1",
        "value": base["value"], "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": min(W, 3),
        "ms_per_step": 1e3 / base["value"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 x W6 -> int64 (fp32 glue)", "data": "synthetic",
        "config": {"workload": f"{cfg}-shape seeded random-init W6 model (W8 head and GDN a/b), batch 1: prefill "
                               f"{base['context']} tokens, then greedy decode, on host cores",
                   "context_at_timing": base["context"] + min(W, 3), "sample": base["sample"]},
        "cpu_baseline": base,
        "prefill": base.get("prefill"),
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_serving(args, rank: int, world: int, local_rank: int):
    """The serving configuration: `--seqs` independent sequences (contexts uniform in [ctx-min, ctx-max], seeded) decode
    `--new` tokens each at temp 0.7 / top-p 0.95 / top-k 40 with per-sequence seeds, one batched step per token.  Not the
    headline line: a second workload, printed in the same format (one step = one token for every sequence).  At N > 1 the
    model is tensor parallel: every GPU serves every sequence with its share of the heads, columns and rows (the weights
    are read once per step for all rows), so `value` is the whole job's rate and the timing is the maximum over ranks."""
    import numpy as np
    from det_b200 import capi
    rt = C.CDLL("libcudart.so.12")
    assert rt.cudaSetDevice(local_rank) == 0
    h, d = capi.host(), capi.cuda()
    cfg, shape = args.config, SHAPES[args.config]
    B, new = args.seqs, args.new
    rng = np.random.default_rng(SEED)
    ctxs = [int(x) for x in rng.integers(args.ctx_min, args.ctx_max + 1, B)]
    bk = h.dh_cuda_backend_new(1, 1)
    if not bk:
        raise RuntimeError(h.dh_last_error().decode())
    if args.compose_rows:
        h.dh_cuda_set_fuse_rows(bk, 0)
    if args.tc_splitk:
        d.det_debug_set_tc_variant(0x100)
    dist, comm, saved_stdout = _tensor_parallel(args, h, rank, world, shape, rows=max(8, B))
    if world == 1 and args.emulate_tp > 1:
        # timing aid: the launch sequence of rank 0 of an N-way shard, every exchange looped back to local memory
        mixw = shape["n_h"] * shape["hd"]
        staging = 16 * max(max(args.chunk, B) * max(mixw, shape["ffn"], shape["hidden"]), shape["vocab"]) + 4096
        comm = h.dh_peer_comm_new(None, 0, args.emulate_tp, staging)
        if not comm:
            raise RuntimeError(h.dh_last_error().decode())
        h.dh_peer_comm_open_loopback(comm)
    model = h.dh_model_new_synth_tp(bk, cfg.encode(), args.layers, SEED, 16, max(args.chunk, B), comm)
    if not model:
        raise RuntimeError(h.dh_last_error().decode())
    batch = h.dh_batch_new(model, B, max(ctxs) + new + 1)
    if not batch:
        raise RuntimeError(h.dh_last_error().decode())
    ev = Events(d.det_cuda_stream())
    sampler = ClockSampler(local_rank)
    sampler.start()
    t0 = time.perf_counter()
    for i, n in enumerate(ctxs):
        ids = np.zeros(n, np.int32)
        h.dh_synth_prompt(PROMPT_SEED + i, n, shape["vocab"], ids.ctypes.data)
        _check(h.dh_batch_prefill(batch, i, ids.ctypes.data, n, 0, 1.0 / 0.7, 40, 0.95, 1000 + i), h)
    d.det_sync()
    prefill_s = time.perf_counter() - t0
    W = args.warmup
    _check(h.dh_batch_step(batch, W), h)
    d.det_sync()
    if dist:
        dist.barrier()
    rt.cudaProfilerStart()      # a profiler started with "--profile-from-start off" sees the timed steps only
    w0 = time.time()
    marks = [ev.record()]
    for _ in range(new - 1 - W):
        _check(h.dh_batch_step(batch, 1), h)
        marks.append(ev.record())
    steps_ms = [ev.ms(a, b) for a, b in zip(marks[:-1], marks[1:])]
    rt.cudaProfilerStop()
    window = (w0, time.time())
    time.sleep(0.3)
    sampler.stop()
    if d.det_last_error():
        raise RuntimeError("device-side wait reported an error")
    K = len(steps_ms)
    head = np.zeros(4, np.int32)
    h.dh_batch_tokens(batch, 0, head.ctypes.data, 4)
    if dist:
        # every rank steps through the same exchanges, so step i ends at about the same time everywhere: take the
        # slowest rank per step; all ranks must have drawn the same tokens
        import torch
        t = torch.tensor(steps_ms, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        steps_ms = [float(x) for x in t]
        heads = [torch.zeros(4, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(heads, torch.from_numpy(head.copy()))
        if any(not torch.equal(heads[0], x) for x in heads):
            raise RuntimeError("ranks disagree on the sampled tokens")
        dist.barrier()
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)
        if rank != 0:
            h.dh_batch_free(batch)
            return
    total_ms = sum(steps_ms)
    # algorithmic bytes of one step: every linear's packed weights once, each sequence's K and V rows up to its position
    # (int8 + int16 per element, plus the fp32 key scales) and its Gated DeltaNet state read and written
    n_attn = shape["layers"] // 4 if not args.layers else args.layers // 4
    n_layers = args.layers or shape["layers"]
    kv_row = shape["n_kv"] * (shape["hd"] * 3 + 4)
    mid = [c + W + (new - 1 - W) // 2 for c in ctxs]
    state = shape["n_v"] * 128 * 128 * 4 * 2
    step_bytes = (_weights_gb(cfg) * 1e9 * (n_layers / shape["layers"] if args.layers else 1.0)
                  + n_attn * kv_row * sum(mid) + (n_layers - n_attn) * state * B)
    hbm, kind = _peaks()
    achieved = step_bytes / (total_ms / K * 1e-3) / 1e9 / world
    print(json.dumps({
        "metric": f"{cfg} W6 serving decode tok/s, {B} sequences", "value": B * K / (total_ms * 1e-3), "unit": "tok/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": total_ms / K, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "int8 x W6 -> int64 (fp32 glue)", "data": "synthetic",
        "config": {"workload": f"{cfg}-shape seeded random-init W6 model, {B} sequences with contexts uniform in "
                               f"[{args.ctx_min}, {args.ctx_max}], {new} tokens each at temp 0.7 / top-k 40 / top-p 0.95, "
                               f"per-sequence seeds; one batched step per token",
                   "contexts": ctxs, **({"layers_built": args.layers, "note": "reduced depth: not a result"} if args.layers else {}),
                   "parallelism": f"tp{world}: every GPU serves every sequence with 1/{world} of the heads, FFN columns and "
                                  f"output rows; exchange {args.exchange}" if world > 1 else
                                  (f"EMULATED rank 0 of tp{args.emulate_tp}, exchanges looped back: not a result"
                                   if args.emulate_tp > 1 else "1 GPU"),
                   "rows_path": "composed per-sequence calls" if args.compose_rows else
                   "det_attention_rows / det_gdn_rows", "l2": "weights streamed per step exceed the 126 MB L2"},
        "per_token_ms": {"p50": float(np.percentile(steps_ms, 50)), "p99": float(np.percentile(steps_ms, 99))},
        "roofline": {"bound": "hbm", "kernel": "whole step", "achieved": achieved, "peak": hbm, "unit": "GB/s per GPU",
                     "frac": achieved / hbm, "peak_kind": f"of {kind}", "traffic": None, "bytes": int(step_bytes),
                     "how": "weights + KV rows + GDN state bytes of one step / mean step time / GPUs"},
        "prefill": {"tokens": int(sum(ctxs)), "value": sum(ctxs) / prefill_s, "unit": "tok/s (host wall clock, sequence by sequence)"},
        "clocks": sampler.summary([window]),
        "tokens_head": [int(x) for x in head],
    }))
    h.dh_batch_free(batch)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="27b", choices=sorted(SHAPES))
    ap.add_argument("--prefill", type=int, default=2048)
    ap.add_argument("--chunk", type=int, default=512)
    ap.add_argument("--exchange", default="peer", choices=["peer", "peer-rows", "peer-unfused", "nccl"],
                    help="N > 1: decode exchanges as one peer-memory kernel per rank (default) or as NCCL all-gathers")
    ap.add_argument("--emulate-tp", type=int, default=0,
                    help="timing aid at N = 1: run rank 0 of a P-way shard with exchanges looped back (values meaningless)")
    ap.add_argument("--layers", type=int, default=0,
                    help="build only the first L layers of the configuration (a small case for profiler captures; the "
                         "line says so and is not a result)")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving"],
                    help="decode: the headline batch-1 token loop; serving: many sequences, one batched step per token")
    ap.add_argument("--seqs", type=int, default=32)
    ap.add_argument("--ctx-min", type=int, default=512)
    ap.add_argument("--ctx-max", type=int, default=8192)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--no-fuse", action="store_true",
                    help="measurement switch: every decode op as its own launch (no prologue / epilogue / dual fusion)")
    ap.add_argument("--no-swiglu-amax", action="store_true",
                    help="measurement switch: quantize the SwiGLU product with its own launch (same tokens)")
    ap.add_argument("--gemv-flags", type=int, default=0,
                    help="measurement switch of the decode GEMV (det_debug_set_gemv): n << 4 = n worker warps per CTA, "
                         "n << 9 = n slots per worker")
    ap.add_argument("--rows-wide-min", type=int, default=-1,
                    help="measurement switch: rows from which the row kernels use one CTA per row (det_debug_set_rows)")
    ap.add_argument("--tc-splitk", action="store_true",
                    help="measurement switch: the tensor-core GEMM splits K for linears with few row tiles (same values)")
    ap.add_argument("--compose-rows", action="store_true",
                    help="serving: per-sequence attention / GDN calls instead of the batched kernels (same tokens)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--cpu-tokens", type=int, default=8, help="decode tokens the CPU baseline times")
    ap.add_argument("--cpu-context", type=int, default=2048,
                    help="prompt tokens the CPU baseline prefills before timing (capped by --prefill)")
    ap.add_argument("--no-pdl", action="store_true", help="measurement switch: plain stream-ordered launches")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    from det_b200 import build
    if rank == 0 and not (build.LIB / "libdet_host.so").exists():
        build.build_all()
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        if world == 1:
            from det_b200 import capi
            capi.host().dh_use_cuda_synth_rows(1)   # the cpu_baseline leg builds its weights with the device generator
        if args.workload == "serving":
            run_serving(args, rank, world, local_rank)
        else:
            run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
