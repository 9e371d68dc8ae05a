#!/usr/bin/env python
"""Benchmark of the fused per-layer operator path.

A *step* is one pass of the hot path over one prompt: the embedding gather followed by the operator
chains of all 64 layers (48 gated-delta-net + 16 full-attention) over every token row of the prompt.
The prompt is the long-context configuration, 131072 tokens (``--config 3`` selects the 60000-token
row-partition configuration instead); with N GPUs its rows are cut into N contiguous chunk-aligned
shards, one per rank, with no collective on the data path (strong scaling: the prompt is the same at
every N).  Every tensor is far larger than the 126 MB L2, so no flush is needed between iterations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 4|3] [--impl ours|reference]

Prints ONE JSON line (rank 0): whole-job tokens/s with inputs resident in HBM (`value`), the same
through the C ABI with host buffers and the copies inside the timed region (`e2e`, with the bound the
copies alone set), the roofline of the dominant kernel, a per-operator table (microseconds, GB/s,
fraction of the HBM peak, and microseconds x SM MHz so that runs under different power-cap states can
be compared), the CPU baseline and the clocks seen under load.

`--impl reference` times the reference's own host reference ops (oracle/_ref when it was built, else
the C restatement) on all host cores, every step a pass of all 64 layers over a bounded sample of the
prompt's rows.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "prefill tokens/s through the fused layer-op chain (embedding + 64 layers)"
UNIT = "tokens/s"
CONFIG_TOKENS = {4: 131072, 3: 60000}
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "swiglu_dram_traffic.txt")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", type=int, default=4, choices=sorted(CONFIG_TOKENS),
                    help="4 = the 131072-token long-context prompt (default), 3 = the 60000-token row partition")
    ap.add_argument("--total-tokens", type=int, default=None, help="prompt length (overrides --config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-sample-tokens", type=int, default=1024)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--probe-ms", type=float, default=120.0, help="aimed-at duration of one operator probe")
    ap.add_argument("--probe-only", action="store_true",
                    help="time each operator alone (few launches; the form profiled under ncu) and exit")
    ap.add_argument("--probe-reps", type=int, default=3)
    ap.add_argument("--no-probes", action="store_true",
                    help="skip the per-operator and decode probes (the form whose launch list is profiled)")
    ap.add_argument("--decode-only", action="store_true",
                    help="time only the batch-one (decode) step and operators and exit")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, the recipe's stated figure)"


def swiglu_traffic():
    """DRAM bytes per token of the dominant kernel from the tracked ncu summary (None when absent)."""
    info = {}
    try:
        with open(TRAFFIC_FILE) as f:
            for line in f:
                if ":" in line and not line.lstrip().startswith("#"):
                    k, v = line.split(":", 1)
                    info[k.strip()] = v.strip()
        return float(info["dram_bytes_per_token"]), info.get("captured_at_commit"), info.get("capture_tokens")
    except Exception:
        return None, None, None


# ------------------------------------------------------------------------------------ clocks

class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU while a region runs: NVML in a thread of
    this process when pynvml is importable (a few hundred samples per second), else an `nvidia-smi -lms`
    child.  Read-only: no clock or limit is ever set."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    _nvml = None
    _handles = {}

    @classmethod
    def _handle(cls, cuda_index):
        if cls._nvml is None:
            import pynvml

            pynvml.nvmlInit()
            cls._nvml = pynvml
        if cuda_index not in cls._handles:
            import torch

            uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            cls._handles[cuda_index] = cls._nvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        return cls._handles[cuda_index]

    def __init__(self, cuda_index: int, period_s: float = 0.004):
        self.sm, self.power, self.reasons = [], [], set()
        self.max_mhz = None
        self.proc = None
        self.thread = None
        self._stop = threading.Event()
        try:
            h = self._handle(cuda_index)
            n = self._nvml
            self.max_mhz = float(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM))

            def loop():
                while not self._stop.is_set():
                    try:
                        self.sm.append(float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)))
                        self.power.append(n.nvmlDeviceGetPowerUsage(h) / 1000.0)
                        mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                        for bit, name in self.REASONS.items():
                            if mask & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    time.sleep(period_s)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
            try:
                self.proc = subprocess.Popen(
                    ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                     "-i", str(cuda_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            except Exception:
                self.proc = None

    def stop(self):
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
        elif self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                out, _ = self.proc.communicate(timeout=5)
            except Exception:
                self.proc.kill()
                out = ""
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            mx = []
            for line in out.splitlines():
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    self.sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                    self.power.append(float(parts[3]))
                except ValueError:
                    continue
                for nme, v in zip(names, parts[5:9]):
                    if v.lower().startswith("active"):
                        self.reasons.add(nme)
            self.max_mhz = max(mx) if mx else None
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source"]}
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "power_w_max": max(self.power) if self.power else None, "samples": len(self.sm),
                "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------------------------ CPU arm

def cpu_chain_runner(sample_tokens: int, threads: int):
    """Sets up the reference's host reference ops over `sample_tokens` token rows: the embedding gather and
    all 64 layers in the model's pattern (GDN, GDN, GDN, full attention, x16), rows split over `threads`
    host threads.  Returns (run, kind); every run() call is one timed pass over the same inputs and returns
    its wall-clock seconds."""
    import ctypes as C

    import numpy as np

    from oracle import oracle as orc

    orc.build()
    L = orc.oracle_lib()
    R = orc.ref_lib()
    kind = "reference" if R is not None else "port"
    u16p, f32p, u8p, u32p = (C.POINTER(C.c_uint16), C.POINTER(C.c_float), C.POINTER(C.c_uint8), C.POINTER(C.c_uint32))
    rng = np.random.default_rng(0)
    T, H, I = sample_tokens, 5120, 17408

    def bf(shape, std=1.0):
        # N(0, std) values; long tensors repeat a 256-row block (the ops are row-local and their cost does
        # not depend on the values)
        rows = shape[0] if len(shape) > 1 else 1
        if rows <= 256:
            return orc.bf16_encode((rng.standard_normal(shape) * std).astype(np.float32))
        block = orc.bf16_encode((rng.standard_normal((256,) + tuple(shape[1:])) * std).astype(np.float32))
        return np.ascontiguousarray(np.tile(block, (-(-rows // 256),) + (1,) * (len(shape) - 1))[:rows])

    inp = dict(proj=bf((T, H)), raw=bf((T, 10240)), core=bf((T, 6144)), z=bf((T, 6144)), qg=bf((T, 12288)),
               key=bf((T, 1024)), val=bf((T, 6144)), gate=bf((T, I)), up=bf((T, I)))
    w = dict(norm=bf((H,), 0.02), qn=bf((256,), 0.02), kn=bf((256,), 0.02), gn=bf((128,), 1.0), conv=bf((10240, 4), 0.5))
    cos, sin = orc.rope_tables(0, T)
    res = [bf((T, H)), np.empty((T, H), np.uint16)]
    nrm = np.empty((T, H), np.uint16)
    conv_out = np.empty((T, 10240), np.uint16)
    q_l2, k_l2 = np.empty((T, 2048), np.uint16), np.empty((T, 2048), np.uint16)
    gdn_out = np.empty((T, 6144), np.uint16)
    q_out, gate_out = np.empty((T, 6144), np.uint16), np.empty((T, 6144), np.uint16)
    attn_out, mlp_out = np.empty((T, 6144), np.uint16), np.empty((T, I), np.uint16)
    codes, scales = np.empty((T, H // 2), np.uint8), np.empty((T, H // 16), np.uint8)
    gcodes, gscales = np.empty((T, 3072), np.uint8), np.empty((T, 384), np.uint8)
    gs = np.full(max(1, -(-T // 512)), 0.0025, np.float32)
    qscale = float(np.float32(1.0) / np.sqrt(np.float32(128.0)))
    eps = 1e-6
    table = bf((4096, H), 0.02)
    ids = rng.integers(0, 4096, size=T, dtype=np.uint32)
    emb = np.empty((T, H), np.uint16)

    def at(a, row, ty=u16p):
        return C.cast(a.ctypes.data + row * a.strides[0], ty)

    def residual_norm(src, dst, lo, hi):
        n = hi - lo
        if R is not None:
            R.residual_add(at(res[src], lo), at(inp["proj"], lo), n * H, at(res[dst], lo))
            R.head_centered(at(res[dst], lo), at(w["norm"], 0), n, H, eps, at(nrm, lo))
        else:
            L.residual_norm(at(res[src], lo), at(inp["proj"], lo), at(w["norm"], 0), n, H, eps, at(res[dst], lo),
                            at(nrm, lo))
        # the NVFP4 activation encoder has no reference implementation: the restatement is timed
        L.quant_ws(at(nrm, lo), n, H, 0, gs.ctypes.data_as(f32p), at(codes, lo, u8p), at(scales, lo, u8p))

    def mlp(lo, hi):
        (R.silu_mul if R is not None else L.silu_mul)(at(inp["gate"], lo), at(inp["up"], lo), (hi - lo) * I,
                                                     at(mlp_out, lo))

    def gdn_layer(src, dst, lo, hi):
        n = hi - lo
        residual_norm(src, dst, lo, hi)
        hist = np.zeros((10240, 3), np.uint16)
        if lo >= 3:
            hist[:] = inp["raw"][lo - 3:lo].T
        if R is not None:
            R.conv_rows(at(inp["raw"], lo), n, at(w["conv"], 0), at(hist, 0), at(conv_out, lo))
        else:
            L.conv(at(inp["raw"], lo), n, 10240, at(w["conv"], 0), at(hist, 0), at(conv_out, lo))
        # q/k L2 norm over the heads of each row (strided views are gathered into compact buffers first,
        # outside the op; the reference's op has no q scale, which costs nothing either way)
        q_l2[lo:hi] = conv_out[lo:hi, :2048]
        k_l2[lo:hi] = conv_out[lo:hi, 2048:4096]
        for blk, sc in ((q_l2, qscale), (k_l2, 1.0)):
            if R is not None:
                R.l2(at(blk, lo), n * 16, 128, eps, at(blk, lo))
            else:
                L.l2(at(blk, lo), n * 16, 128, eps, sc, at(blk, lo))
        if R is not None:
            R.head_plain_gate(at(inp["core"], lo), at(w["gn"], 0), at(inp["z"], lo), n * 48, 128, eps, at(gdn_out, lo))
        else:
            L.headwise(at(inp["core"], lo), at(w["gn"], 0), at(inp["z"], lo), n * 48, 128, eps, 0, at(gdn_out, lo))
        L.quant_ws(at(gdn_out, lo), n, 6144, 0, gs.ctypes.data_as(f32p), at(gcodes, lo, u8p), at(gscales, lo, u8p))
        residual_norm(dst, src, lo, hi)
        mlp(lo, hi)

    def fa_layer(src, dst, lo, hi):
        n = hi - lo
        residual_norm(src, dst, lo, hi)
        fn = R.preprocess_rows if R is not None else L.preprocess
        fn(at(inp["qg"], lo), at(inp["key"], lo), at(w["qn"], 0), at(w["kn"], 0), eps, at(q_out, lo), at(gate_out, lo),
           cos.ctypes.data_as(f32p), sin.ctypes.data_as(f32p), lo, n)
        (R.sigmoid_gate if R is not None else L.sigmoid_gate)(at(inp["val"], lo), at(gate_out, lo), n * 6144,
                                                             at(attn_out, lo))
        residual_norm(dst, src, lo, hi)
        mlp(lo, hi)

    def whole_chain(lo, hi):
        if R is not None:
            R.embedding_rows(at(table, 0), 4096, H, C.cast(ids.ctypes.data + lo * 4, u32p), hi - lo, at(emb, lo))
        else:
            L.embedding(at(table, 0), 4096, H, C.cast(ids.ctypes.data + lo * 4, u32p), hi - lo, at(emb, lo))
        for layer in range(64):
            (fa_layer if (layer + 1) % 4 == 0 else gdn_layer)(0, 1, lo, hi)

    def run():
        t0 = time.perf_counter()
        orc.parallel_rows(whole_chain, T, threads)
        return time.perf_counter() - t0

    return run, kind


CPU_SAMPLE_NOTE = ("{n}-token sample of the prompt, embedding gather + all 64 layers (GDN,GDN,GDN,FA x16) through the "
                   "reference's host ops, rows over {c} threads; NVFP4 encoder from the C restatement; "
                   "tokens/s = sample tokens / wall time of the pass (the ops are row-local, so the rate does not "
                   "depend on the prompt length)")


def cpu_tokens_per_second(sample_tokens: int, threads: int, warmup: int = 1, repeats: int = 3):
    run, kind = cpu_chain_runner(sample_tokens, threads)
    for _ in range(warmup):
        run()
    times = [run() for _ in range(max(1, repeats))]
    mean = sum(times) / len(times)
    return sample_tokens / mean, mean, kind


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    run, kind = cpu_chain_runner(args.cpu_sample_tokens, threads)
    times = []
    for i in range(args.warmup + args.steps):
        t = run()
        if i >= args.warmup:
            times.append(t)
    per_step = sum(times) / len(times)
    value = args.cpu_sample_tokens / per_step
    total = args.total_tokens or CONFIG_TOKENS[args.config]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 storage, fp32 arithmetic", "data": "synthetic",
        "config": workload_config(total, args.gpus, None),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "extrapolated": False,
                         "sample_tokens": args.cpu_sample_tokens,
                         "sample": CPU_SAMPLE_NOTE.format(n=args.cpu_sample_tokens, c=threads)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def workload_config(total_tokens, gpus, tokens_this_rank):
    name = {131072: "configs[4] long context: the 131072-token synthetic prompt",
            60000: "configs[3]: 60000 uniformly drawn token ids"}.get(total_tokens, f"{total_tokens}-token prompt")
    cfg = {
        "workload": name + ", embedding gather + 64 layers (48 GDN + 16 full-attention) of fused layer ops, "
                           f"token rows partitioned over {gpus} GPU(s) in 512-token chunks",
        "total_tokens": total_tokens, "layers": 64, "hidden": 5120, "intermediate": 17408,
        "nvfp4_scale_scope_tokens": 512, "parallelism": f"token-row shards x{gpus}, no collective",
        "l2_policy": "every tensor is larger than L2 (>= 140 MB per operand at the smallest shard); no flush",
    }
    if tokens_this_rank is not None:
        cfg["tokens_rank0"] = tokens_this_rank
    return cfg


# ------------------------------------------------------------------------------------ GPU arm

def probe_ops(stack, chain, stream_obj, T, peak, warm, reps=None, aim_ms=120.0, cuda_index=0, sample_clocks=True):
    """Times every fused operator alone with CUDA events on its own stream: microseconds per call,
    algorithmic GB/s, the fraction of the HBM peak, and the SM clock sampled while the probe ran
    (us x MHz compares runs whose power-cap state differs).  Each probe repeats its operator for about
    `aim_ms` so that the clock samples fall inside it."""
    import torch

    stream = stream_obj.cuda_stream
    probes = {
        "embedding_gather": lambda: stack.op_embedding(stream),
        "residual_rmsnorm_nvfp4": lambda: stack.op_residual_norm(0, 0, 0, 1, stream),
        "conv1d_silu_l2norm": lambda: stack.op_conv(0, stream),
        "gated_rmsnorm_nvfp4": lambda: stack.op_gated_norm(0, stream),
        "attention_preprocess": lambda: stack.op_preprocess(3, stream),
        "sigmoid_gate": lambda: stack.op_sigmoid_gate(stream),
        "swiglu": lambda: stack.op_swiglu(stream),
        # extra operators, not part of the step: the pointwise ops with the NVFP4 operand of the next projection
        "swiglu_nvfp4": lambda: stack.op_swiglu_nvfp4(stream),
        "sigmoid_gate_nvfp4": lambda: stack.op_sigmoid_gate_nvfp4(stream),
    }
    per_op = {}
    with torch.cuda.stream(stream_obj):
        for name, fn in probes.items():
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(warm - 1):
                fn()
            e0.record(stream_obj)
            fn()
            e1.record(stream_obj)
            stream_obj.synchronize()
            n = reps if reps else max(5, min(2000, int(math.ceil(aim_ms / max(e0.elapsed_time(e1), 1e-3)))))
            sampler = ClockSampler(cuda_index) if sample_clocks else None
            e0.record(stream_obj)
            for _ in range(n):
                fn()
            e1.record(stream_obj)
            stream_obj.synchronize()
            clk = sampler.stop() if sampler else {"sm_mhz": None}
            us = e0.elapsed_time(e1) * 1e3 / n
            gbs = chain.BYTES_PER_TOKEN[name] * T / (us * 1e-6) / 1e9
            per_op[name] = {"us": round(us, 2), "algorithmic_GBs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4),
                            "bytes_per_token": chain.BYTES_PER_TOKEN[name], "kernels": chain.KERNELS[name],
                            "launches_timed": n, "sm_mhz": clk.get("sm_mhz"),
                            "us_x_mhz": round(us * clk["sm_mhz"], 0) if clk.get("sm_mhz") else None}
    stack.check_error("operator probes")
    return per_op


def decode_step_probe(chain, position=131071, reps=20):
    """The same 64-layer operator chain for ONE token at `position` (batch-one decode runs on one GPU):
    microseconds per step of a CUDA-graph replay, launch-latency bound.  Two graphs: every operator in stream
    order (321 dependent kernel nodes), and the operators that do not depend on one another on three parallel
    branches (the residual + norm chain, 129 nodes, is then the critical path)."""
    import torch

    def replay_us(capture):
        stack = chain.LayerStack(1, first_position=position, seed=5, table_rows=8192)
        side = torch.cuda.Stream()
        extra = (torch.cuda.Stream(), torch.cuda.Stream())
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            capture(stack, side, extra)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            capture(stack, torch.cuda.current_stream(), extra)
        with torch.cuda.stream(side):
            graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(reps):
                graph.replay()
            e1.record(side)
        side.synchronize()
        stack.check_error("decode probe")
        return round(e0.elapsed_time(e1) * 1e3 / reps, 1), stack

    serial, ref = replay_us(lambda st, main, extra: st.enqueue_step(main.cuda_stream))
    branched, got = replay_us(lambda st, main, extra: st.enqueue_step_branched(main, *extra))
    same = all(torch.equal(getattr(ref, n).view(torch.uint8), getattr(got, n).view(torch.uint8))
               for n in ("normalized", "codes", "scales", "conv_out", "gdn_out", "gdn_codes", "q_out", "attn_out", "mlp_out"))
    same = same and all(torch.equal(a.view(torch.uint8), b.view(torch.uint8)) for a, b in zip(ref.residual, got.residual))
    if not same:
        raise SystemExit("the branched decode graph does not reproduce the serial one bit for bit")
    return {"tokens": 1, "position": position, "us_per_step": branched, "us_per_step_stream_order": serial,
            "kernels_per_step": chain.kernels_per_step(), "critical_path_kernels": 1 + 2 * chain.LAYERS,
            "note": "us_per_step: independent operators on three parallel graph branches; us_per_step_stream_order: "
                    "all 321 kernels in one dependency chain; outputs bit-identical"}


def probe_decode_ops(peak, cuda_index=0, aim_ms=60.0):
    """The batch-one (decode) operators that sit between the fused layer ops, each alone at the model's shapes,
    timed like the per-operator table: the GDN recurrence step with its gated-norm epilogue (state 48 x 128 x 128
    bf16 in and out), split-KV attention + sigmoid gate at position 131071 (K and V caches read once), the
    MLP-sized NVFP4 / FP8 / bf16 GEMVs (weights read once) and the greedy argmax over the vocabulary.  Bytes are
    algorithmic: every operand crosses HBM once.  Operands are rotated over several copies so that the 126 MB L2
    cannot serve a repeat."""
    import torch

    pkg = importlib.import_module("qwen3x-orin_b200")
    capi = pkg.capi
    dev = torch.device("cuda", cuda_index)
    gen = torch.Generator(device=dev).manual_seed(77)
    stream_obj = torch.cuda.Stream()
    stream = stream_obj.cuda_stream

    def bf(shape, std=1.0):
        return (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std).to(torch.bfloat16)

    def u8(shape, lo=0, hi=256):
        return torch.randint(lo, hi, shape, generator=gen, device=dev, dtype=torch.int32).to(torch.uint8)

    out = {}

    def timed(name, calls, nbytes):
        """calls: list of zero-argument launches (rotating operand copies); nbytes: bytes one launch moves.
        The launches are captured into one CUDA graph (a Python call costs more than the shortest of these
        kernels runs) and the graph is replayed for about aim_ms."""
        with torch.cuda.stream(stream_obj):
            for c in calls:
                c()
        stream_obj.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream_obj):
            for c in calls:
                c()
        with torch.cuda.stream(stream_obj):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream_obj)
            graph.replay()
            e1.record(stream_obj)
            stream_obj.synchronize()
            reps = max(3, min(4000, int(math.ceil(aim_ms / max(e0.elapsed_time(e1), 1e-3)))))
            sampler = ClockSampler(cuda_index)
            e0.record(stream_obj)
            for _ in range(reps):
                graph.replay()
            e1.record(stream_obj)
            stream_obj.synchronize()
            clk = sampler.stop()
        n = reps * len(calls)
        us = e0.elapsed_time(e1) * 1e3 / n
        gbs = nbytes / (us * 1e-6) / 1e9
        out[name] = {"us": round(us, 2), "bytes": nbytes, "algorithmic_GBs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4),
                     "launches_timed": n, "sm_mhz": clk.get("sm_mhz")}

    # --- GDN recurrence step + gated norm (decode): 40 state copies = 126 MB
    copies = 40
    conv, a, b = bf((1, 10240)), bf((1, 48)), bf((1, 48))
    A_log, dt = bf((48,)), bf((48,))
    states = [bf((48, 128, 128), 0.05) for _ in range(copies)]
    z, w = bf((1, 6144)), bf((128,))
    y = torch.empty((1, 6144), device=dev, dtype=torch.bfloat16)
    timed("gdn_update_rmsnorm_gate", [lambda s=s: capi.check("q3x_b200_gated_delta_net_update_rms_norm_silu_gate", conv, 1, a, b,
                                                             A_log, dt, s, s, 1e-6, w, z, 1e-6, y, stream) for s in states],
          2 * 48 * 128 * 128 * 2 + 10240 * 2 + 2 * 6144 * 2 + 4 * 48 * 2 + 256)
    del states
    # --- split-KV decode attention + sigmoid gate at position 131071 (one layer's cache: 537 MB, larger than L2)
    length = 131072
    q, gate = bf((24, 256)), bf((24, 256))
    kc, vc = bf((length, 4, 256)), bf((length, 4, 256))
    words = capi.lib().q3x_b200_gqa_decode_workspace_floats(length)
    ws = torch.empty(words, device=dev, dtype=torch.float32)
    o = torch.empty((24, 256), device=dev, dtype=torch.bfloat16)
    timed("gqa_decode_sigmoid_gate_131072", [lambda: capi.check("q3x_b200_gqa_attention_decode_sigmoid_gate", q, kc, vc, length,
                                                                0.0625, ws, words, gate, o, stream)],
          2 * length * 4 * 256 * 2 + 3 * 24 * 256 * 2)
    del kc, vc
    # --- batch-one projections: weights rotated over copies totalling > L2
    x5120, x17408 = bf((5120,)), bf((17408,))
    for name, rows, cols, x in (("nvfp4_gemv_17408x5120", 17408, 5120, x5120), ("nvfp4_gemv_5120x17408", 5120, 17408, x17408)):
        packs = [(u8((rows, cols // 2)), u8((rows, cols // 16), 0x20, 0x50)) for _ in range(4)]
        yb = torch.empty(rows, device=dev, dtype=torch.bfloat16)
        timed(name, [lambda p=p, x=x, yb=yb, rows=rows, cols=cols: capi.check("q3x_b200_nvfp4_gemv", p[0], p[1], 0.01, x, rows, cols,
                                                                              None, yb, stream) for p in packs],
              rows * cols // 2 + rows * cols // 16 + cols * 2 + rows * 2)
        del packs
    w8 = [u8((12288, 5120), 0x10, 0x70) for _ in range(3)]
    yb = torch.empty(12288, device=dev, dtype=torch.bfloat16)
    timed("fp8_gemv_12288x5120", [lambda p=p: capi.check("q3x_b200_fp8_gemv", p, 0.02, x5120, 12288, 5120, None, yb, stream)
                                  for p in w8], 12288 * 5120 + 5120 * 2 + 12288 * 2)
    del w8
    wb = [bf((6144, 5120), 0.05) for _ in range(3)]
    yb = torch.empty(6144, device=dev, dtype=torch.bfloat16)
    timed("bf16_gemv_6144x5120", [lambda p=p: capi.check("q3x_b200_bf16_gemv", p, x5120, 6144, 5120, None, yb, stream) for p in wb],
          6144 * 5120 * 2 + 5120 * 2 + 6144 * 2)
    del wb
    logits = [bf((248320,), 3.0) for _ in range(8)]
    rec = torch.empty(66, device=dev, dtype=torch.int32)
    timed("greedy_argmax_248320", [lambda p=p: capi.check("q3x_b200_bf16_greedy_argmax", p, 248320, rec, stream) for p in logits],
          248320 * 2)
    torch.cuda.empty_cache()
    return out


def probe_projection_ops(cuda_index=0, aim_ms=60.0, tokens=8192):
    """The prefill projection that consumes the NVFP4 activations (q3x_b200_nvfp4_gemm_bf16: block-scaled tensor
    cores, one 512-row launch per activation scale group), alone at the model's MLP and GDN-input shapes over a
    panel of `tokens` rows.  flops = 2 x tokens x out_features x in_features per call; the fractions are against
    the nominal dense FP4 rate of the part and against the measured dense bf16 GEMM of this pool (the driver
    measures no FP4 figure), both named in the record."""
    import torch

    pkg = importlib.import_module("qwen3x-orin_b200")
    capi = pkg.capi
    dev = torch.device("cuda", cuda_index)
    gen = torch.Generator(device=dev).manual_seed(78)
    stream_obj = torch.cuda.Stream()
    stream = stream_obj.cuda_stream
    bf16_peak = None
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            bf16_peak = float(json.load(f)["bf16_tflops"])
    except Exception:
        pass

    def u8(shape, lo=0, hi=256):
        return torch.randint(lo, hi, shape, generator=gen, device=dev, dtype=torch.int32).to(torch.uint8)

    out = {}
    for name, n, k in (("nvfp4_gemm_17408x5120", 17408, 5120), ("nvfp4_gemm_5120x17408", 5120, 17408),
                       ("nvfp4_gemm_10240x5120", 10240, 5120)):
        a_codes, w_codes = u8((tokens, k // 2)), u8((n, k // 2))
        a_scales = u8((capi.lib().q3x_b200_nvfp4_swizzled_scale_bytes(tokens, k),), 0x28, 0x48)
        w_scales = u8((capi.lib().q3x_b200_nvfp4_swizzled_scale_bytes(n, k),), 0x28, 0x48)
        groups = tokens // 512
        a_gs = torch.full((groups,), 0.01, device=dev, dtype=torch.float32)
        need = capi.lib().q3x_b200_nvfp4_gemm_workspace_bytes(tokens, n, k, 512)
        ws = torch.empty(need, device=dev, dtype=torch.uint8)
        y = torch.empty((tokens, n), device=dev, dtype=torch.bfloat16)

        def call():
            capi.check("q3x_b200_nvfp4_gemm_bf16", a_codes, a_scales, a_gs, 512, w_codes, w_scales, 0.01, tokens, n, k, y, ws,
                       need, stream)

        with torch.cuda.stream(stream_obj):
            call()
        stream_obj.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream_obj):
            call()
        with torch.cuda.stream(stream_obj):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream_obj)
            graph.replay()
            e1.record(stream_obj)
            stream_obj.synchronize()
            reps = max(3, min(2000, int(math.ceil(aim_ms / max(e0.elapsed_time(e1), 1e-3)))))
            sampler = ClockSampler(cuda_index)
            e0.record(stream_obj)
            for _ in range(reps):
                graph.replay()
            e1.record(stream_obj)
            stream_obj.synchronize()
            clk = sampler.stop()
        us = e0.elapsed_time(e1) * 1e3 / reps
        tflops = 2.0 * tokens * n * k / (us * 1e-6) / 1e12
        out[name] = {"tokens": tokens, "launches_per_call": 2, "us": round(us, 1), "TFLOPs": round(tflops, 1),
                     "frac_of_nominal_fp4_dense_9000": round(tflops / 9000.0, 4),
                     "frac_of_measured_bf16_dense": round(tflops / bf16_peak, 3) if bf16_peak else None,
                     "sm_mhz": clk.get("sm_mhz"), "reasons": clk.get("reasons")}
        del a_codes, w_codes, a_scales, w_scales, ws, y
    # bulk causal attention of a 512-token tile appended at positions 0, 8192 and 65536 (one layer's cache)
    for first, tile in ((0, 512), (8192, 512), (65536, 512), (0, 8192)):  # the last one runs in the wide CTA shape
        length = first + tile
        q = torch.randn((tile, 24, 256), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        gate_t = torch.randn((tile, 24, 256), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        kc = torch.randn((length, 4, 256), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        vc = torch.randn((length, 4, 256), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        y = torch.empty((tile, 24, 256), device=dev, dtype=torch.bfloat16)

        def attend():
            capi.check("q3x_b200_gqa_attention_prefill_sigmoid_gate", q, kc, vc, gate_t, first, tile, 0.0625, y, stream)

        with torch.cuda.stream(stream_obj):
            attend()
        stream_obj.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream_obj):
            attend()
        with torch.cuda.stream(stream_obj):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream_obj)
            graph.replay()
            e1.record(stream_obj)
            stream_obj.synchronize()
            reps = max(3, min(2000, int(math.ceil(aim_ms / max(e0.elapsed_time(e1), 1e-3)))))
            sampler = ClockSampler(cuda_index)
            e0.record(stream_obj)
            for _ in range(reps):
                graph.replay()
            e1.record(stream_obj)
            stream_obj.synchronize()
            clk = sampler.stop()
        us = e0.elapsed_time(e1) * 1e3 / reps
        # visible (query, key) pairs x 24 heads x 256 dims x 2 products x 2 flops
        pairs = tile * first + tile * (tile + 1) // 2
        tflops = 4.0 * pairs * 24 * 256 / (us * 1e-6) / 1e12
        out[f"gqa_prefill_{tile}_tokens_at_{first}"] = {"us": round(us, 1), "TFLOPs": round(tflops, 1),
                                                     "frac_of_measured_bf16_dense": round(tflops / bf16_peak, 3) if bf16_peak else None,
                                                     "sm_mhz": clk.get("sm_mhz")}
        del q, gate_t, kc, vc, y
    # the weight-only FP8 projections (bf16 activations, E4M3 weights, per-tensor scale) at the attention / GDN shapes
    # (and the same projections against a bf16 copy of the weight made once: exact widening, dense tensor-core path)
    for name, n, k, widened in (("fp8_w8a16_gemm_10240x5120", 10240, 5120, False), ("fp8_w8a16_gemm_12288x5120", 12288, 5120, False),
                                ("fp8_w8a16_gemm_5120x6144", 5120, 6144, False),
                                ("fp8_widened_gemm_10240x5120", 10240, 5120, True), ("fp8_widened_gemm_12288x5120", 12288, 5120, True),
                                ("fp8_widened_gemm_5120x6144", 5120, 6144, True)):
        x = (torch.randn((tokens, k), generator=gen, device=dev, dtype=torch.float32)).to(torch.bfloat16)
        w8 = u8((n, k), 0x10, 0x70)
        y = torch.empty((tokens, n), device=dev, dtype=torch.bfloat16)
        wide = torch.empty((n, k) if widened else (1,), device=dev, dtype=torch.bfloat16)
        if widened:
            capi.check("q3x_b200_fp8_weights_to_bf16", w8, n * k, wide, stream)

        def call8():
            if widened:
                capi.check("q3x_b200_bf16_gemm_scaled_bf16", wide, 0.02, x, tokens, n, k, y, None, 0, stream)
            else:
                capi.check("q3x_b200_fp8_gemm_bf16", w8, 0.02, x, tokens, n, k, y, None, 0, stream)

        with torch.cuda.stream(stream_obj):
            call8()
        stream_obj.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream_obj):
            call8()
        with torch.cuda.stream(stream_obj):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream_obj)
            graph.replay()
            e1.record(stream_obj)
            stream_obj.synchronize()
            reps = max(3, min(2000, int(math.ceil(aim_ms / max(e0.elapsed_time(e1), 1e-3)))))
            sampler = ClockSampler(cuda_index)
            e0.record(stream_obj)
            for _ in range(reps):
                graph.replay()
            e1.record(stream_obj)
            stream_obj.synchronize()
            clk = sampler.stop()
        us = e0.elapsed_time(e1) * 1e3 / reps
        tflops = 2.0 * tokens * n * k / (us * 1e-6) / 1e12
        out[name] = {"tokens": tokens, "launches_per_call": 1, "us": round(us, 1), "TFLOPs": round(tflops, 1),
                     "frac_of_measured_bf16_dense": round(tflops / bf16_peak, 3) if bf16_peak else None,
                     "frac_of_nominal_bf16_dense_2250": round(tflops / 2250.0, 4),
                     "sm_mhz": clk.get("sm_mhz"), "reasons": clk.get("reasons")}
        del x, w8, y, wide
    # the weight-only NVFP4 projections (bf16 activations, E2M1 weights, block scales as the transposed bf16 sidecar)
    # (and against a bf16 copy of code x block scale made once: exact widening, dense tensor-core path)
    for name, n, k, widened in (("nvfp4_w4a16_gemm_17408x5120", 17408, 5120, False), ("nvfp4_w4a16_gemm_5120x17408", 5120, 17408, False),
                                ("nvfp4_widened_gemm_17408x5120", 17408, 5120, True), ("nvfp4_widened_gemm_5120x17408", 5120, 17408, True)):
        x = (torch.randn((tokens, k), generator=gen, device=dev, dtype=torch.float32)).to(torch.bfloat16)
        w4 = u8((n, k // 2))
        row_scales = u8((n, k // 16), 0x28, 0x48)
        sidecar = torch.empty((k // 16, n), device=dev, dtype=torch.bfloat16)
        capi.check("q3x_b200_nvfp4_transpose_block_scales", row_scales, n, k, sidecar, stream)
        wide = torch.empty((n, k) if widened else (1,), device=dev, dtype=torch.bfloat16)
        if widened:
            capi.check("q3x_b200_nvfp4_weights_to_bf16", w4, row_scales, n, k, wide, stream)
        y = torch.empty((tokens, n), device=dev, dtype=torch.bfloat16)

        def call4():
            if widened:
                capi.check("q3x_b200_bf16_gemm_scaled_bf16", wide, 0.01, x, tokens, n, k, y, None, 0, stream)
            else:
                capi.check("q3x_b200_nvfp4_w4a16_gemm_bf16", w4, sidecar, 0.01, x, tokens, n, k, y, None, 0, stream)

        with torch.cuda.stream(stream_obj):
            call4()
        stream_obj.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream_obj):
            call4()
        with torch.cuda.stream(stream_obj):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream_obj)
            graph.replay()
            e1.record(stream_obj)
            stream_obj.synchronize()
            reps = max(3, min(2000, int(math.ceil(aim_ms / max(e0.elapsed_time(e1), 1e-3)))))
            sampler = ClockSampler(cuda_index)
            e0.record(stream_obj)
            for _ in range(reps):
                graph.replay()
            e1.record(stream_obj)
            stream_obj.synchronize()
            clk = sampler.stop()
        us = e0.elapsed_time(e1) * 1e3 / reps
        tflops = 2.0 * tokens * n * k / (us * 1e-6) / 1e12
        out[name] = {"tokens": tokens, "launches_per_call": 1, "us": round(us, 1), "TFLOPs": round(tflops, 1),
                     "frac_of_measured_bf16_dense": round(tflops / bf16_peak, 3) if bf16_peak else None,
                     "frac_of_nominal_bf16_dense_2250": round(tflops / 2250.0, 4),
                     "sm_mhz": clk.get("sm_mhz"), "reasons": clk.get("reasons")}
        del x, w4, row_scales, sidecar, y, wide
    # the MLP block with its projections: residual + norm + NVFP4 -> gate / up -> SwiGLU + NVFP4 -> down
    chain = importlib.import_module("qwen3x-orin_b200.chain")
    block = chain.ProjectedMlp(tokens, dev)
    with torch.cuda.stream(stream_obj):
        block.enqueue(stream)
    stream_obj.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream_obj):
        block.enqueue(stream)
    with torch.cuda.stream(stream_obj):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream_obj)
        graph.replay()
        e1.record(stream_obj)
        stream_obj.synchronize()
        reps = max(3, min(500, int(math.ceil(aim_ms / max(e0.elapsed_time(e1), 1e-3)))))
        sampler = ClockSampler(cuda_index)
        e0.record(stream_obj)
        for _ in range(reps):
            graph.replay()
        e1.record(stream_obj)
        stream_obj.synchronize()
        clk = sampler.stop()
    block.check_error()
    us = e0.elapsed_time(e1) * 1e3 / reps
    gemm_us = 2 * out["nvfp4_gemm_17408x5120"]["us"] + out["nvfp4_gemm_5120x17408"]["us"]
    out["mlp_block_with_projections"] = {
        "tokens": tokens, "us": round(us, 1), "tokens_per_s": round(tokens / (us * 1e-6), 1),
        "TFLOPs": round(block.flops() / (us * 1e-6) / 1e12, 1), "kernels": 10,
        "share_outside_the_projections": round(1.0 - gemm_us / us, 3), "sm_mhz": clk.get("sm_mhz"),
        "note": "residual+RMSNorm+NVFP4, scale re-layout, gate and up projections, SwiGLU+NVFP4, scale re-layout, down "
                "projection; synthetic NVFP4 weights"}
    del block
    # one full-attention layer end to end (FP8 projections, head norms + RoPE, bulk causal attention + gate, output
    # projection, MLP block) for a panel of `tokens` tokens at the start of a sequence
    layer = chain.ProjectedAttentionLayer(tokens, 0, dev)
    with torch.cuda.stream(stream_obj):
        layer.enqueue(stream)
    stream_obj.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream_obj):
        layer.enqueue(stream)
    with torch.cuda.stream(stream_obj):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream_obj)
        graph.replay()
        e1.record(stream_obj)
        stream_obj.synchronize()
        reps = max(3, min(200, int(math.ceil(aim_ms / max(e0.elapsed_time(e1), 1e-3)))))
        sampler = ClockSampler(cuda_index)
        e0.record(stream_obj)
        for _ in range(reps):
            graph.replay()
        e1.record(stream_obj)
        stream_obj.synchronize()
        clk = sampler.stop()
    layer.mlp.check_error()
    us = e0.elapsed_time(e1) * 1e3 / reps
    out["full_attention_layer_with_projections"] = {
        "tokens": tokens, "first_position": 0, "us": round(us, 1), "tokens_per_s": round(tokens / (us * 1e-6), 1),
        "TFLOPs": round(layer.flops() / (us * 1e-6) / 1e12, 1), "kernels": 17, "sm_mhz": clk.get("sm_mhz"),
        "note": "residual+RMSNorm, q|gate / k / v projections (FP8 weights) into the caches, head norms + RoPE, bulk causal "
                "attention + sigmoid gate, output projection, MLP block; synthetic weights"}
    del layer
    # one gated-delta-net layer end to end (FP8 qkv / z projections, conv, token-sequential recurrence, gated norm +
    # NVFP4, NVFP4 output projection, MLP block) for the same panel
    gdn = chain.ProjectedGdnLayer(tokens, dev, chunked=True)
    with torch.cuda.stream(stream_obj):
        gdn.enqueue(stream)
    stream_obj.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream_obj):
        gdn.enqueue(stream)
    with torch.cuda.stream(stream_obj):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream_obj)
        graph.replay()
        e1.record(stream_obj)
        stream_obj.synchronize()
        reps = max(3, min(200, int(math.ceil(aim_ms / max(e0.elapsed_time(e1), 1e-3)))))
        e0.record(stream_obj)
        for _ in range(reps):
            graph.replay()
        e1.record(stream_obj)
        stream_obj.synchronize()
        # the recurrence alone, on the conv output the layer left behind: chunked (what the layer ran) and token by token
        r0, r1, r2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        r0.record(stream_obj)
        capi.check("q3x_b200_gated_delta_net_update_chunked", gdn.conv_out, tokens, gdn.a, gdn.b, gdn.A_log, gdn.dt_bias,
                   gdn.state, gdn.state, 1e-6, gdn.core, gdn.recurrence_workspace, gdn.recurrence_workspace.numel(), stream)
        r1.record(stream_obj)
        capi.check("q3x_b200_gated_delta_net_update", gdn.conv_out, tokens, gdn.a, gdn.b, gdn.A_log, gdn.dt_bias, gdn.state,
                   gdn.state, 1e-6, gdn.core, stream)
        r2.record(stream_obj)
        stream_obj.synchronize()
    gdn.check_error()
    us = e0.elapsed_time(e1) * 1e3 / reps
    out["gdn_layer_with_projections"] = {
        "tokens": tokens, "us": round(us, 1), "tokens_per_s": round(tokens / (us * 1e-6), 1), "kernels": 21,
        "recurrence_us": round(r0.elapsed_time(r1) * 1e3, 1),
        "recurrence_token_sequential_us": round(r1.elapsed_time(r2) * 1e3, 1),
        "note": "residual+RMSNorm, qkv / z (FP8 weights) and a / b (bf16 weights) projections, conv1d+SiLU, recurrence in 64-token chunks, gated "
                "RMSNorm+NVFP4, scale re-layout, NVFP4 output projection, MLP block; synthetic weights"}
    del gdn
    torch.cuda.empty_cache()
    return out


def host_memory_available_bytes():
    """What this process may still take from host memory: MemAvailable, capped by the cgroup limit."""
    avail = None
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    avail = int(line.split()[1]) * 1024
    except Exception:
        pass
    for limit_path, usage_path in (("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory.current"),
                                   ("/sys/fs/cgroup/memory/memory.limit_in_bytes",
                                    "/sys/fs/cgroup/memory/memory.usage_in_bytes")):
        try:
            with open(limit_path) as f:
                raw = f.read().strip()
            if raw != "max":
                with open(usage_path) as f:
                    used = int(f.read().strip())
                room = int(raw) - used
                avail = room if avail is None else min(avail, room)
        except Exception:
            pass
    return avail


def pinned_empty(shape, dtype):
    """A page-locked host tensor of exactly the asked size (cudaHostRegister on ordinary memory; torch's own
    pinned allocator rounds every block up to a power of two, a third more than this workload needs)."""
    import torch

    t = torch.empty(shape, dtype=dtype)
    nbytes = t.numel() * t.element_size()
    if nbytes == 0:
        return t, False
    err = torch.cuda.cudart().cudaHostRegister(t.data_ptr(), nbytes, 0)
    code = int(getattr(err, "value", err))
    if code != 0:
        return torch.empty(shape, dtype=dtype, pin_memory=True), False
    return t, True


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist

    pkg = importlib.import_module("qwen3x-orin_b200")
    chain = importlib.import_module("qwen3x-orin_b200.chain")
    shard_mod = importlib.import_module("qwen3x-orin_b200.shard")
    capi = pkg.capi
    capi.load()  # raises when the CUDA library is missing: there is no other implementation

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        # NCCL only carries the barrier, the max-over-ranks of the timings and the untimed validation
        # gather.  Whatever the communicator set-up prints (its banner, NCCL_DEBUG output) is sent to
        # stderr so that stdout holds exactly one JSON line.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    if args.decode_only:
        peak, _ = measured_peak()
        print(json.dumps({"decode_only": True, "decode_step": decode_step_probe(chain),
                          "decode_ops": probe_decode_ops(peak, local_rank, aim_ms=args.probe_ms / 2),
                          "projection_ops": probe_projection_ops(local_rank, aim_ms=args.probe_ms / 2)}), flush=True)
        return 0

    total = args.total_tokens or CONFIG_TOKENS[args.config]
    mine = shard_mod.shard_for(total, rank, world)
    T = mine.tokens
    if T == 0:
        raise SystemExit(f"rank {rank} owns no rows of a {total}-token prompt over {world} ranks")
    stack = chain.LayerStack(T, first_position=mine.first_token, seed=1234 + rank)
    stream_obj = torch.cuda.Stream()
    stream = stream_obj.cuda_stream

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        if distributed:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.probe_only:
        peak, _ = measured_peak()
        print(json.dumps({"probe_only": True, "tokens": T,
                          "per_op": probe_ops(stack, chain, stream_obj, T, peak, 1, reps=args.probe_reps,
                                              cuda_index=local_rank, sample_clocks=False)}), flush=True)
        return 0

    # ---- warm-up (eager), then capture one step into a CUDA graph ------------------------------
    with torch.cuda.stream(stream_obj):
        final_idx = stack.enqueue_step(stream)
    stream_obj.synchronize()
    graph = None
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream_obj):
                stack.enqueue_step(torch.cuda.current_stream().cuda_stream)
        except Exception as exc:  # capture is an optimisation, never a requirement
            print(f"[bench] graph capture unavailable ({exc}); launching eagerly", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def one_step():
        if graph is not None:
            graph.replay()
        else:
            stack.enqueue_step(stream)

    warmup = max(args.warmup, 3)
    with torch.cuda.stream(stream_obj):
        for _ in range(warmup):
            one_step()
    barrier()

    # ---- timed region: K steps, HBM-resident inputs ----------------------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream_obj):
        start.record(stream_obj)
        for _ in range(args.steps):
            one_step()
        stop.record(stream_obj)
    barrier()
    clocks = sampler.stop() if sampler else None
    stack.check_error("timed steps")  # sticky flag: covers every NVFP4 call since the stack was built
    ms_per_step = max_over_ranks(start.elapsed_time(stop)) / args.steps
    value = total / (ms_per_step * 1e-3)

    # ---- per-operator timing (each op alone, CUDA events on its stream) --------------------------
    peak, peak_kind = measured_peak()
    probing = rank == 0 and not args.no_probes
    per_op = probe_ops(stack, chain, stream_obj, T, peak, 3, aim_ms=args.probe_ms, cuda_index=local_rank) if probing else {}
    # dominant kernel = the SwiGLU stream (the largest share of the step's bytes, one kernel per launch)
    roofline = None
    if probing:
        sw = per_op["swiglu"]
        per_token, traffic_commit, capture_tokens = swiglu_traffic()
        roofline = {"bound": "hbm", "kernel": "binary_vec_kernel<SiluMul> (SwiGLU)", "achieved": sw["algorithmic_GBs"],
                    "peak": peak, "unit": "GB/s", "frac": round(sw["algorithmic_GBs"] / peak, 4), "peak_source": peak_kind,
                    "traffic": per_token * T if per_token else None,
                    "traffic_source": (f"ncu dram__bytes_read.sum + dram__bytes_write.sum of a {capture_tokens}-token "
                                       f"launch, scaled by tokens (profiles/{os.path.basename(TRAFFIC_FILE)})"
                                       if per_token else None),
                    "traffic_commit": traffic_commit,
                    "algorithmic_bytes_per_launch": chain.BYTES_PER_TOKEN["swiglu"] * T,
                    "us_per_launch": sw["us"], "launch_tokens": T}
        step_bytes = chain.bytes_per_token_per_step() * T
        rank_ms = start.elapsed_time(stop) / args.steps
        roofline["whole_step"] = {"algorithmic_GBs": round(step_bytes / (rank_ms * 1e-3) / 1e9, 1),
                                  "frac": round(step_bytes / (rank_ms * 1e-3) / 1e9 / peak, 4),
                                  "bytes_per_token": chain.bytes_per_token_per_step(),
                                  "sum_of_per_op_ms": round(sum(per_op[o]["us"] for l in range(64) for o in chain.layer_ops(l)) / 1e3
                                                            + per_op["embedding_gather"]["us"] / 1e3, 3),
                                  "ms_per_step_rank0": round(rank_ms, 3)}

    # ---- end to end: host buffers, H2D of the step's inputs and D2H of its result inside the timing --
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, torch, dist, stack, graph, stream_obj, final_idx, T, total, world, barrier, max_over_ranks)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        v, secs, kind = cpu_tokens_per_second(args.cpu_sample_tokens, threads)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": kind, "extrapolated": False,
               "sample_tokens": args.cpu_sample_tokens, "seconds_per_pass": round(secs, 3),
               "sample": CPU_SAMPLE_NOTE.format(n=args.cpu_sample_tokens, c=threads)}

    decode = decode_step_probe(chain) if probing else None
    decode_ops = probe_decode_ops(peak, local_rank, aim_ms=args.probe_ms / 2) if probing else None
    projection_ops = probe_projection_ops(local_rank, aim_ms=args.probe_ms / 2) if probing else None
    validation = validate_shards(rank, world, dist) if distributed else None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 storage, fp32 arithmetic", "data": "synthetic", "config": workload_config(total, world, T),
            "roofline": roofline, "per_op": per_op, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": chain.kernels_per_step() * args.steps, "cuda_graph": graph is not None, "clocks": clocks,
        }
        line["decode_step"] = decode
        line["decode_ops"] = decode_ops
        line["projection_ops"] = projection_ops
        if validation is not None:
            line["validation"] = validation
        print(json.dumps(line), flush=True)
    failed = validation is not None and not validation.get("all_ranks_bit_exact", False)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        print("[bench] the sharded run is NOT bit-identical to the unsharded run", file=sys.stderr)
        return 3
    return 0


def run_e2e(args, torch, dist, stack, graph, stream_obj, final_idx, T, total, world, barrier, max_over_ranks):
    """The step through the C ABI from pinned host buffers: two device input sets, each baked into its own
    graph; while step i computes on set i % 2 the copy engine brings step i + 1's nine synthetic projection
    outputs + ids in from pinned host memory and takes step i - 1's final residual out.  Every step's inputs
    and result cross PCIe inside the timed region.  Then the same loop with the kernels left out gives the
    bound the copies alone set on this host (all ranks copying at once)."""
    names = list(stack.inputs)
    need = sum(stack.inputs[n].numel() * 2 for n in names) + 2 * T * 5120 * 2
    avail = host_memory_available_bytes()
    # collective decision, so that every rank takes the same branch
    ok = torch.tensor([int(avail is None or need * 1.5 < avail / max(1, min(world, 8)))], device="cuda")
    if dist.is_initialized():
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if not bool(ok.item()):
        return {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "skipped": f"host memory: {need / 1e9:.1f} GB of pinned buffers needed per rank, "
                           f"{(avail or 0) / 1e9:.1f} GB available"}
    stream = stream_obj.cuda_stream
    host_in, registered = {}, []
    for n in names:
        host_in[n], reg = pinned_empty(stack.inputs[n].shape, torch.bfloat16)
        registered.append(reg)
        host_in[n].copy_(stack.inputs[n])
    host_ids, _ = pinned_empty(stack.token_ids.shape, torch.int32)
    host_ids.copy_(stack.token_ids)
    host_out = [pinned_empty((T, 5120), torch.bfloat16)[0] for _ in range(2)]
    staged_out = [torch.empty((T, 5120), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    h2d = sum(v.numel() * 2 for v in host_in.values()) + host_ids.numel() * 4
    d2h = host_out[0].numel() * 2
    stack.add_input_set()
    graphs = [graph, None]
    if graph is not None:
        try:
            stack.active = 1
            graphs[1] = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graphs[1], stream=stream_obj):
                stack.enqueue_step(torch.cuda.current_stream().cuda_stream)
        except Exception as exc:
            print(f"[bench] second graph capture failed ({exc}); e2e launches eagerly", file=sys.stderr)
            graphs = [None, None]
            torch.cuda.synchronize()
        stack.active = 0
    h2d_stream, d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
    filled = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    staged = [torch.cuda.Event() for _ in range(2)]
    drained = [torch.cuda.Event() for _ in range(2)]

    def e2e_steps(count, compute=True):
        for i in range(count):
            s = i % 2
            with torch.cuda.stream(h2d_stream):
                if i >= 2:
                    h2d_stream.wait_event(consumed[s])      # step i - 2 no longer reads this set
                for n in names:
                    stack.input_sets[s][n].copy_(host_in[n], non_blocking=True)
                stack.id_sets[s].copy_(host_ids, non_blocking=True)
                filled[s].record(h2d_stream)
            with torch.cuda.stream(stream_obj):
                stream_obj.wait_event(filled[s])
                if compute:
                    if graphs[s] is not None:
                        graphs[s].replay()
                    else:
                        stack.active = s
                        stack.enqueue_step(stream)
                        stack.active = 0
                consumed[s].record(stream_obj)
                if i >= 2:
                    stream_obj.wait_event(drained[s])       # the host copy of step i - 2's result is done
                staged_out[s].copy_(stack.residual[final_idx], non_blocking=True)
                staged[s].record(stream_obj)
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(staged[s])
                host_out[s].copy_(staged_out[s], non_blocking=True)
                drained[s].record(d2h_stream)

    def timed(count, compute):
        e2e_steps(2, compute)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(h2d_stream)
        e2e_steps(count, compute)
        d2h_stream.wait_stream(stream_obj)
        d2h_stream.wait_stream(h2d_stream)
        e1.record(d2h_stream)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / count

    e2e_ms = timed(args.steps, True)
    stack.check_error("end-to-end steps")
    copy_ms = timed(max(2, min(args.steps, 5)), False)
    out = {"value": total / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": e2e_ms,
           "copy_bound_tokens_per_s": total / (copy_ms * 1e-3), "copy_only_ms_per_step": copy_ms,
           "frac_of_copy_bound": round(copy_ms / e2e_ms, 4),
           "copy_GBs_per_gpu": round((h2d + d2h) / (copy_ms * 1e-3) / 1e9, 1),
           "host_buffers": "cudaHostRegister" if all(registered) else "torch pinned allocator",
           "note": "per step: pinned-host inputs -> device, 64-layer chain, final residual -> pinned host; the "
                   "copies of neighbouring steps overlap the chain (two device input sets); copy_bound = the same "
                   "loop with the kernels left out, all ranks copying at once (what this host's PCIe / memory "
                   "delivers), bytes counted per rank"}
    for t in list(host_in.values()) + [host_ids] + host_out:
        try:
            torch.cuda.cudart().cudaHostUnregister(t.data_ptr())
        except Exception:
            pass
    return out


def validate_shards(rank, world, dist):
    """Untimed: the shards' outputs all-gathered over NVLink and compared with an unsharded run."""
    import torch

    shard = importlib.import_module("qwen3x-orin_b200.shard")
    report = shard.validate_sharded_chain(rank, world)
    ok = torch.tensor([int(report["local_equals_unsharded"] and report["gathered_equals_unsharded"])], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    report["all_ranks_bit_exact"] = bool(ok.item())
    return report


if __name__ == "__main__":
    sys.exit(main())
