#!/usr/bin/env python
"""Benchmark of the fused per-layer operator path.

A *step* is one pass of the hot path over one batch: the embedding gather followed by the operator
chains of all 64 layers (48 gated-delta-net + 16 full-attention) over this rank's token shard.  The
default shard is 16384 tokens per GPU, i.e. the 8-way share of the 131072-token long-context
configuration, so N GPUs process N x 16384 tokens per step (weak scaling, no collective on the data
path).  Every tensor is far larger than the 126 MB L2, so no flush is needed between iterations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl ours|reference]

Prints ONE JSON line (rank 0): whole-job tokens/s with inputs resident in HBM (`value`), the same
through the C ABI with host buffers and the copies inside the timed region (`e2e`), the roofline of
the dominant kernel, a per-operator table, the CPU baseline and the clocks seen under load.

`--impl reference` times the reference's own host reference ops (oracle/_ref when it was built, else
the C restatement) on all host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "prefill tokens/s through the fused layer-op chain (embedding + 64 layers)"
UNIT = "tokens/s"


# DRAM traffic of the dominant kernel (SwiGLU), from one ncu capture of an 8192-token launch:
# dram__bytes.sum.per_second x gpu__time_duration = 817.9 MB read + written, i.e. 99841 bytes per token
# against 104448 algorithmic ones (the tail of the output is still dirty in L2 when the kernel ends).
# Traffic grows in proportion to the tokens, so a launch of T tokens is reported as this figure x T.
SWIGLU_DRAM_BYTES_PER_TOKEN = 99841
SWIGLU_TRAFFIC_SOURCE = "ncu, 8192-token launch scaled by tokens (profiles/layer_ops_8192_tokens_ncu_sections.md)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=16384, help="token rows per GPU")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-sample-tokens", type=int, default=8192)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--probe-reps", type=int, default=3)
    ap.add_argument("--probe-only", action="store_true",
                    help="time each operator alone (few launches; the form profiled under ncu) and exit")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ------------------------------------------------------------------------------------ clocks

class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu = gpu_index
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------ CPU arm

def cpu_chain_runner(sample_tokens: int, threads: int):
    """Sets up the reference's host reference ops over `sample_tokens` rows of the 4-layer pattern
    (GDN, GDN, GDN, full attention) plus the embedding gather, rows split over `threads` host threads.
    Returns (run, kind); every run() call is one timed pass over the same inputs and returns
    (seconds for 4 layers, seconds for the embedding)."""
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
        # N(0, std) values; long tensors repeat a 256-row block (the ops are row-local and their cost
        # does not depend on the values, and drawing a billion normals would take longer than the timing)
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
    gdn_out = np.empty((T, 6144), np.uint16)
    q_out, gate_out = np.empty((T, 6144), np.uint16), np.empty((T, 6144), np.uint16)
    attn_out, mlp_out = np.empty((T, 6144), np.uint16), np.empty((T, I), np.uint16)
    codes, scales = np.empty((T, H // 2), np.uint8), np.empty((T, H // 16), np.uint8)
    gcodes, gscales = np.empty((T, 3072), np.uint8), np.empty((T, 384), np.uint8)
    gs = np.empty(max(1, -(-T // 512)), np.float32)
    qscale = float(np.float32(1.0) / np.sqrt(np.float32(128.0)))
    eps = 1e-6

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

    def quantize(x, c, s, cols, lo, hi):
        # the NVFP4 activation encoder has no reference implementation: the restatement is timed
        L.quant_ws(at(x, lo), hi - lo, cols, 0, gs.ctypes.data_as(f32p), at(c, lo, u8p), at(s, lo, u8p))

    def gdn_layer(src, dst, lo, hi):
        n = hi - lo
        residual_norm(src, dst, lo, hi)
        quantize(nrm, codes, scales, H, lo, hi)
        hist = np.zeros((10240, 3), np.uint16)
        if lo >= 3:
            hist[:] = inp["raw"][lo - 3:lo].T
        if R is not None:
            for t in range(lo, hi):
                R.conv(at(inp["raw"], t), at(w["conv"], 0), at(hist, 0), at(conv_out, t))
        else:
            L.conv(at(inp["raw"], lo), n, 10240, at(w["conv"], 0), at(hist, 0), at(conv_out, lo))
        for off, sc in ((0, qscale), (2048, 1.0)):
            blk = np.ascontiguousarray(conv_out[lo:hi, off:off + 2048])
            L.l2(at(blk, 0), n * 16, 128, eps, sc, at(blk, 0))
            conv_out[lo:hi, off:off + 2048] = blk
        if R is not None:
            R.head_plain_gate(at(inp["core"], lo), at(w["gn"], 0), at(inp["z"], lo), n * 48, 128, eps, at(gdn_out, lo))
        else:
            L.headwise(at(inp["core"], lo), at(w["gn"], 0), at(inp["z"], lo), n * 48, 128, eps, 0, at(gdn_out, lo))
        quantize(gdn_out, gcodes, gscales, 6144, lo, hi)
        residual_norm(dst, src, lo, hi)
        quantize(nrm, codes, scales, H, lo, hi)
        (R.silu_mul if R is not None else L.silu_mul)(at(inp["gate"], lo), at(inp["up"], lo), n * I, at(mlp_out, lo))

    def fa_layer(src, dst, lo, hi):
        n = hi - lo
        residual_norm(src, dst, lo, hi)
        quantize(nrm, codes, scales, H, lo, hi)
        if R is not None:
            ref_preprocess(lo, hi)
        else:
            L.preprocess(at(inp["qg"], lo), at(inp["key"], lo), at(w["qn"], 0), at(w["kn"], 0), eps, at(q_out, lo),
                         at(gate_out, lo), cos.ctypes.data_as(f32p), sin.ctypes.data_as(f32p), lo, n)
        (R.sigmoid_gate if R is not None else L.sigmoid_gate)(at(inp["val"], lo), at(gate_out, lo), n * 6144,
                                                             at(attn_out, lo))
        residual_norm(dst, src, lo, hi)
        quantize(nrm, codes, scales, H, lo, hi)
        (R.silu_mul if R is not None else L.silu_mul)(at(inp["gate"], lo), at(inp["up"], lo), n * I, at(mlp_out, lo))

    def ref_preprocess(lo, hi):
        n = hi - lo
        for t in range(lo, hi):
            R.split(at(inp["qg"], t), 24, 256, at(q_out, t), at(gate_out, t))
        R.head_centered(at(q_out, lo), at(w["qn"], 0), n * 24, 256, eps, at(q_out, lo))
        R.head_centered(at(inp["key"], lo), at(w["kn"], 0), n * 4, 256, eps, at(inp["key"], lo))
        for t in range(lo, hi):
            c, s = C.cast(cos.ctypes.data + t * 128, f32p), C.cast(sin.ctypes.data + t * 128, f32p)
            R.rope(at(q_out, t), c, s, 24, at(q_out, t))
            R.rope(at(inp["key"], t), c, s, 4, at(inp["key"], t))

    def four_layers(lo, hi):
        gdn_layer(0, 1, lo, hi)
        gdn_layer(0, 1, lo, hi)
        gdn_layer(0, 1, lo, hi)
        fa_layer(0, 1, lo, hi)

    gs[:] = 0.0025
    table = bf((4096, H), 0.02)
    ids = rng.integers(0, 4096, size=T, dtype=np.uint32)
    emb = np.empty((T, H), np.uint16)

    def embed(lo, hi):
        if R is not None:
            for t in range(lo, hi):
                R.embedding(at(table, 0), 4096, H, int(ids[t]), at(emb, t))
        else:
            L.embedding(at(table, 0), 4096, H, C.cast(ids.ctypes.data + lo * 4, u32p), hi - lo, at(emb, lo))

    def run():
        t0 = time.perf_counter()
        orc.parallel_rows(four_layers, T, threads)
        t_layers = time.perf_counter() - t0
        t0 = time.perf_counter()
        orc.parallel_rows(embed, T, threads)
        return t_layers, time.perf_counter() - t0

    return run, kind


def cpu_tokens_per_second(sample_tokens: int, threads: int, repeats: int = 1):
    run, kind = cpu_chain_runner(sample_tokens, threads)
    best = None
    for _ in range(max(1, repeats)):
        t_layers, t_embed = run()
        total = t_layers * 16 + t_embed  # 4-layer pattern x 16 = 64 layers
        best = total if best is None else min(best, total)
    return sample_tokens / best, best, kind


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    times = []
    run, kind = cpu_chain_runner(args.cpu_sample_tokens, threads)
    for i in range(args.warmup + args.steps):
        t_layers, t_embed = run()
        if i >= args.warmup:
            times.append(t_layers * 16 + t_embed)
    per_step = sum(times) / len(times)
    value = args.cpu_sample_tokens / per_step
    sample = (f"{args.cpu_sample_tokens} tokens x the 4-layer pattern (GDN,GDN,GDN,FA) timed, x16 for 64 layers, "
              f"+ embedding gather; NVFP4 encoder from the C restatement")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 storage, fp32 arithmetic", "data": "synthetic",
        "config": workload_config(args.tokens, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def workload_config(tokens, gpus):
    return {
        "workload": ("configs[4] long-context shard: 131072-token prompt token-sharded 8-way = 16384 tokens per GPU"
                     if tokens == 16384 else f"{tokens}-token shard per GPU") +
                    ", embedding gather + 64 layers (48 GDN + 16 full-attention) of fused layer ops",
        "tokens_per_gpu": tokens, "total_tokens": tokens * gpus, "layers": 64, "hidden": 5120,
        "intermediate": 17408, "nvfp4_scale_scope_tokens": 512, "parallelism": f"token-row shards x{gpus}, no collective",
        "l2_policy": "every tensor is larger than L2 (>= 168 MB per operand at 16384 tokens); no flush",
    }


# ------------------------------------------------------------------------------------ GPU arm

def probe_ops(stack, chain, stream_obj, T, peak, warm, reps):
    """Times every fused operator alone with CUDA events on its own stream: microseconds per call,
    algorithmic GB/s and the fraction of the HBM peak."""
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
        # extra operator, not part of the step: SwiGLU with the NVFP4 operand of the down projection
        "swiglu_nvfp4": lambda: stack.op_swiglu_nvfp4(stream),
        "sigmoid_gate_nvfp4": lambda: stack.op_sigmoid_gate_nvfp4(stream),
    }
    per_op = {}
    with torch.cuda.stream(stream_obj):
        for name, fn in probes.items():
            for _ in range(warm):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream_obj)
            for _ in range(reps):
                fn()
            e1.record(stream_obj)
            stream_obj.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            base = name.split("/")[0]
            gbs = chain.BYTES_PER_TOKEN[base] * T / (us * 1e-6) / 1e9
            per_op[name] = {"us": round(us, 2), "algorithmic_GBs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4),
                            "bytes_per_token": chain.BYTES_PER_TOKEN[base], "kernels": chain.KERNELS[base]}
    return per_op


def decode_step_probe(chain, position=131071, reps=20):
    """The same 64-layer operator chain for ONE token at `position` (batch-one decode runs on one GPU):
    microseconds per step of a CUDA-graph replay.  Launch-latency bound, reported for completeness."""
    import torch

    stack = chain.LayerStack(1, first_position=position, seed=5, table_rows=8192)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        stack.enqueue_step(side.cuda_stream)
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        stack.enqueue_step(torch.cuda.current_stream().cuda_stream)
    with torch.cuda.stream(side):
        graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(side)
        for _ in range(reps):
            graph.replay()
        e1.record(side)
    side.synchronize()
    if int(stack.amax[-1].item()) != 0:
        raise SystemExit("a bounded device-side wait gave up during the decode probe")
    return {"tokens": 1, "position": position, "us_per_step": round(e0.elapsed_time(e1) * 1e3 / reps, 1),
            "kernels_per_step": chain.kernels_per_step()}


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist

    pkg = importlib.import_module("qwen3x-orin_b200")
    chain = importlib.import_module("qwen3x-orin_b200.chain")
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
        # NCCL only carries the barrier and the max-over-ranks of the timings; keep its banner
        # ("NCCL version ...") off stdout, which must hold exactly one JSON line
        os.environ["NCCL_DEBUG"] = os.environ.get("Q3X_NCCL_DEBUG", "WARN")
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)  # whatever the communicator set-up prints goes to stderr
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    T = args.tokens
    stack = chain.LayerStack(T, first_position=rank * T, seed=1234 + rank)
    stream_obj = torch.cuda.Stream()
    stream = stream_obj.cuda_stream

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    if args.probe_only:
        peak, _ = measured_peak()
        print(json.dumps({"probe_only": True, "tokens": T, "per_op": probe_ops(stack, chain, stream_obj, T, peak, 1, args.probe_reps)}),
              flush=True)
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

    with torch.cuda.stream(stream_obj):
        for _ in range(max(args.warmup, 3)):
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
    elapsed_ms = start.elapsed_time(stop)
    clocks = sampler.stop() if sampler else None
    # the single-kernel NVFP4 operators report a bounded wait that gave up in the last scratch word
    if int(stack.amax[-1].item()) != 0:
        raise SystemExit("a bounded device-side wait gave up during the timed steps: results invalid")
    t = torch.tensor([elapsed_ms], device="cuda", dtype=torch.float64)
    if distributed:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = T * world / (ms_per_step * 1e-3)

    # ---- per-operator timing (each op alone, CUDA events on its stream) --------------------------
    peak, peak_kind = measured_peak()
    per_op = probe_ops(stack, chain, stream_obj, T, peak, 3, 10) if rank == 0 else {}
    # dominant kernel = the SwiGLU stream (the largest share of the step's bytes, one kernel per launch)
    roofline = None
    if rank == 0:
        sw = per_op["swiglu"]
        roofline = {"bound": "hbm", "kernel": "binary_vec_kernel<SiluMul> (SwiGLU)", "achieved": sw["algorithmic_GBs"],
                    "peak": peak, "unit": "GB/s", "frac": round(sw["algorithmic_GBs"] / peak, 4), "peak_source": peak_kind,
                    "traffic": SWIGLU_DRAM_BYTES_PER_TOKEN * T, "traffic_source": SWIGLU_TRAFFIC_SOURCE,
                    "algorithmic_bytes_per_launch": chain.BYTES_PER_TOKEN["swiglu"] * T,
                    "us_per_launch": sw["us"]}
        step_bytes = chain.bytes_per_token_per_step() * T
        roofline["whole_step"] = {"algorithmic_GBs": round(step_bytes / (ms_per_step * 1e-3) / 1e9, 1),
                                  "frac": round(step_bytes / (ms_per_step * 1e-3) / 1e9 / peak, 4),
                                  "bytes_per_token": chain.bytes_per_token_per_step()}

    # ---- end to end: host buffers, H2D of the step's inputs and D2H of its result inside the timing --
    e2e = None
    if not args.no_e2e:
        # Two device input sets, each baked into its own graph: while step i computes on set i % 2,
        # the copy engine brings step i + 1's inputs from pinned host memory into the other set and
        # takes step i - 1's result back.  Every step's inputs and result cross PCIe inside the timing.
        names = list(stack.inputs)
        host_in = {n: torch.empty(stack.inputs[n].shape, dtype=torch.bfloat16, pin_memory=True) for n in names}
        for n in names:
            host_in[n].copy_(stack.inputs[n])
        host_ids = torch.empty(stack.token_ids.shape, dtype=torch.int32, pin_memory=True)
        host_ids.copy_(stack.token_ids)
        host_out = [torch.empty((T, 5120), dtype=torch.bfloat16, pin_memory=True) for _ in range(2)]
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

        def e2e_steps(count):
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

        e2e_steps(2)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(h2d_stream)
        e2e_steps(args.steps)
        d2h_stream.wait_stream(stream_obj)
        d2h_stream.wait_stream(h2d_stream)
        e1.record(d2h_stream)
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        if distributed:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / args.steps
        e2e = {"value": T * world / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms,
               "note": "per step: pinned-host inputs -> device, 64-layer chain, final residual -> pinned host; the "
                       "copies of neighbouring steps overlap the chain (two device input sets)"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        v, secs, kind = cpu_tokens_per_second(args.cpu_sample_tokens, threads)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": kind,
               "sample": f"{args.cpu_sample_tokens} tokens x 4-layer pattern timed, x16 for 64 layers, + embedding gather "
                         f"({secs:.2f} s extrapolated per pass)"}

    decode = decode_step_probe(chain) if rank == 0 else None
    validation = validate_shards(rank, world, dist) if distributed else None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 storage, fp32 arithmetic", "data": "synthetic", "config": workload_config(T, world),
            "roofline": roofline, "per_op": per_op, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": chain.kernels_per_step() * args.steps, "cuda_graph": graph is not None, "clocks": clocks,
        }
        line["decode_step"] = decode
        if validation is not None:
            line["validation"] = validation
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()
    return 0


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
