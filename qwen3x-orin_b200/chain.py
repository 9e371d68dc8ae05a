"""The per-layer operator chains of the 64-layer hybrid stack, driven through the C ABI.

A `LayerStack` owns the device buffers of one token shard and enqueues, layer by layer, exactly the
fused operators the reference runner calls between its projections
(src/runtime/reference_runner.cpp:9565-10584): the projections themselves are out of scope, so their
outputs are synthetic tensors that stay fixed while the residual stream, the key rows and the conv
histories evolve.  Layer l is a full-attention layer when (l + 1) % 4 == 0, else a gated-delta-net
layer (reference_runner.cpp:1463-1471).

Per layer:
  GDN : residual+RMSNorm+NVFP4 -> conv1d+SiLU+q/k L2 norm -> gated RMSNorm*silu(z)+NVFP4
        -> residual+RMSNorm+NVFP4 -> SwiGLU
  FA  : residual+RMSNorm+NVFP4 -> split+q/k head norm+RoPE -> sigmoid gate
        -> residual+RMSNorm+NVFP4 -> SwiGLU
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch

from . import capi

HIDDEN = 5120
INTERMEDIATE = 17408
VOCAB = 248320
LAYERS = 64
Q_HEADS, KV_HEADS, HEAD_DIM = 24, 4, 256
GDN_CHANNELS, GDN_V = 10240, 48 * 128
CHUNK = 512            # the reference's prefill chunk: the scope of one NVFP4 global scale
EPS = 1e-6
ROPE_THETA = 1e7

# Algorithmic HBM bytes per token of each fused operator: every input read once, every output
# written once, weights amortised.
BYTES_PER_TOKEN = {
    "embedding_gather": 2 * HIDDEN * 2 + 4,
    "residual_rmsnorm_nvfp4": 4 * HIDDEN * 2 + HIDDEN // 2 + HIDDEN // 16,
    "conv1d_silu_l2norm": 2 * GDN_CHANNELS * 2,
    "gated_rmsnorm_nvfp4": 3 * GDN_V * 2 + GDN_V // 2 + GDN_V // 16,
    "attention_preprocess": (2 * Q_HEADS + KV_HEADS) * HEAD_DIM * 2 + 256 + (2 * Q_HEADS + KV_HEADS) * HEAD_DIM * 2,
    "sigmoid_gate": 3 * Q_HEADS * HEAD_DIM * 2,
    "swiglu": 3 * INTERMEDIATE * 2,
    # not part of the step (the benchmark configurations quantise the norm outputs only): SwiGLU with
    # the NVFP4 operand of the down projection produced in the same kernel
    "swiglu_nvfp4": 3 * INTERMEDIATE * 2 + INTERMEDIATE // 2 + INTERMEDIATE // 16,
    # likewise: the sigmoid gate with the NVFP4 operand of the attention output projection
    "sigmoid_gate_nvfp4": 3 * Q_HEADS * HEAD_DIM * 2 + Q_HEADS * HEAD_DIM // 2 + Q_HEADS * HEAD_DIM // 16,
}
# kernels each entry point launches (memset nodes not counted); the norm + NVFP4 entries run their
# single-kernel form at the chain's scale scope of 512 tokens
KERNELS = {
    "embedding_gather": 1, "residual_rmsnorm_nvfp4": 1, "conv1d_silu_l2norm": 1, "gated_rmsnorm_nvfp4": 1,
    "attention_preprocess": 1, "sigmoid_gate": 1, "swiglu": 1, "swiglu_nvfp4": 1,
    "sigmoid_gate_nvfp4": 1,
}
GDN_OPS = ["residual_rmsnorm_nvfp4", "conv1d_silu_l2norm", "gated_rmsnorm_nvfp4", "residual_rmsnorm_nvfp4", "swiglu"]
FA_OPS = ["residual_rmsnorm_nvfp4", "attention_preprocess", "sigmoid_gate", "residual_rmsnorm_nvfp4", "swiglu"]


class profiler_range:
    """An NVTX range around a stretch of enqueued work (the reference brackets its runner phases the same way,
    src/runtime/reference_engine_control.cpp:38-89), so that a timeline capture of a step shows layers and
    operators by name.  Off unless Q3X_B200_NVTX=1: a push / pop pair costs more than a batch-one launch."""

    enabled = os.environ.get("Q3X_B200_NVTX", "0") not in ("", "0")

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if profiler_range.enabled:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if profiler_range.enabled:
            torch.cuda.nvtx.range_pop()
        return False


def is_full_attention(layer: int) -> bool:
    return (layer + 1) % 4 == 0


def layer_ops(layer: int):
    return FA_OPS if is_full_attention(layer) else GDN_OPS


def bytes_per_token_per_step(layers: int = LAYERS) -> int:
    total = BYTES_PER_TOKEN["embedding_gather"]
    for l in range(layers):
        total += sum(BYTES_PER_TOKEN[o] for o in layer_ops(l))
    return total


def kernels_per_step(layers: int = LAYERS) -> int:
    return KERNELS["embedding_gather"] + sum(KERNELS[o] for l in range(layers) for o in layer_ops(l))


def rope_tables(first_position: int, positions: int, device):
    """[positions, 32] cos / sin FP32 tables whose values went through bf16, the recipe of the
    reference's request state (src/runtime/request_state.cpp:2092-2108)."""
    pair = torch.arange(32, dtype=torch.float32)
    inv = 1.0 / torch.pow(torch.tensor(ROPE_THETA, dtype=torch.float32), 2.0 * pair / 64.0)
    pos = torch.arange(first_position, first_position + positions, dtype=torch.float32)[:, None]
    ang = pos * inv[None, :]
    cos = torch.cos(ang).to(torch.bfloat16).to(torch.float32)
    sin = torch.sin(ang).to(torch.bfloat16).to(torch.float32)
    return cos.to(device).contiguous(), sin.to(device).contiguous()


@dataclass
class ShardInputs:
    """Names of the synthetic per-shard inputs, their per-token widths (bf16 elements) and std."""
    names = ("proj_out", "conv_raw", "gdn_core", "gdn_z", "q_gate", "key", "attn_value", "mlp_gate", "mlp_up")
    widths = (HIDDEN, GDN_CHANNELS, GDN_V, GDN_V, 2 * Q_HEADS * HEAD_DIM, KV_HEADS * HEAD_DIM, Q_HEADS * HEAD_DIM,
              INTERMEDIATE, INTERMEDIATE)


class LayerStack:
    """Device state of one token shard: synthetic projection outputs, weights, evolving tensors."""

    def __init__(self, tokens: int, first_position: int = 0, seed: int = 0, device="cuda", layers: int = LAYERS,
                 table_rows: int = VOCAB):
        self.tokens, self.layers, self.first_position = tokens, layers, first_position
        dev = torch.device(device)
        gen = torch.Generator(device=dev).manual_seed(seed)

        def normal(shape, std=1.0):
            return (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std).to(torch.bfloat16)

        T = tokens
        # input sets: the step reads the active one; a second set lets the next step's host->device
        # copies overlap the current step (each set is baked into its own CUDA graph)
        self.input_sets = [{n: normal((T, w)) for n, w in zip(ShardInputs.names, ShardInputs.widths)}]
        self.active = 0
        self.table = normal((table_rows, HIDDEN), 0.02)
        self.id_sets = [torch.randint(0, table_rows, (T,), generator=gen, device=dev, dtype=torch.int64).to(torch.int32)]
        # weights: distinct per layer, all tiny
        self.norm_w = normal((layers, 2, HIDDEN), 0.02)
        self.q_norm_w = normal((layers, HEAD_DIM), 0.02)
        self.k_norm_w = normal((layers, HEAD_DIM), 0.02)
        self.gdn_norm_w = (1.0 + normal((layers, 128), 0.1).float()).to(torch.bfloat16)
        self.conv_w = normal((layers, GDN_CHANNELS, 4), 0.5)
        self.conv_hist = torch.zeros((layers, GDN_CHANNELS, 3), device=dev, dtype=torch.bfloat16)
        self.cos, self.sin = rope_tables(0, first_position + T, dev)
        # evolving / output tensors
        bf = dict(device=dev, dtype=torch.bfloat16)
        self.residual = [torch.empty((T, HIDDEN), **bf) for _ in range(2)]
        self.normalized = torch.empty((T, HIDDEN), **bf)
        self.conv_out = torch.empty((T, GDN_CHANNELS), **bf)
        self.gdn_out = torch.empty((T, GDN_V), **bf)
        self.q_out = torch.empty((T, Q_HEADS * HEAD_DIM), **bf)
        self.gate_out = torch.empty((T, Q_HEADS * HEAD_DIM), **bf)
        self.attn_out = torch.empty((T, Q_HEADS * HEAD_DIM), **bf)
        self.mlp_out = torch.empty((T, INTERMEDIATE), **bf)
        groups = max(1, math.ceil(T / CHUNK))
        self.groups = groups
        # NVFP4 scratch: zeroed once here, left zero by every call; the last word is the sticky error flag
        self.amax = torch.zeros(capi.lib().q3x_b200_nvfp4_scratch_words(T, CHUNK), device=dev, dtype=torch.int32)
        self.global_scales = torch.empty(groups, device=dev, dtype=torch.float32)
        self.codes = torch.empty((T, HIDDEN // 2), device=dev, dtype=torch.uint8)
        self.scales = torch.empty((T, HIDDEN // 16), device=dev, dtype=torch.uint8)
        self.gdn_codes = torch.empty((T, GDN_V // 2), device=dev, dtype=torch.uint8)
        self.gdn_scales = torch.empty((T, GDN_V // 16), device=dev, dtype=torch.uint8)
        self.q_scale = 1.0 / math.sqrt(128.0)

    @property
    def inputs(self):
        return self.input_sets[self.active]

    @property
    def token_ids(self):
        return self.id_sets[self.active]

    def add_input_set(self) -> int:
        """Clones input set 0 into a new device-resident set and returns its index."""
        self.input_sets.append({n: t.clone() for n, t in self.input_sets[0].items()})
        self.id_sets.append(self.id_sets[0].clone())
        return len(self.input_sets) - 1

    def check_error(self, what: str = "the operator chain") -> None:
        """Synchronises and raises when a bounded device-side wait of a single-kernel NVFP4 operator gave up
        at any point since the scratch was allocated (the flag is sticky), or when a call left scratch words
        behind; the outputs are not valid then."""
        words = self.amax.cpu()
        if int(words[-1]) != 0:
            raise RuntimeError(f"{what}: a bounded device-side wait gave up (error word {int(words[-1]):#x})")
        if bool(words[:-1].any()):
            raise RuntimeError(f"{what}: NVFP4 scratch words were left non-zero")

    # ---- individual operators (each is one C-ABI call) ------------------------------------
    def op_embedding(self, stream):
        capi.check("q3x_b200_embedding_gather", self.table, self.table.shape[0], HIDDEN, self.token_ids, self.tokens,
                   self.residual[0], stream)

    def op_residual_norm(self, layer, which, src, dst, stream):
        capi.check("q3x_b200_residual_add_rms_norm_nvfp4", self.residual[src], self.inputs["proj_out"],
                   self.norm_w[layer, which], self.tokens, HIDDEN, EPS, CHUNK, self.residual[dst], self.normalized,
                   self.amax, self.global_scales, self.codes, self.scales, stream)

    def op_conv(self, layer, stream):
        capi.check("q3x_b200_causal_conv1d_silu_l2norm", self.inputs["conv_raw"], self.tokens, self.conv_w[layer],
                   self.conv_hist[layer], EPS, self.q_scale, self.conv_out, stream)

    def op_gated_norm(self, layer, stream):
        capi.check("q3x_b200_rms_norm_silu_gate_nvfp4", self.inputs["gdn_core"], self.gdn_norm_w[layer],
                   self.inputs["gdn_z"], self.tokens, 48, 128, EPS, CHUNK, self.gdn_out, self.amax,
                   self.global_scales, self.gdn_codes, self.gdn_scales, stream)

    def op_preprocess(self, layer, stream):
        capi.check("q3x_b200_full_attention_preprocess", self.inputs["q_gate"], self.inputs["key"], self.q_norm_w[layer],
                   self.k_norm_w[layer], EPS, self.q_out, self.gate_out, self.cos, self.sin, self.first_position,
                   self.tokens, stream)

    def op_sigmoid_gate(self, stream):
        capi.check("q3x_b200_sigmoid_gate", self.inputs["attn_value"], self.gate_out, self.tokens * Q_HEADS * HEAD_DIM,
                   self.attn_out, stream)

    def op_swiglu(self, stream):
        capi.check("q3x_b200_silu_mul", self.inputs["mlp_gate"], self.inputs["mlp_up"], self.tokens * INTERMEDIATE,
                   self.mlp_out, stream)

    def op_swiglu_nvfp4(self, stream):
        """SwiGLU + NVFP4 of its output (extra operator, not in the step); allocates its code buffers once."""
        if not hasattr(self, "mlp_codes"):
            dev = self.mlp_out.device
            self.mlp_codes = torch.empty((self.tokens, INTERMEDIATE // 2), device=dev, dtype=torch.uint8)
            self.mlp_scales = torch.empty((self.tokens, INTERMEDIATE // 16), device=dev, dtype=torch.uint8)
        capi.check("q3x_b200_silu_mul_nvfp4", self.inputs["mlp_gate"], self.inputs["mlp_up"], self.tokens, INTERMEDIATE,
                   CHUNK, self.mlp_out, self.amax, self.global_scales, self.mlp_codes, self.mlp_scales, stream)

    def op_sigmoid_gate_nvfp4(self, stream):
        """Sigmoid gate + NVFP4 of its output (extra operator, not in the step); reuses the GDN code buffers,
        which have the same [tokens, 6144] geometry."""
        capi.check("q3x_b200_sigmoid_gate_nvfp4", self.inputs["attn_value"], self.gate_out, self.tokens,
                   Q_HEADS * HEAD_DIM, CHUNK, self.attn_out, self.amax, self.global_scales, self.gdn_codes,
                   self.gdn_scales, stream)

    def enqueue_step_branched(self, main, side_a, side_b) -> int:
        """The same step with the operators that do not depend on one another placed on three streams
        (torch.cuda.Stream objects): the residual stream's chain of residual + norm + NVFP4 operators stays on
        `main` (it is the only true dependency chain between the operators of this path: every other operator
        reads projection outputs), the mixer operators of a layer (conv + gated norm, or pre-processing + sigmoid
        gate) go to `side_a` and SwiGLU to `side_b`.  Captured into a CUDA graph this gives three parallel
        branches, which is what a batch-one (launch-latency-bound) step wants; the two norm operators of a layer
        do not share their NVFP4 scratch with the side branches (those get scratch of their own).  Returns the
        index of the residual buffer that holds the final residual stream."""
        import torch

        if not hasattr(self, "amax_side"):
            self.amax_side = torch.zeros_like(self.amax)
            self.global_scales_side = torch.empty_like(self.global_scales)
        fork = torch.cuda.Event()
        fork.record(main)
        side_a.wait_event(fork)
        side_b.wait_event(fork)
        m, a, b = main.cuda_stream, side_a.cuda_stream, side_b.cuda_stream
        self.op_embedding(m)
        cur = 0
        for layer in range(self.layers):
            self.op_residual_norm(layer, 0, cur, 1 - cur, m)
            cur = 1 - cur
            if is_full_attention(layer):
                self.op_preprocess(layer, a)
                self.op_sigmoid_gate(a)
            else:
                self.op_conv(layer, a)
                capi.check("q3x_b200_rms_norm_silu_gate_nvfp4", self.inputs["gdn_core"], self.gdn_norm_w[layer],
                           self.inputs["gdn_z"], self.tokens, 48, 128, EPS, CHUNK, self.gdn_out, self.amax_side,
                           self.global_scales_side, self.gdn_codes, self.gdn_scales, a)
            self.op_residual_norm(layer, 1, cur, 1 - cur, m)
            cur = 1 - cur
            self.op_swiglu(b)
        join_a, join_b = torch.cuda.Event(), torch.cuda.Event()
        join_a.record(side_a)
        join_b.record(side_b)
        main.wait_event(join_a)
        main.wait_event(join_b)
        return cur

    # ---- the whole step ------------------------------------------------------------------------
    def enqueue_step(self, stream) -> int:
        """Embedding gather + every layer's chain on `stream` (a raw cudaStream_t).  Returns the
        index of the residual buffer that holds the final residual stream."""
        # (the key rows are normalised and rotated in place by every full-attention layer, as the
        # reference does inside its KV cache; they stay bounded, so no reset is needed per step)
        with profiler_range("embedding"):
            self.op_embedding(stream)
        cur = 0
        for layer in range(self.layers):
            with profiler_range(f"layer {layer} {'full-attention' if is_full_attention(layer) else 'gdn'}"):
                with profiler_range("input residual+norm+nvfp4"):
                    self.op_residual_norm(layer, 0, cur, 1 - cur, stream)
                cur = 1 - cur
                with profiler_range("mixer operators"):
                    if is_full_attention(layer):
                        self.op_preprocess(layer, stream)
                        self.op_sigmoid_gate(stream)
                    else:
                        self.op_conv(layer, stream)
                        self.op_gated_norm(layer, stream)
                with profiler_range("post-attention residual+norm+nvfp4"):
                    self.op_residual_norm(layer, 1, cur, 1 - cur, stream)
                cur = 1 - cur
                with profiler_range("swiglu"):
                    self.op_swiglu(stream)
        return cur


class ProjectedMlp:
    """One layer's MLP block WITH its projections, every operand of every projection in NVFP4:

        residual + RMSNorm + NVFP4  ->  gate, up = x W_gate^T, x W_up^T  (block-scaled tensor cores)
        ->  SwiGLU + NVFP4  ->  down = h W_down^T  ->  (the next residual + RMSNorm takes `down` as its right operand)

    which is the reference's post-attention composite followed by its MLP-down composite
    (launch_post_attention_residual_norm_mlp_gate_up_silu_to_bf16_cuda, launch_mlp_down_residual_norm_to_bf16_cuda,
    include/q3x/runtime/model_weights.h:928-992) for a panel of tokens.  The weights are synthetic: random bf16
    matrices quantised row-wise by the library's own quantiser (one second-level scale per matrix)."""

    def __init__(self, tokens: int, device, hidden: int = HIDDEN, intermediate: int = INTERMEDIATE, seed: int = 11):
        self.tokens, self.hidden, self.intermediate = tokens, hidden, intermediate
        self.device = device
        gen = torch.Generator(device=device).manual_seed(seed)
        L = capi.lib()
        u8 = dict(device=device, dtype=torch.uint8)
        bf = dict(device=device, dtype=torch.bfloat16)

        def weight(rows, cols):
            dense = (torch.randn((rows, cols), generator=gen, device=device) * 0.03).to(torch.bfloat16)
            codes, scales = torch.empty((rows, cols // 2), **u8), torch.empty((rows, cols // 16), **u8)
            gs = torch.empty(1, device=device, dtype=torch.float32)
            scratch = torch.zeros(L.q3x_b200_nvfp4_scratch_words(rows, 0), device=device, dtype=torch.int32)
            capi.check("q3x_b200_nvfp4_quantize_dynamic", dense, rows, cols, 0, scratch, gs, codes, scales, None)
            swizzled = torch.empty(L.q3x_b200_nvfp4_swizzled_scale_bytes(rows, cols), **u8)
            capi.check("q3x_b200_nvfp4_swizzle_block_scales", scales, rows, cols, swizzled, None)
            torch.cuda.synchronize(device)
            return {"codes": codes, "scales": scales, "swizzled": swizzled, "scale_2": float(gs.item()), "dense": dense}

        self.w_gate, self.w_up = weight(intermediate, hidden), weight(intermediate, hidden)
        self.w_down = weight(hidden, intermediate)
        self.norm_w = (torch.randn(hidden, generator=gen, device=device) * 0.02).to(torch.bfloat16)
        self.left = torch.randn((tokens, hidden), generator=gen, device=device).to(torch.bfloat16)
        self.right = torch.randn((tokens, hidden), generator=gen, device=device).to(torch.bfloat16)
        groups = (tokens + CHUNK - 1) // CHUNK
        self.residual, self.normalized = torch.empty((tokens, hidden), **bf), torch.empty((tokens, hidden), **bf)
        self.scratch = torch.zeros(L.q3x_b200_nvfp4_scratch_words(tokens, CHUNK), device=device, dtype=torch.int32)
        self.x_gs = torch.empty(groups, device=device, dtype=torch.float32)
        self.x_codes, self.x_scales = torch.empty((tokens, hidden // 2), **u8), torch.empty((tokens, hidden // 16), **u8)
        self.x_swizzled = torch.empty(L.q3x_b200_nvfp4_swizzled_scale_bytes(tokens, hidden), **u8)
        self.gate, self.up = torch.empty((tokens, intermediate), **bf), torch.empty((tokens, intermediate), **bf)
        self.h = torch.empty((tokens, intermediate), **bf)
        self.h_gs = torch.empty(groups, device=device, dtype=torch.float32)
        self.h_codes = torch.empty((tokens, intermediate // 2), **u8)
        self.h_scales = torch.empty((tokens, intermediate // 16), **u8)
        self.h_swizzled = torch.empty(L.q3x_b200_nvfp4_swizzled_scale_bytes(tokens, intermediate), **u8)
        self.down = torch.empty((tokens, hidden), **bf)
        need = max(L.q3x_b200_nvfp4_gemm_workspace_bytes(tokens, intermediate, hidden, CHUNK),
                   L.q3x_b200_nvfp4_gemm_workspace_bytes(tokens, hidden, intermediate, CHUNK))
        self.workspace = torch.empty(need, **u8)

    def flops(self) -> float:
        return 2.0 * self.tokens * self.hidden * self.intermediate * 3

    def _project(self, codes, swizzled, gs, weight, out_features, in_features, out, stream):
        capi.check("q3x_b200_nvfp4_gemm_bf16", codes, swizzled, gs, CHUNK, weight["codes"], weight["swizzled"],
                   weight["scale_2"], self.tokens, out_features, in_features, out, self.workspace, self.workspace.numel(),
                   stream)

    def enqueue(self, stream) -> None:
        T, H, I = self.tokens, self.hidden, self.intermediate
        capi.check("q3x_b200_residual_add_rms_norm_nvfp4", self.left, self.right, self.norm_w, T, H, EPS, CHUNK,
                   self.residual, self.normalized, self.scratch, self.x_gs, self.x_codes, self.x_scales, stream)
        capi.check("q3x_b200_nvfp4_swizzle_block_scales", self.x_scales, T, H, self.x_swizzled, stream)
        self._project(self.x_codes, self.x_swizzled, self.x_gs, self.w_gate, I, H, self.gate, stream)
        self._project(self.x_codes, self.x_swizzled, self.x_gs, self.w_up, I, H, self.up, stream)
        capi.check("q3x_b200_silu_mul_nvfp4", self.gate, self.up, T, I, CHUNK, self.h, self.scratch, self.h_gs,
                   self.h_codes, self.h_scales, stream)
        capi.check("q3x_b200_nvfp4_swizzle_block_scales", self.h_scales, T, I, self.h_swizzled, stream)
        self._project(self.h_codes, self.h_swizzled, self.h_gs, self.w_down, H, I, self.down, stream)

    def check_error(self) -> None:
        if int(self.scratch[-1].item()) != 0:
            raise RuntimeError("a bounded wait of a single-kernel NVFP4 operator gave up: outputs are invalid")


WIDEN_FP8_FROM_TOKENS = 128


def fp8_projection(weight: dict, x, tokens: int, out, stream) -> None:
    """out = bf16((x @ decode(codes).T) * scale) for an FP8 (E4M3, per-tensor scale) weight.  Panels of 128 tokens or
    more run on the dense tensor-core path against a bf16 copy of the weight, made once on first use (E4M3 -> bf16 is
    exact, so products, FP32 accumulation and output bytes are those of the mixed-input kernel, at 1.5 times its
    speed for twice the weight memory); shorter tiles, which are bound by reading the weight, keep the FP8 bytes."""
    if tokens >= WIDEN_FP8_FROM_TOKENS and weight["rows"] % 8 == 0 and weight["cols"] % 16 == 0:
        if "wide" not in weight:
            weight["wide"] = torch.empty((weight["rows"], weight["cols"]), device=weight["codes"].device, dtype=torch.bfloat16)
            capi.check("q3x_b200_fp8_weights_to_bf16", weight["codes"], weight["rows"] * weight["cols"], weight["wide"], None)
            torch.cuda.synchronize(weight["codes"].device)
        capi.check("q3x_b200_bf16_gemm_scaled_bf16", weight["wide"], weight["scale"], x, tokens, weight["rows"], weight["cols"],
                   out, None, 0, stream)
    else:
        capi.check("q3x_b200_fp8_gemm_bf16", weight["codes"], weight["scale"], x, tokens, weight["rows"], weight["cols"],
                   out, None, 0, stream)


class ProjectedAttentionLayer:
    """One full-attention layer of the stack for a tile of tokens appended at `first_position`, every operator and
    every projection from this library (the call order of the reference's layer segment,
    src/runtime/reference_runner.cpp:9565-10584):

        residual + RMSNorm  ->  q|gate, k, v projections (FP8 weights, bf16 activations, tensor cores; k and v land
        in the KV caches)  ->  q / k head norm + partial RoPE (keys in place, in the cache)  ->  bulk causal attention
        + sigmoid gate  ->  output projection (FP8)  ->  the MLP block (ProjectedMlp: residual + RMSNorm + NVFP4,
        gate / up, SwiGLU + NVFP4, down)

    Weights are synthetic (random E4M3 bytes with a per-tensor scale; the MLP's as in ProjectedMlp); cache positions
    before the tile hold random keys and values."""

    def __init__(self, tokens: int, first_position: int, device, intermediate: int = INTERMEDIATE, seed: int = 21):
        self.tokens, self.first_position, self.device = tokens, first_position, device
        gen = torch.Generator(device=device).manual_seed(seed)
        bf = dict(device=device, dtype=torch.bfloat16)
        q_dim, kv_dim = 2 * Q_HEADS * HEAD_DIM, KV_HEADS * HEAD_DIM

        def fp8_weight(rows, cols, scale):
            codes = torch.randint(0x08, 0x70, (rows, cols), generator=gen, device=device, dtype=torch.int32)
            signs = torch.randint(0, 2, (rows, cols), generator=gen, device=device, dtype=torch.int32) << 7
            return {"codes": (codes | signs).to(torch.uint8), "scale": scale, "rows": rows, "cols": cols}

        # scales chosen so that the projections of a unit-variance input have roughly unit variance
        self.w_q = fp8_weight(q_dim, HIDDEN, 0.0016)
        self.w_k = fp8_weight(kv_dim, HIDDEN, 0.0016)
        self.w_v = fp8_weight(kv_dim, HIDDEN, 0.0016)
        self.w_o = fp8_weight(HIDDEN, Q_HEADS * HEAD_DIM, 0.0015)
        rand = lambda shape, std=1.0: (torch.randn(shape, generator=gen, device=device) * std).to(torch.bfloat16)
        self.input_norm_w, self.q_norm_w, self.k_norm_w = rand((HIDDEN,), 0.02), rand((HEAD_DIM,), 0.02), rand((HEAD_DIM,), 0.02)
        self.residual_in, self.previous_mlp_out = rand((tokens, HIDDEN)), rand((tokens, HIDDEN))
        length = first_position + tokens
        self.key_cache, self.value_cache = rand((length, KV_HEADS, HEAD_DIM)), rand((length, KV_HEADS, HEAD_DIM))
        self.cos, self.sin = rope_tables(0, length, device)
        self.residual_mid = torch.empty((tokens, HIDDEN), **bf)
        self.normalized = torch.empty((tokens, HIDDEN), **bf)
        self.q_gate = torch.empty((tokens, q_dim), **bf)
        self.q_out = torch.empty((tokens, Q_HEADS, HEAD_DIM), **bf)
        self.gate_out = torch.empty((tokens, Q_HEADS, HEAD_DIM), **bf)
        self.attention = torch.empty((tokens, Q_HEADS, HEAD_DIM), **bf)
        self.attention_projected = torch.empty((tokens, HIDDEN), **bf)
        # the MLP block takes (residual_mid, attention_projected) as its (left, right)
        self.mlp = ProjectedMlp(tokens, device, intermediate=intermediate, seed=seed + 1)
        self.mlp.left, self.mlp.right = self.residual_mid, self.attention_projected

    def _tile(self, cache):
        return cache[self.first_position:]  # the tile's own rows of a cache: [tokens, 4, 256], contiguous

    def _fp8(self, weight, x, out, stream):
        fp8_projection(weight, x, self.tokens, out, stream)

    def enqueue(self, stream) -> None:
        T = self.tokens
        capi.check("q3x_b200_residual_add_rms_norm", self.residual_in, self.previous_mlp_out, self.input_norm_w, T, HIDDEN,
                   EPS, self.residual_mid, self.normalized, stream)
        self._fp8(self.w_q, self.normalized, self.q_gate, stream)
        self._fp8(self.w_k, self.normalized, self._tile(self.key_cache), stream)
        self._fp8(self.w_v, self.normalized, self._tile(self.value_cache), stream)
        capi.check("q3x_b200_full_attention_preprocess", self.q_gate, self._tile(self.key_cache), self.q_norm_w,
                   self.k_norm_w, EPS, self.q_out, self.gate_out, self.cos, self.sin, self.first_position, T, stream)
        capi.check("q3x_b200_gqa_attention_prefill_sigmoid_gate", self.q_out, self.key_cache, self.value_cache,
                   self.gate_out, self.first_position, T, 1.0 / math.sqrt(HEAD_DIM), self.attention, stream)
        self._fp8(self.w_o, self.attention, self.attention_projected, stream)
        self.mlp.enqueue(stream)

    def flops(self) -> float:
        T, first = self.tokens, self.first_position
        projections = 2.0 * T * HIDDEN * (2 * Q_HEADS * HEAD_DIM + 2 * KV_HEADS * HEAD_DIM + Q_HEADS * HEAD_DIM)
        pairs = T * first + T * (T + 1) // 2
        return projections + 4.0 * pairs * Q_HEADS * HEAD_DIM + self.mlp.flops()


class ProjectedGdnLayer:
    """One gated-delta-net layer of the stack for a tile of tokens, every operator and every projection from this
    library (the reference's layer segment, src/runtime/reference_runner.cpp:9565-10584):

        residual + RMSNorm  ->  qkv and z projections (FP8 weights, bf16 activations, tensor cores) and the two gate
        projections a, b (bf16 weights, 48 x 5120)  ->  causal
        conv1d + SiLU (history carried)  ->  gated-delta-net recurrence (state carried; token by token inside one
        launch, or with ``chunked`` in 64-token chunks on the tensor cores, the reference's production prefill form,
        src/kernels/sm87/gdn_prefill_chunk64_native_sm87.h:96-109)  ->  gated RMSNorm * silu(z) + NVFP4  ->  output
        projection (NVFP4 x NVFP4)  ->  the MLP block

    Weights are synthetic."""

    def __init__(self, tokens: int, device, intermediate: int = INTERMEDIATE, seed: int = 31, chunked: bool = False):
        self.tokens, self.device, self.chunked = tokens, device, chunked
        gen = torch.Generator(device=device).manual_seed(seed)
        L = capi.lib()
        bf = dict(device=device, dtype=torch.bfloat16)
        u8 = dict(device=device, dtype=torch.uint8)
        rand = lambda shape, std=1.0: (torch.randn(shape, generator=gen, device=device) * std).to(torch.bfloat16)

        def fp8_weight(rows, cols, scale):
            codes = torch.randint(0x08, 0x70, (rows, cols), generator=gen, device=device, dtype=torch.int32)
            signs = torch.randint(0, 2, (rows, cols), generator=gen, device=device, dtype=torch.int32) << 7
            return {"codes": (codes | signs).to(torch.uint8), "scale": scale, "rows": rows, "cols": cols}

        self.w_qkv = fp8_weight(GDN_CHANNELS, HIDDEN, 0.0003)
        self.w_z = fp8_weight(GDN_V, HIDDEN, 0.0003)
        dense = rand((HIDDEN, GDN_V), 0.03)  # output projection, quantised row-wise by the library's own quantiser
        self.w_o = {"codes": torch.empty((HIDDEN, GDN_V // 2), **u8), "scales": torch.empty((HIDDEN, GDN_V // 16), **u8)}
        gs = torch.empty(1, device=device, dtype=torch.float32)
        scratch = torch.zeros(L.q3x_b200_nvfp4_scratch_words(HIDDEN, 0), device=device, dtype=torch.int32)
        capi.check("q3x_b200_nvfp4_quantize_dynamic", dense, HIDDEN, GDN_V, 0, scratch, gs, self.w_o["codes"], self.w_o["scales"],
                   None)
        self.w_o["swizzled"] = torch.empty(L.q3x_b200_nvfp4_swizzled_scale_bytes(HIDDEN, GDN_V), **u8)
        capi.check("q3x_b200_nvfp4_swizzle_block_scales", self.w_o["scales"], HIDDEN, GDN_V, self.w_o["swizzled"], None)
        torch.cuda.synchronize(device)
        self.w_o["scale_2"] = float(gs.item())
        self.input_norm_w, self.gdn_norm_w = rand((HIDDEN,), 0.02), (0.75 + 0.5 * torch.rand(128, generator=gen, device=device)).to(torch.bfloat16)
        self.conv_w = rand((GDN_CHANNELS, 4), 0.5)
        self.conv_history = torch.zeros((GDN_CHANNELS, 3), **bf)
        self.A_log = (torch.rand(48, generator=gen, device=device) * 5.5 - 4.0).to(torch.bfloat16)
        self.dt_bias = (torch.rand(48, generator=gen, device=device) * 6.0 - 3.0).to(torch.bfloat16)
        self.w_a, self.w_b = rand((48, HIDDEN), 0.03), rand((48, HIDDEN), 0.03)
        self.a, self.b = torch.empty((tokens, 48), **bf), torch.empty((tokens, 48), **bf)
        self.state = rand((48, 128, 128), 0.05)
        self.residual_in, self.previous_mlp_out = rand((tokens, HIDDEN)), rand((tokens, HIDDEN))
        self.residual_mid, self.normalized = torch.empty((tokens, HIDDEN), **bf), torch.empty((tokens, HIDDEN), **bf)
        self.qkv, self.conv_out = torch.empty((tokens, GDN_CHANNELS), **bf), torch.empty((tokens, GDN_CHANNELS), **bf)
        self.z, self.core = torch.empty((tokens, GDN_V), **bf), torch.empty((tokens, GDN_V), **bf)
        self.gated = torch.empty((tokens, GDN_V), **bf)
        groups = (tokens + CHUNK - 1) // CHUNK
        self.scratch = torch.zeros(L.q3x_b200_nvfp4_scratch_words(tokens, CHUNK), device=device, dtype=torch.int32)
        self.gated_gs = torch.empty(groups, device=device, dtype=torch.float32)
        self.gated_codes, self.gated_scales = torch.empty((tokens, GDN_V // 2), **u8), torch.empty((tokens, GDN_V // 16), **u8)
        self.gated_swizzled = torch.empty(L.q3x_b200_nvfp4_swizzled_scale_bytes(tokens, GDN_V), **u8)
        self.mixer_projected = torch.empty((tokens, HIDDEN), **bf)
        self.workspace = torch.empty(L.q3x_b200_nvfp4_gemm_workspace_bytes(tokens, HIDDEN, GDN_V, CHUNK), **u8)
        self.recurrence_workspace = torch.empty(L.q3x_b200_gated_delta_net_chunked_workspace_bytes(tokens) if chunked else 0, **u8)
        self.mlp = ProjectedMlp(tokens, device, intermediate=intermediate, seed=seed + 1)
        self.mlp.left, self.mlp.right = self.residual_mid, self.mixer_projected

    def _fp8(self, weight, x, out, stream):
        fp8_projection(weight, x, self.tokens, out, stream)

    def enqueue(self, stream) -> None:
        T = self.tokens
        capi.check("q3x_b200_residual_add_rms_norm", self.residual_in, self.previous_mlp_out, self.input_norm_w, T, HIDDEN,
                   EPS, self.residual_mid, self.normalized, stream)
        self._fp8(self.w_qkv, self.normalized, self.qkv, stream)
        self._fp8(self.w_z, self.normalized, self.z, stream)
        capi.check("q3x_b200_bf16_gemm_bf16", self.w_a, self.normalized, T, 48, HIDDEN, self.a, None, 0, stream)
        capi.check("q3x_b200_bf16_gemm_bf16", self.w_b, self.normalized, T, 48, HIDDEN, self.b, None, 0, stream)
        capi.check("q3x_b200_causal_conv1d_silu", self.qkv, T, GDN_CHANNELS, self.conv_w, self.conv_history, self.conv_out, stream)
        if self.chunked:
            capi.check("q3x_b200_gated_delta_net_update_chunked", self.conv_out, T, self.a, self.b, self.A_log, self.dt_bias,
                       self.state, self.state, EPS, self.core, self.recurrence_workspace, self.recurrence_workspace.numel(), stream)
        else:
            capi.check("q3x_b200_gated_delta_net_update", self.conv_out, T, self.a, self.b, self.A_log, self.dt_bias, self.state,
                       self.state, EPS, self.core, stream)
        capi.check("q3x_b200_rms_norm_silu_gate_nvfp4", self.core, self.gdn_norm_w, self.z, T, 48, 128, EPS, CHUNK, self.gated,
                   self.scratch, self.gated_gs, self.gated_codes, self.gated_scales, stream)
        capi.check("q3x_b200_nvfp4_swizzle_block_scales", self.gated_scales, T, GDN_V, self.gated_swizzled, stream)
        capi.check("q3x_b200_nvfp4_gemm_bf16", self.gated_codes, self.gated_swizzled, self.gated_gs, CHUNK, self.w_o["codes"],
                   self.w_o["swizzled"], self.w_o["scale_2"], T, HIDDEN, GDN_V, self.mixer_projected, self.workspace,
                   self.workspace.numel(), stream)
        self.mlp.enqueue(stream)

    def check_error(self) -> None:
        if int(self.scratch[-1].item()) != 0:
            raise RuntimeError("a bounded wait of a single-kernel NVFP4 operator gave up: outputs are invalid")
        self.mlp.check_error()
