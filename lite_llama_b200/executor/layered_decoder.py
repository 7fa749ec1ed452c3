"""Decoder for layer-list models: each layer = one mixer (looked up in ``MIXERS`` by the layer's kind) + an optional
feed-forward (``FEED_FORWARDS``), around an fp32 residual stream with the norm on the sublayer OUTPUT:

    x <- x + norm(mixer(x));   x <- x + norm(ff(x))          (the sublayers read x itself)

The forward is a flat op list over the library's kernels, like ``executor.decoder.Decoder`` is for the uniform
rotary decoders (reference: lite_llama/models/base.py:299-319,447-489), but over a RAGGED step (``RaggedBatch``):
prompt portions and single decode tokens of different requests in one flat ``[tokens, hidden]`` batch.  Projections
run in the activation dtype (bf16 / fp16 on tcgen05, or TRUE fp32 on the CUDA cores); norms, softmax, the residual
sum, decays, step sizes and the recurrent state are fp32 in every mode.

Designs registered here:
  * ``Gufotar``: learned absolute positions, Mamba-2 style state-space layers and position-free attention layers
    (whole-row q/k norm, log-position query gain, tanh soft cap, per-head softmax sink, cross-layer value mixing),
    squared-ReLU feed-forward, zero-centred norm weights.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..kernels import (
    attn_prepare,
    causal_conv_silu,
    embed_positions,
    gated_group_norm,
    linear,
    post_norm_residual,
    relu_squared,
    rmsnorm_from_f32,
    sink_attention,
    ssm_scan,
)
from .model_config import DenseMlpSpec, LayeredConfig, LayerSpec, Mamba2Spec, SinkAttentionSpec
from .ragged_batch import RaggedBatch
from .registry import Architecture, register


# ------------------------------------------------------------------------------------------------------ weights #
@dataclass
class LayeredLayerWeights:
    norm1: torch.Tensor
    mix: dict[str, torch.Tensor]
    norm2: torch.Tensor | None = None
    mlp: dict[str, torch.Tensor] | None = None


@dataclass
class LayeredWeights:
    embed: torch.Tensor
    pos: torch.Tensor | None
    final_norm: torch.Tensor
    head: torch.Tensor
    layers: list[LayeredLayerWeights] = field(default_factory=list)

    def nbytes_per_step(self) -> int:
        """Weight bytes one step streams (embedding / position gathers excluded)."""
        total = self.head.numel() * self.head.element_size()
        for lw in self.layers:
            for d in (lw.mix, lw.mlp or {}):
                total += sum(t.numel() * t.element_size() for t in d.values())
        return total


# ------------------------------------------------------------------------------------------------------- mixers #
class StepContext:
    """What the mixers of one forward share: the step's metadata, the caches, and values one layer hands to later
    ones (the first value-mixing layer's values)."""

    def __init__(self, batch: RaggedBatch, kv_buffer: dict[int, torch.Tensor], table: torch.Tensor, states) -> None:
        self.batch = batch
        self.kv_buffer = kv_buffer
        self.table = table
        self.states = states
        self.v_first: torch.Tensor | None = None


def mamba2_mixer(li: int, spec: Mamba2Spec, w: dict[str, torch.Tensor], x: torch.Tensor, ctx: StepContext,
                 eps: float) -> torch.Tensor:
    """in-projection -> [z | x B C | dt]; short causal convolution + SiLU on x B C (tail kept per slot); fp32 scan
    against the slot's state; gate, grouped unit-RMS norm, out-projection."""
    b = ctx.batch
    proj = linear(x, w["in"])
    inner = spec.inner
    xbc = causal_conv_silu(proj, inner, spec.conv_channels, w["conv"], w["conv_b"], ctx.states.conv_tail[li],
                           b.seq_start, b.seq_ctx, b.seq_slot)
    dt_raw = proj[:, inner + spec.conv_channels:]
    y = ssm_scan(xbc, dt_raw, w["dt_bias"], w["A_log"], w["D"], ctx.states.ssm_state[li], b.seq_start, b.seq_ctx,
                 b.seq_slot, spec.heads, spec.groups, spec.state, spec.head_dim)
    gated = gated_group_norm(y, proj[:, :inner], w["norm"], spec.norm_groups, eps)
    return linear(gated, w["o"])


_SPLIT_KEYS = 128          # keys per CTA of the single-token attention kernel (4 warps x 32 keys per pass)
_MAX_SPLITS = 128


def sink_attention_mixer(li: int, spec: SinkAttentionSpec, w: dict[str, torch.Tensor], x: torch.Tensor,
                         ctx: StepContext, eps: float) -> torch.Tensor:
    """fused q|k|v projection -> per-token preparation (norms, query gain, value mixing, cache write) -> attention
    over the pool: the tiled kernel for prompt portions, the key-split kernel for single tokens."""
    b = ctx.batch
    qn, kn, vn = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim, spec.kv_heads * spec.v_head_dim
    qkv = linear(x, w["qkv"])
    pool = ctx.kv_buffer[li]
    v_in = v_out = None
    if spec.v_mix:
        if ctx.v_first is None:
            ctx.v_first = v_out = torch.empty((b.tokens, vn), dtype=qkv.dtype, device=qkv.device)
        else:
            v_in = ctx.v_first
    attn_prepare(qkv, pool, b.kv_rows, b.positions, qn, kn, vn, w.get("q_norm"), w.get("k_norm"), eps,
                 spec.gain_coef, spec.gain_every, v_in, v_out, w.get("vmix") if v_in is not None else None)
    out = torch.empty((b.tokens, spec.heads * spec.v_head_dim), dtype=qkv.dtype, device=qkv.device)
    common = (spec.heads, spec.kv_heads, spec.head_dim, spec.v_head_dim, spec.scale, spec.softcap)
    if b.num_portions:
        sink_attention(out, qkv, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.portion_list, b.num_portions,
                       b.max_portion, w.get("sink"), *common)
    if b.num_singles:
        keys = b.max_single_ctx + 1
        splits = max(1, min(_MAX_SPLITS, -(-keys // _SPLIT_KEYS)))
        per = -(-keys // splits)
        per = -(-per // 32) * 32
        sink_attention(out, qkv, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.single_list, b.num_singles, 1,
                       w.get("sink"), *common, num_splits=splits, split_keys=per)
    return linear(out, w["o"])


def dense_feed_forward(spec: DenseMlpSpec, w: dict[str, torch.Tensor], x: torch.Tensor) -> torch.Tensor:
    if spec.activation != "relu2":
        raise ValueError(f"unknown feed-forward activation {spec.activation!r}")
    return linear(relu_squared(linear(x, w["up"])), w["down"])


MIXERS = {"mamba2": mamba2_mixer, "attention": sink_attention_mixer}
FEED_FORWARDS = {"dense": dense_feed_forward}


class LayeredDecoder:
    def __init__(self, cfg: LayeredConfig, weights: LayeredWeights, device: str = "cuda",
                 dtype: torch.dtype = torch.bfloat16, norm_weight_offset: float = 1.0) -> None:
        cfg.validate()
        self.cfg, self.w, self.device, self.dtype = cfg, weights, device, dtype
        self.norm_offset = norm_weight_offset
        self.layer_trace: list[torch.Tensor] | None = None       # set to [] to record the residual after every layer

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, batch: RaggedBatch, kv_buffer: dict[int, torch.Tensor],
                table: torch.Tensor, states, want_rows: torch.Tensor | None = None) -> torch.Tensor:
        """``tokens [T]`` int32 -> logits ``[T or len(want_rows), vocab]`` in the activation dtype."""
        cfg, eps, off = self.cfg, self.cfg.rms_norm_eps, self.norm_offset
        ctx = StepContext(batch, kv_buffer, table, states)
        resid, act = embed_positions(tokens, batch.positions, self.w.embed, self.w.pos)
        for li, (spec, lw) in enumerate(zip(cfg.layers, self.w.layers)):
            x = resid if act is None else act
            y = MIXERS[spec.kind](li, spec.mixer, lw.mix, x, ctx, eps)
            act = post_norm_residual(resid, y, lw.norm1, eps, off)
            if spec.mlp is not None:
                x = resid if act is None else act
                y = FEED_FORWARDS["dense"](spec.mlp, lw.mlp, x)
                act = post_norm_residual(resid, y, lw.norm2, eps, off)
            if self.layer_trace is not None:
                self.layer_trace.append(resid.clone())
        if want_rows is not None and want_rows.numel() == 0:
            return torch.empty((0, cfg.vocab_size), dtype=self.dtype, device=resid.device)
        hidden = rmsnorm_from_f32(resid, self.w.final_norm, eps, off, want_rows)
        return linear(hidden, self.w.head)


# ---------------------------------------------------------------------------------------------- Gufotar plumbing #
def parse_gufotar_config(raw: dict) -> LayeredConfig:
    layers = []
    for entry in raw["layers"]:
        kind, m = entry["type"], entry["mixer"]
        if kind == "mamba2":
            mixer = Mamba2Spec(heads=m["heads"], head_dim=m["vdim"], state=m["state"], groups=m.get("groups", 1),
                               norm_groups=m.get("norm_groups", 1), conv=m.get("conv", 1))
        elif kind == "attention":
            qt = m.get("q_temp") or {}
            mixer = SinkAttentionSpec(heads=m["heads"], kv_heads=m.get("kv_heads", m["heads"]), head_dim=m["dim"],
                                      v_head_dim=m.get("vdim", m["dim"]), scale=float(m["scale"]),
                                      softcap=float(m.get("softcap") or 0.0), gain_coef=float(qt.get("coef", 0.0)),
                                      gain_every=float(qt.get("every", 0.0)) if qt else 0.0, v_mix=bool(m.get("v_mix")))
        else:
            raise ValueError(f"unknown layer type {kind!r}")
        mlp = entry.get("mlp")
        if mlp is not None and mlp.get("kind", "dense") != "dense":
            raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(LayerSpec(kind, mixer, DenseMlpSpec(ff=mlp["ff"]) if mlp is not None else None))
    return LayeredConfig(name=raw.get("architecture", "Gufotar"), hidden_size=raw["width"], vocab_size=raw["vocab"],
                         max_seq_len=raw["max_positions"], rms_norm_eps=float(raw["norm"]["eps"]), layers=tuple(layers))


def map_gufotar_weights(cfg: LayeredConfig, tensors: dict[str, torch.Tensor], device: str,
                        dtype: torch.dtype) -> LayeredWeights:
    """Checkpoint names -> the decoder's weights in the activation dtype; q, k and v are row-concatenated so the three
    projections are one GEMM (each output element is the same dot product)."""

    def get(name: str) -> torch.Tensor:
        if name not in tensors:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return tensors[name].to(device=device, dtype=dtype).contiguous()

    out = LayeredWeights(embed=get("embed"), pos=get("pos"), final_norm=get("final.norm"), head=get("head"))
    for i, spec in enumerate(cfg.layers):
        p = f"l{i}.mix."
        if isinstance(spec.mixer, Mamba2Spec):
            mix = {"in": get(p + "in"), "conv": get(p + "conv"), "conv_b": get(p + "conv.b"),
                   "dt_bias": get(p + "dt_bias"), "A_log": get(p + "A_log"), "D": get(p + "D"),
                   "norm": get(p + "norm"), "o": get(p + "o")}
        else:
            mix = {"qkv": torch.cat([get(p + "q"), get(p + "k"), get(p + "v")], dim=0).contiguous(),
                   "q_norm": get(p + "q.norm"), "k_norm": get(p + "k.norm"), "o": get(p + "o")}
            if p + "sink" in tensors:
                mix["sink"] = get(p + "sink")
            if spec.mixer.v_mix and p + "vmix" in tensors:
                mix["vmix"] = get(p + "vmix").reshape(1)
        lw = LayeredLayerWeights(norm1=get(f"l{i}.norm1"), mix=mix)
        if spec.mlp is not None:
            lw.norm2 = get(f"l{i}.norm2")
            lw.mlp = {"up": get(f"l{i}.mlp.up"), "down": get(f"l{i}.mlp.down")}
        out.layers.append(lw)
    return out


def gufotar_tensor_shapes(cfg: LayeredConfig) -> dict[str, tuple[int, ...]]:
    """Checkpoint tensor names and shapes of a configuration (random initialisation, shape checks)."""
    w = cfg.hidden_size
    shapes: dict[str, tuple[int, ...]] = {"embed": (cfg.vocab_size, w), "pos": (cfg.max_seq_len, w)}
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", spec.mixer
        shapes[f"l{i}.norm1"] = (w,)
        if isinstance(m, Mamba2Spec):
            shapes.update({p + "in": (m.in_rows, w), p + "conv": (m.conv_channels, m.conv), p + "conv.b": (m.conv_channels,),
                           p + "dt_bias": (m.heads,), p + "A_log": (m.heads,), p + "D": (m.heads,),
                           p + "norm": (m.inner,), p + "o": (w, m.inner)})
        else:
            shapes.update({p + "q": (m.heads * m.head_dim, w), p + "k": (m.kv_heads * m.head_dim, w),
                           p + "v": (m.kv_heads * m.v_head_dim, w), p + "q.norm": (m.heads * m.head_dim,),
                           p + "k.norm": (m.kv_heads * m.head_dim,), p + "vmix": (), p + "sink": (m.heads,),
                           p + "o": (w, m.heads * m.v_head_dim)})
        if spec.mlp is not None:
            shapes.update({f"l{i}.norm2": (w,), f"l{i}.mlp.up": (spec.mlp.ff, w), f"l{i}.mlp.down": (w, spec.mlp.ff)})
    shapes.update({"final.norm": (w,), "head": (cfg.vocab_size, w)})
    return shapes


def random_gufotar_tensors(cfg: LayeredConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    """Seeded random bf16 tensors with checkpoint names (benchmarks; there are no trained checkpoints offline)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in gufotar_tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if len(shape) == 2 and leaf != "conv":
            t = torch.randn(shape, generator=g) / (shape[1] ** 0.5)
        elif leaf in ("norm", "D"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf in ("dt_bias", "A_log"):
            t = -1.0 + 0.5 * torch.randn(shape, generator=g)
        elif leaf == "vmix":
            t = torch.tensor(0.4)
        elif name.endswith("q.norm") or name.endswith("k.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        else:
            t = 0.3 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out


register(Architecture("Gufotar", parse_gufotar_config, map_gufotar_weights, LayeredDecoder, ragged_steps=True))
