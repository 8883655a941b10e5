"""``Pufevik`` laid out as parts: a token embedding multiplied by a constant; "outnorm" blocks (the sublayers
read the stream itself, RMS norms on what they put out) whose mixer is gated softmax attention
(``maps_attention`` with one map: queries and keys normed per head, the heads' first entries rotated in
neighbouring pairs, a gate per output entry, values blended with those of the first such layer) or a pair
side by side (``parallel_mixers``): windowed attention with a sink, norms over the whole projection and a
gate per head, beside a matrix memory with exponential gates (``matrix_memory``); a dense gated feed-forward
with the tanh GELU, or none; a final RMS norm and a head of its own.  Tensor names: ``embed``,
``l<i>.norm1|norm2``, ``l<i>.mix.*`` (``l<i>.mix.left.*`` / ``l<i>.mix.right.*`` in a pair), ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

import math
from typing import Iterator, Tuple

import torch

from ..config.model_config import PufevikAttention, PufevikConfig
from ..config.registry import Architecture, register_architecture
from ..parts.attention_maps import MapsAttentionParams
from ..parts.embedding import EmbeddingParams, HeadParams
from ..parts.layernorm import LayerNormParams
from ..parts.matrix_memory import MatrixMemoryParams
from ..parts.mlp import GatedMLPParams
from ..parts.parallel import parallel_spec
from ..parts.rmsnorm import RMSNormParams
from ..parts.rope import RotaryPairsParams
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MEMORY_DENOMINATOR_FLOOR = 1e-6      # the design fixes it


def _attention_spec(c: PufevikConfig, a: PufevikAttention, prefix: str, paired: bool, value_mix: str) -> PartSpec:
    names = {n: prefix + n for n in ("q", "k", "v", "o", "g")}
    names.update({"q_norm": prefix + "q.norm", "k_norm": prefix + "k.norm"})
    if paired:
        names["sink"] = prefix + "sink"
    if value_mix != "none":
        names["vmix"] = prefix + "vmix"
    position = None
    if a.rot is not None:
        position = PartSpec("rope_pairs", RotaryPairsParams(a.rot.dims, a.rot.base, c.max_position_embeddings))
    return PartSpec("maps_attention", MapsAttentionParams(
        hidden_size=c.hidden_size, num_heads=a.heads, num_kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim, maps=1,
        window=a.window, scale=a.scale, eps=c.norm_eps, position=position,
        head_norm="whole" if paired else "each", sink=paired, gate="head" if paired else "entry",
        value_mix=value_mix), names)


def pufevik_spec(c: PufevikConfig) -> ModelSpec:
    W = c.hidden_size

    def out_norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm_sandwich", LayerNormParams(W, c.norm_eps), {"weight": name})

    layers = []
    mixing = False           # a layer before this one already provides the values that later ones blend in
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "attention":
            mix = "none" if not m.v_mix else ("blend" if mixing else "keep")
            mixing = mixing or m.v_mix
            mixer = _attention_spec(c, m, p + "mix.", False, mix)
        else:
            r = m.right
            names = {n: f"{p}mix.right.{n}" for n in ("q", "k", "v", "g", "o", "norm", "i", "f")}
            names.update({"i_bias": p + "mix.right.i.b", "f_bias": p + "mix.right.f.b"})
            memory = PartSpec("matrix_memory", MatrixMemoryParams(
                hidden_size=W, num_heads=r.heads, dim=r.dim, vdim=r.vdim, gate_cap=r.gate_cap, eps=c.norm_eps,
                floor=MEMORY_DENOMINATOR_FLOOR), names)
            mixer = parallel_spec(W, _attention_spec(c, m.left, p + "mix.left.", True, "none"), memory,
                                  m.left_scale, m.right_scale)
        ffn = None
        if layer.ff > 0:
            ffn = PartSpec("swiglu_mlp", GatedMLPParams(W, layer.ff, activation="gelu_tanh"),
                           {n: f"{p}mlp.{n}" for n in ("gate", "up", "down")})
        layers.append(LayerSpec(arrangement="outnorm", mixer_norm=None, mixer=mixer, ffn=ffn,
                                mixer_post_norm=out_norm(p + "norm1"),
                                ffn_post_norm=out_norm(p + "norm2") if ffn is not None else None))
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab_size, max_positions=c.max_position_embeddings,
        embedding=PartSpec("token_embedding", EmbeddingParams(c.vocab_size, W, c.embedding_scale), {"weight": "embed"}),
        layers=tuple(layers), order=tuple(LayerCall(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", RMSNormParams(W, c.norm_eps), {"weight": "final.norm"}),
        head=PartSpec("lm_head", HeadParams(c.vocab_size, W, False), {"weight": "head"}))


def pufevik_random_tensors(c: PufevikConfig, seed: int, dtype: torch.dtype) -> Iterator[Tuple[str, tuple, object]]:
    """Yields (name, shape, make) in file order: matrices N(0, 1 / fan_in), the embedding N(0, 1), norm
    weights 1 + N(0, 0.1^2), sinks and gate biases N(0, 1) (the forget gate's around 2), blend numbers in
    (0.2, 0.7); one seeded generator run in order."""
    g = torch.Generator().manual_seed(seed)
    W = c.hidden_size

    def mat(n, k, std=None):
        return (n, k), lambda: (torch.randn(n, k, generator=g) * (std if std is not None else 1.0 / math.sqrt(k))).to(dtype)

    def vec(n, mean, std):
        return (n,), lambda: (mean + std * torch.randn(n, generator=g)).to(dtype)

    def emit(name, shape_make):
        return name, shape_make[0], shape_make[1]

    def attention(p: str, a: PufevikAttention, paired: bool):
        for n, rows in (("q", a.heads * a.dim), ("k", a.kv_heads * a.dim), ("v", a.kv_heads * a.vdim)):
            yield emit(p + n, mat(rows, W))
        yield emit(p + "q.norm", vec(a.heads * a.dim if paired else a.dim, 1.0, 0.1))
        yield emit(p + "k.norm", vec(a.kv_heads * a.dim if paired else a.dim, 1.0, 0.1))
        if paired:
            yield emit(p + "sink", vec(a.heads, 0.0, 1.0))
        yield emit(p + "g", mat(a.heads if paired else a.heads * a.vdim, W))
        yield emit(p + "o", mat(W, a.heads * a.vdim))

    yield emit("embed", mat(c.vocab_size, W, 1.0))
    mixing = False
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        m = layer.mixer
        yield emit(p + "norm1", vec(W, 1.0, 0.1))
        if layer.type == "attention":
            yield from attention(p + "mix.", m, False)
            if m.v_mix:
                yield emit(p + "mix.vmix", ((), lambda: (0.2 + 0.5 * torch.rand((), generator=g)).to(dtype)))
            mixing = mixing or m.v_mix
        else:
            yield from attention(p + "mix.left.", m.left, True)
            r = m.right
            q = p + "mix.right."
            for n, rows in (("q", r.heads * r.dim), ("k", r.heads * r.dim), ("v", r.heads * r.vdim), ("g", r.heads * r.vdim)):
                yield emit(q + n, mat(rows, W))
            yield emit(q + "o", mat(W, r.heads * r.vdim))
            yield emit(q + "norm", vec(r.heads * r.vdim, 1.0, 0.1))
            yield emit(q + "i", mat(r.heads, W))
            yield emit(q + "i.b", vec(r.heads, 0.0, 1.0))
            yield emit(q + "f", mat(r.heads, W))
            yield emit(q + "f.b", vec(r.heads, 2.0, 1.0))
        if layer.ff > 0:
            yield emit(p + "norm2", vec(W, 1.0, 0.1))
            yield emit(p + "mlp.gate", mat(layer.ff, W))
            yield emit(p + "mlp.up", mat(layer.ff, W))
            yield emit(p + "mlp.down", mat(W, layer.ff))
    yield emit("final.norm", vec(W, 1.0, 0.1))
    yield emit("head", mat(c.vocab_size, W))


register_architecture(Architecture(
    name="Pufevik",
    config_from_hf=PufevikConfig.from_hf,
    build_spec=pufevik_spec,
    random_tensors=pufevik_random_tensors,
))
