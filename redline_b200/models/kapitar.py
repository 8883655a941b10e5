"""``Kapitar`` laid out as parts: token embedding; "sandwich" blocks (layer norm before and after every
sublayer) whose mixer is differential attention over a window with kept first tokens (``maps_attention``
with two maps, a capped score, no position encoding) or linear attention with a decaying state
(``linear_attention``), and whose feed-forward is dense (``act_mlp``, squared ReLU), routed
(``routed_experts``: sigmoid router, groups scored by their two best experts, erf GELU, a shared expert)
or absent; a final layer norm and the embedding table as the head.  Tensor names: ``embed``,
``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""

from __future__ import annotations

import math
from typing import Iterator, Tuple

import torch

from ..config.model_config import KapitarConfig
from ..config.registry import Architecture, register_architecture
from ..parts.attention_maps import MapsAttentionParams
from ..parts.embedding import EmbeddingParams, HeadParams
from ..parts.layernorm import LayerNormParams
from ..parts.linear_attention import LinearAttentionParams
from ..parts.moe import ActMLPParams, RoutedExpertsParams
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

GROUP_TOP = 2          # a group of experts is scored by its two best


def kapitar_spec(c: KapitarConfig) -> ModelSpec:
    W = c.hidden_size

    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", LayerNormParams(W, c.norm_eps), {"weight": name})

    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "attention":
            names = {n: f"{p}mix.{n}" for n in ("q", "k", "v", "o", "lq1", "lk1", "lq2", "lk2")}
            names.update({f"{n}_bias": f"{p}mix.{n}.b" for n in "qkv"})
            mixer = PartSpec("maps_attention", MapsAttentionParams(
                hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, maps=2, bias=True,
                window=m.mask.size, keep_first=m.mask.keep_first, scale=m.scale, softcap=m.softcap, diff=m.diff,
                unit_norm=True, post_scale=1.0 - m.diff, eps=c.norm_eps), names)
        else:
            mixer = PartSpec("linear_attention", LinearAttentionParams(
                hidden_size=W, num_heads=m.heads, dim=m.dim, vdim=m.vdim, decay=tuple(m.decay), eps=c.norm_eps,
                activation="silu"), {n: f"{p}mix.{n}" for n in ("q", "k", "v", "g", "o", "norm")})
        f = layer.mlp
        ffn = None
        if f is not None and f.kind == "dense":
            ffn = PartSpec("act_mlp", ActMLPParams(W, f.ff, "relu_squared"), {"up": p + "mlp.up", "down": p + "mlp.down"})
        elif f is not None:
            names = {"router": p + "mlp.router"}
            for e in range(f.experts):
                names[f"up{e}"] = f"{p}mlp.e{e}.up"
                names[f"down{e}"] = f"{p}mlp.e{e}.down"
            if f.shared_ff > 0:
                names.update({"shared_up": p + "mlp.shared.up", "shared_down": p + "mlp.shared.down"})
            ffn = PartSpec("routed_experts", RoutedExpertsParams(
                hidden_size=W, intermediate_size=f.ff, num_experts=f.experts, top=f.top, groups=f.groups,
                group_keep=f.groups_keep, group_top=GROUP_TOP, score="sigmoid", renormalize=False, activation="gelu",
                shared_intermediate_size=f.shared_ff), names)
        layers.append(LayerSpec(
            arrangement="sandwich", mixer_norm=norm(p + "norm1"), mixer=mixer,
            ffn_norm=norm(p + "norm2") if ffn is not None else None, ffn=ffn,
            mixer_post_norm=norm(p + "norm1b"), ffn_post_norm=norm(p + "norm2b") if ffn is not None else None))
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab_size, max_positions=c.max_position_embeddings,
        embedding=PartSpec("token_embedding", EmbeddingParams(c.vocab_size, W), {"weight": "embed"}),
        layers=tuple(layers), order=tuple(LayerCall(i) for i in range(len(layers))),
        final_norm=norm("final.norm"), head=PartSpec("lm_head", HeadParams(c.vocab_size, W, True), {}))


def kapitar_random_tensors(c: KapitarConfig, seed: int, dtype: torch.dtype) -> Iterator[Tuple[str, tuple, object]]:
    """Yields (name, shape, make) in file order: matrices N(0, 1 / fan_in), the embedding N(0, 1), norm
    weights 1 + N(0, 0.1^2), biases and the lambda vectors N(0, 0.1^2); one seeded generator run in order."""
    g = torch.Generator().manual_seed(seed)
    W = c.hidden_size

    def mat(n, k, std=None):
        return (n, k), lambda: (torch.randn(n, k, generator=g) * (std if std is not None else 1.0 / math.sqrt(k))).to(dtype)

    def vec(n, mean, std):
        return (n,), lambda: (mean + std * torch.randn(n, generator=g)).to(dtype)

    def emit(name, shape_make):
        return name, shape_make[0], shape_make[1]

    yield emit("embed", mat(c.vocab_size, W, 1.0))
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        m = layer.mixer
        yield emit(p + "norm1", vec(W, 1.0, 0.1))
        yield emit(p + "norm1b", vec(W, 1.0, 0.1))
        if layer.type == "attention":
            for n, rows in (("q", m.heads * 2 * m.dim), ("k", m.kv_heads * 2 * m.dim), ("v", m.kv_heads * m.vdim)):
                yield emit(f"{p}mix.{n}", mat(rows, W))
                yield emit(f"{p}mix.{n}.b", vec(rows, 0.0, 0.1))
            for n in ("lq1", "lk1", "lq2", "lk2"):
                yield emit(f"{p}mix.{n}", vec(m.dim, 0.0, 0.1))
            yield emit(p + "mix.o", mat(W, m.heads * m.vdim))
        else:
            for n, rows in (("q", m.heads * m.dim), ("k", m.heads * m.dim), ("v", m.heads * m.vdim), ("g", m.heads * m.vdim)):
                yield emit(f"{p}mix.{n}", mat(rows, W))
            yield emit(p + "mix.o", mat(W, m.heads * m.vdim))
            yield emit(p + "mix.norm", vec(m.heads * m.vdim, 1.0, 0.1))
        f = layer.mlp
        if f is None:
            continue
        yield emit(p + "norm2", vec(W, 1.0, 0.1))
        yield emit(p + "norm2b", vec(W, 1.0, 0.1))
        if f.kind == "dense":
            yield emit(p + "mlp.up", mat(f.ff, W))
            yield emit(p + "mlp.down", mat(W, f.ff))
        else:
            for e in range(f.experts):
                yield emit(f"{p}mlp.e{e}.up", mat(f.ff, W))
                yield emit(f"{p}mlp.e{e}.down", mat(W, f.ff))
            yield emit(p + "mlp.router", mat(f.experts, W))
            if f.shared_ff > 0:
                yield emit(p + "mlp.shared.up", mat(f.shared_ff, W))
                yield emit(p + "mlp.shared.down", mat(W, f.shared_ff))
    yield emit("final.norm", vec(W, 1.0, 0.1))


register_architecture(Architecture(
    name="Kapitar",
    config_from_hf=KapitarConfig.from_hf,
    build_spec=kapitar_spec,
    random_tensors=kapitar_random_tensors,
))
