"""Grouped-query causal attention with score maps over the paged cache.

Every head has ``maps`` score maps (queries and keys of ``dim`` each) over the same values of ``vdim``;
two maps are combined as a difference, o = a1 - lambda * a2 (differential attention), one is ordinary
attention.  Scores may be capped, s <- cap * tanh(s / cap); the mask is causal with a sliding window that
keeps the first ``keep_first`` tokens of the sequence visible; a head's output may be divided by its root
mean square and multiplied by ``post_scale``.  q, k and v come from one fused projection [q | k | v] with
optional biases; a position encoding, if the layer has one, is applied to q and k before the cache write.

The cache holds keys [kv_heads * maps, dim] and values [kv_heads, vdim] per token (a window group that
keeps its first pages); sequences that bring one token go to the partitioned decode kernel, longer
portions to the tiled kernel (csrc/attention_maps.cu); scores, softmax, combination and norm in float32.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import LayerCache, Mixer, build_part, op_mark, register
from .spec import CacheSpec, CacheTensor, PartSpec, TensorSpec


@dataclass(frozen=True)
class MapsAttentionParams:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    dim: int                     # size of a query / key of one map
    vdim: int                    # size of a value
    maps: int = 1                # 2: differential attention
    bias: bool = False           # q, k, v projections have biases
    window: int = 0              # 0: every earlier key
    keep_first: int = 0          # the first tokens stay visible behind the window
    scale: Optional[float] = None
    softcap: float = 0.0         # 0: scores are not capped
    diff: float = 0.0            # maps = 2: lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
    unit_norm: bool = False      # divide a head's output by its root mean square
    post_scale: float = 1.0      # and multiply it by this
    eps: float = 1e-6
    position: Optional[PartSpec] = None


@register("mixer", "maps_attention")
class MapsAttention(Mixer):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        if p.num_heads % p.num_kv_heads != 0:
            raise ValueError(f"num_heads {p.num_heads} is no multiple of num_kv_heads {p.num_kv_heads}")
        if p.maps not in (1, 2):
            raise ValueError(f"attention with {p.maps} score maps is not supported (1 or 2)")
        if not (1 <= p.dim <= 256 and 4 <= p.vdim <= 256 and p.vdim % 4 == 0):
            raise ValueError(f"attention_maps kernels take key sizes up to 256 and value sizes that are multiples "
                             f"of 4 up to 256; got dim={p.dim}, vdim={p.vdim}")
        self.position = build_part("position", p.position, rt) if p.position is not None else None
        if self.position is not None and self.position.rotary_tables() is not None:
            raise ValueError("maps_attention applies a position encoding through its apply(); rotary tables are "
                             "for the attention part whose cache-write kernel rotates")
        self.scale = p.scale if p.scale is not None else 1.0 / math.sqrt(p.dim)
        self.q_size = p.num_heads * p.maps * p.dim
        self.k_size = p.num_kv_heads * p.maps * p.dim
        self.v_size = p.num_kv_heads * p.vdim
        self.qkv_size = self.q_size + self.k_size + self.v_size
        self.out_size = p.num_heads * p.vdim
        self.lam = 0.0

    def cache_spec(self) -> CacheSpec:
        p = self.params
        tensors = (CacheTensor("k", (p.num_kv_heads * p.maps, p.dim)), CacheTensor("v", (p.num_kv_heads, p.vdim)))
        if p.window > 0:
            return CacheSpec("window", tensors, p.window, p.keep_first)
        return CacheSpec("full", tensors)

    def tiling(self):
        return kernels.PREFILL_TILE_ROWS, kernels.DECODE_PARTITION

    def tensors(self) -> Dict[str, TensorSpec]:
        p = self.params
        t = {
            "q": TensorSpec((self.q_size, p.hidden_size)),
            "k": TensorSpec((self.k_size, p.hidden_size)),
            "v": TensorSpec((self.v_size, p.hidden_size)),
            "o": TensorSpec((p.hidden_size, self.out_size)),
            "q_bias": TensorSpec((self.q_size,), optional=not p.bias),
            "k_bias": TensorSpec((self.k_size,), optional=not p.bias),
            "v_bias": TensorSpec((self.v_size,), optional=not p.bias),
        }
        if p.maps == 2:
            t.update({n: TensorSpec((p.dim,)) for n in ("lq1", "lk1", "lq2", "lk2")})
        return t

    def fused(self) -> Dict[str, list]:
        return {"qkv": ["q", "k", "v"]}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.params
        if "qkv" in tensors:
            self.w_qkv = tensors["qkv"]
        else:
            q, k, v = tensors["q"], tensors["k"], tensors["v"]
            dt = torch.float32 if torch.float32 in (q.dtype, k.dtype, v.dtype) else q.dtype
            self.w_qkv = torch.cat([q.to(dt), k.to(dt), v.to(dt)], dim=0).contiguous()
        self.w_o = tensors["o"]
        self.b_qkv = None
        if p.bias:
            self.b_qkv = torch.cat([tensors[n].float() for n in ("q_bias", "k_bias", "v_bias")]).contiguous()
        if p.maps == 2:
            # one number for the layer, in float32 like everything around the scores
            lq1, lk1, lq2, lk2 = (tensors[n].float() for n in ("lq1", "lk1", "lq2", "lk2"))
            self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + p.diff)

    def nbytes(self) -> int:
        return self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()

    def forward(self, x, ctx, cache: Optional[LayerCache], state=None) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        ws = rt.workspace
        qkv = ws.get("mattn.qkv", (rt.max_tokens, self.qkv_size), rt.dtype)[:T]
        linear(x, self.w_qkv, qkv)
        if self.b_qkv is not None:
            kernels.bias_act(qkv, self.b_qkv, kernels.ACT_NONE)
        op_mark(ctx, "qkv_proj", self.w_qkv, T)
        if self.position is not None:
            self.position.apply(qkv, p.num_heads * p.maps, p.num_kv_heads * p.maps, p.dim, ctx)
        g = ctx.groups[cache.group]
        k_cache, v_cache = cache.tensors["k"], cache.tensors["v"]
        if cache.write:
            kernels.cache_store(qkv, self.q_size, p.num_kv_heads * p.maps, p.dim, g.slots, k_cache, rt.page_size,
                                ctx.status, tokens=T)
            kernels.cache_store(qkv, self.q_size + self.k_size, p.num_kv_heads, p.vdim, g.slots, v_cache,
                                rt.page_size, ctx.status, tokens=T)
            op_mark(ctx, "kv_write", nbytes=2.0 * T * (self.k_size + self.v_size) * qkv.element_size())
        attn = ws.get("mattn.out", (rt.max_tokens, self.out_size), rt.dtype)[:T]
        common = (p.num_heads, p.num_kv_heads, p.dim, p.vdim, p.maps, rt.page_size, p.window, p.keep_first,
                  self.scale, p.softcap, self.lam, p.post_scale, p.eps, p.unit_norm)
        if ctx.num_decode > 0:
            rows = ctx.max_items * p.num_heads * p.maps * ctx.parts_capacity
            part_o = ws.get("mattn.part_o", (rows * p.vdim,), torch.float32)
            part_ml = ws.get("mattn.part_ml", (rows * 2,), torch.float32)
            kernels.maps_attn_decode(qkv, self.qkv_size, k_cache, v_cache, g.block_table, ctx.decode_info, part_o,
                                     part_ml, ctx.decode_parts, attn, ctx.num_decode, *common)
            self._mark(ctx, "attention_decode", "decode")
        if ctx.num_tiles > 0:
            kernels.maps_attn_prefill(qkv, self.qkv_size, k_cache, v_cache, g.block_table, ctx.tile_seq, ctx.tile_tok,
                                      ctx.tile_rows, ctx.positions, attn, ctx.num_tiles, kernels.PREFILL_TILE_ROWS,
                                      *common)
            self._mark(ctx, "attention_prefill", "prefill")
        out = ws.get("mixer.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        linear(attn, self.w_o, out)
        op_mark(ctx, "o_proj", self.w_o, T)
        return out

    def _mark(self, ctx, op: str, which: str) -> None:
        if ctx.profiler is None:
            return
        from ..engine.profiler import attention_work
        p = self.params
        elem = 2 if self.rt.dtype == torch.bfloat16 else 4
        window = p.window + p.keep_first if p.window > 0 else 0
        nbytes, flops = attention_work(ctx.host, p.num_heads * p.maps, p.num_kv_heads * p.maps, (p.dim + p.vdim) // 2,
                                       window, elem)[which]
        ctx.profiler.mark(op, nbytes, flops)
