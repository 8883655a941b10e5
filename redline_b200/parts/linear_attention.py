"""Linear attention with a decaying state per head ("lightning" attention).

q = f(W_q h), k = f(W_k h) (heads x dim), v = f(W_v h) (heads x vdim), f an activation (SiLU); per head
S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t.  The joined heads are RMS-normed with a weight,
multiplied by sigmoid(W_g h) and projected by W_o.  The state S (float32, [heads, dim, vdim]) is this
mixer's per-request state: zero for a new request, carried from step to step in the request's slot;
there is no cache of keys.  q, k, v and g come from one fused projection [q | k | v | g]; the recurrence
(csrc/linear_attention.cu), its output and the norm are float32.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, op_mark, register
from .spec import StateSpec, TensorSpec


@dataclass(frozen=True)
class LinearAttentionParams:
    hidden_size: int
    num_heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]       # one per head
    eps: float = 1e-6
    activation: str = "silu"       # of q, k and v
    gated: bool = True             # multiply the normed output by sigmoid(W_g h)


@register("mixer", "linear_attention")
class LinearAttention(Mixer):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        if len(p.decay) != p.num_heads:
            raise ValueError(f"linear attention of {p.num_heads} heads needs as many decays, got {len(p.decay)}")
        if not 1 <= p.dim <= 256:
            raise ValueError(f"linear attention kernels take key sizes up to 256; got {p.dim}")
        if not p.gated:
            raise ValueError("linear attention without an output gate is not built")
        self.qk_size = p.num_heads * p.dim
        self.v_size = p.num_heads * p.vdim
        self.proj_size = 2 * self.qk_size + 2 * self.v_size
        self.decay = torch.tensor(p.decay, dtype=torch.float32, device=rt.device)
        self.act = kernels.ACTIVATIONS[p.activation]

    def state_spec(self) -> StateSpec:
        p = self.params
        return StateSpec((p.num_heads, p.dim, p.vdim), "float32")

    def state_in_graphs(self) -> bool:
        return True

    def tensors(self) -> Dict[str, TensorSpec]:
        p = self.params
        return {
            "q": TensorSpec((self.qk_size, p.hidden_size)),
            "k": TensorSpec((self.qk_size, p.hidden_size)),
            "v": TensorSpec((self.v_size, p.hidden_size)),
            "g": TensorSpec((self.v_size, p.hidden_size)),
            "o": TensorSpec((p.hidden_size, self.v_size)),
            "norm": TensorSpec((self.v_size,)),
        }

    def fused(self) -> Dict[str, list]:
        return {"qkvg": ["q", "k", "v", "g"]}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        if "qkvg" in tensors:
            self.w_in = tensors["qkvg"]
        else:
            ws = [tensors[n] for n in ("q", "k", "v", "g")]
            dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
            self.w_in = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.w_o = tensors["o"]
        self.w_norm = tensors["norm"]

    def nbytes(self) -> int:
        return self.w_in.numel() * self.w_in.element_size() + self.w_o.numel() * self.w_o.element_size()

    def forward(self, x, ctx, cache, state) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        ws = rt.workspace
        proj = ws.get("lin.proj", (rt.max_tokens, self.proj_size), rt.dtype)[:T]
        linear(x, self.w_in, proj)
        kernels.bias_act(proj, None, self.act, cols=2 * self.qk_size + self.v_size)
        op_mark(ctx, "qkvg_proj", self.w_in, T)
        o = ws.get("lin.o", (rt.max_tokens, self.v_size), torch.float32)[:T]
        # (how a step is cut depends on its shape alone: single-token steps and full portions replay as graphs)
        chunk, max_chunks = kernels.linear_attention_chunks(1 if ctx.num_tiles == 0 else max(ctx.host.q_len))
        chunk_state = None
        if max_chunks > 1:
            chunk_state = ws.get("lin.chunks", (ctx.S * max_chunks * p.num_heads * p.dim * p.vdim,), torch.float32)
        kernels.linear_attention(proj, 0, self.qk_size, 2 * self.qk_size, ctx.seq_of_token, ctx.state_slot, self.decay,
                                 state, o, T, ctx.S, p.num_heads, p.dim, p.vdim, chunk_state, chunk, max_chunks)
        op_mark(ctx, "linear_attention", nbytes=T * (self.proj_size * proj.element_size() + 4.0 * self.v_size),
                flops=4.0 * T * p.num_heads * p.dim * p.vdim)
        y = ws.get("lin.y", (rt.max_tokens, self.v_size), rt.dtype)[:T]
        kernels.gated_rmsnorm(o, proj[:, 2 * self.qk_size + self.v_size:], self.w_norm, y, p.eps, rows=T)
        out = ws.get("mixer.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        linear(y, self.w_o, out)
        op_mark(ctx, "o_proj", self.w_o, T)
        return out
