"""A matrix memory per head with exponential gates (the mLSTM cell of xLSTM).

q = W_q h * q_scale, k = W_k h (heads x dim), v = W_v h (heads x vdim); per head the logarithm of an input
gate i = cap * tanh((W_i h + b_i) / cap) and of a forget gate f = logsigmoid(cap * tanh((W_f h + b_f) / cap)).
With a running stabiliser m (0 at the start of a sequence, like the state):

    m_t = max(f + m_(t-1), i)
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T        n_t likewise with k alone
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + floor)

Every head's o is divided by its root mean square, the joined heads multiplied by a weight and by
sigmoid(W_g h), then projected by W_o.  S, n and m (float32) are this mixer's per-request state, carried
from step to step in the request's slot; there is no cache of keys.  q, k, v and g come from one fused
projection [q | k | v | g]; the gates' projections [i | f] are a product of their own with a float32
result; gates, stabiliser, recurrence, division and norm are float32 (csrc/matrix_memory.cu).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, op_mark, register
from .spec import StateSpec, TensorSpec


@dataclass(frozen=True)
class MatrixMemoryParams:
    hidden_size: int
    num_heads: int
    dim: int
    vdim: int
    gate_cap: float = 0.0              # 0: the gates' projections are not capped
    eps: float = 1e-6                  # of the heads' unit norm
    q_scale: Optional[float] = None    # None: dim^(-1/2)
    floor: float = 1e-6                # added to the denominator


@register("mixer", "matrix_memory")
class MatrixMemory(Mixer):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        if not 1 <= p.dim <= 256:
            raise ValueError(f"matrix memory kernels take key sizes up to 256; got {p.dim}")
        self.qk_size = p.num_heads * p.dim
        self.v_size = p.num_heads * p.vdim
        self.proj_size = 2 * self.qk_size + 2 * self.v_size
        self.q_scale = p.q_scale if p.q_scale is not None else p.dim ** -0.5

    def state_spec(self) -> StateSpec:
        p = self.params
        return StateSpec((kernels.matrix_memory_state_floats(p.num_heads, p.dim, p.vdim),), "float32")

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
            "i": TensorSpec((p.num_heads, p.hidden_size)),
            "f": TensorSpec((p.num_heads, p.hidden_size)),
            "i_bias": TensorSpec((p.num_heads,)),
            "f_bias": TensorSpec((p.num_heads,)),
        }

    def fused(self) -> Dict[str, list]:
        return {"qkvg": ["q", "k", "v", "g"], "gates": ["i", "f"]}

    @staticmethod
    def _joined(tensors, fused_name, members):
        if fused_name in tensors:
            return tensors[fused_name]
        ws = [tensors[n] for n in members]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        return torch.cat([w.to(dt) for w in ws], dim=0).contiguous()

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_in = self._joined(tensors, "qkvg", ["q", "k", "v", "g"])
        self.w_gates = self._joined(tensors, "gates", ["i", "f"])
        self.w_o = tensors["o"]
        self.w_norm = tensors["norm"]
        self.b_i = tensors["i_bias"].float().contiguous()
        self.b_f = tensors["f_bias"].float().contiguous()

    def nbytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_gates, self.w_o))

    def inner_size(self) -> int:
        return self.v_size

    def out_weight(self) -> torch.Tensor:
        return self.w_o

    def forward(self, x, ctx, cache, state) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        y = rt.workspace.get("mem.y", (rt.max_tokens, self.v_size), rt.dtype)[:T]
        self.forward_inner(x, ctx, cache, state, y)
        out = rt.workspace.get("mixer.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        linear(y, self.w_o, out)
        op_mark(ctx, "o_proj", self.w_o, T)
        return out

    def forward_inner(self, x, ctx, cache, state, y: torch.Tensor, scale: float = 1.0) -> None:
        """Everything before the output projection: y [T, heads * vdim] (possibly a view of columns of a
        wider buffer) <- scale * the normed, gated heads."""
        p, rt = self.params, self.rt
        T = ctx.T
        ws = rt.workspace
        proj = ws.get("mem.proj", (rt.max_tokens, self.proj_size), rt.dtype)[:T]
        linear(x, self.w_in, proj)
        op_mark(ctx, "qkvg_proj", self.w_in, T)
        gates = ws.get("mem.gates", (rt.max_tokens, 2 * p.num_heads), torch.float32)[:T]
        linear(x, self.w_gates, gates)
        op_mark(ctx, "gate_proj", self.w_gates, T)
        stab = ws.get("mem.stab", (rt.max_tokens, p.num_heads), torch.float32)[:T]
        qn = ws.get("mem.qn", (rt.max_tokens, p.num_heads), torch.float32)[:T]
        num = ws.get("mem.num", (rt.max_tokens, self.v_size), torch.float32)[:T]
        # (how a step is cut depends on its shape alone: single-token steps and full portions replay as graphs)
        chunk, max_chunks = kernels.linear_attention_chunks(1 if ctx.num_tiles == 0 else max(ctx.host.q_len))
        chunk_state = None
        if max_chunks > 1:
            chunk_state = ws.get("mem.chunks", (ctx.S * max_chunks * p.num_heads * p.dim * (p.vdim + 1),), torch.float32)
        kernels.matrix_memory(proj, 0, self.qk_size, 2 * self.qk_size, self.q_scale, gates, self.b_i, self.b_f,
                              p.gate_cap, ctx.seq_of_token, ctx.state_slot, state, stab, num, qn, T, ctx.S,
                              p.num_heads, p.dim, p.vdim, chunk_state, chunk, max_chunks)
        op_mark(ctx, "matrix_memory", nbytes=T * (self.proj_size * proj.element_size() + 4.0 * self.v_size),
                flops=4.0 * T * p.num_heads * p.dim * (p.vdim + 1))
        kernels.matrix_memory_output(num, qn, stab, proj[:, 2 * self.qk_size + self.v_size:], self.w_norm, y, T,
                                     p.num_heads, p.dim, p.vdim, p.eps, p.floor, scale)
        op_mark(ctx, "memory_norm+gate", nbytes=T * self.v_size * (4.0 + 2.0 * proj.element_size()))
