"""Plain, slow implementation of the Kapitar decoder: the oracle of its tests.

Whole sequences, no cache, no batching, float64, one function per mechanism.  It shares
no code with ``redline_b200``: it reads the configuration dictionary itself, draws its own
random weights and writes its own safetensors file.

The model in this file's notation (x_t is the stream at token t, W applied as W x):

  layer:      x += LN_1b(mixer(LN_1(x)));  x += LN_2b(ff(LN_2(x)))      LN = layer norm, weight only
  attention:  two score maps per head over shared values, no positional rotation;
              s = cap * tanh(scale * (q . k) / cap); key j visible from i when j <= i and
              (i - j < size or j < keep_first); softmax; o = a1 - lam * a2 with
              lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff; o is divided by its root mean square
              per head and multiplied by (1 - diff); output projection
  lightning:  q, k, v = silu(projections); S_t = decay_h S_(t-1) + k_t v_t^T; o_t = S_t^T q_t;
              heads joined, RMS norm with a weight, times sigmoid(W_g h), output projection
  dense ff:   W_down relu(W_up h)^2
  routed ff:  sigmoid router scores; experts in equal groups of neighbours, a group scored by
              its two best experts, the best ``keep`` groups stay; the ``top`` best experts of
              those, weighted by their scores as they are; expert = W_down gelu(W_up h) (erf
              form); a shared expert of the same form is added
  output:     LN_final, logits with the embedding table
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

F64 = torch.float64

# When set to a 16-bit type, what a 16-bit engine stores in that type is rounded here as well (norm
# outputs, projections and activations, cached keys and values, mixer and feed-forward outputs);
# the stream, scores, states, routers and norms' arithmetic stay in double precision.
STORE_DTYPE: Optional[torch.dtype] = None


def stored(x: torch.Tensor) -> torch.Tensor:
    return x if STORE_DTYPE is None else x.to(STORE_DTYPE).to(F64)


# ------------------------------------------------------------------ small pieces

def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    return j <= i and (i - j < size or j < keep_first)


# ------------------------------------------------------------------ mixers

def diff_lambda(w: Dict[str, torch.Tensor], p: str, diff: float) -> float:
    a = float(torch.exp((w[p + "lq1"].to(F64) * w[p + "lk1"].to(F64)).sum()))
    b = float(torch.exp((w[p + "lq2"].to(F64) * w[p + "lk2"].to(F64)).sum()))
    return a - b + diff


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """h [T, width] -> [T, width].  ``m`` is the layer's ``mixer`` dictionary."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, keep = m["mask"]["size"], m["mask"]["keep_first"]
    cap, scale, diff = m["softcap"], m["scale"], m["diff"]
    q = stored(h @ w[p + "q"].to(F64).T + w[p + "q.b"].to(F64)).view(T, H, 2, D)
    k = stored(h @ w[p + "k"].to(F64).T + w[p + "k.b"].to(F64)).view(T, G, 2, D)
    v = stored(h @ w[p + "v"].to(F64).T + w[p + "v.b"].to(F64)).view(T, G, DV)
    lam = diff_lambda(w, p, diff)
    mask = torch.tensor([[visible(i, j, size, keep) for j in range(T)] for i in range(T)])
    out = torch.zeros(T, H, DV, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        maps = []
        for mp in range(2):
            s = (q[:, hd, mp] @ k[:, g, mp].T) * scale
            s = cap * torch.tanh(s / cap)
            s = s.masked_fill(~mask, -math.inf)
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, hd] = unit_rms(o, eps) * (1.0 - diff)
    return stored(stored(out.reshape(T, H * DV)) @ w[p + "o"].to(F64).T)


def lightning_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    q = stored(silu(h @ w[p + "q"].to(F64).T)).view(T, H, D)
    k = stored(silu(h @ w[p + "k"].to(F64).T)).view(T, H, D)
    v = stored(silu(h @ w[p + "v"].to(F64).T)).view(T, H, DV)
    gate = torch.sigmoid(stored(h @ w[p + "g"].to(F64).T))
    o = torch.zeros(T, H, DV, dtype=F64)
    for hd in range(H):
        S = torch.zeros(D, DV, dtype=F64)
        for t in range(T):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    y = unit_rms(o.reshape(T, H * DV), eps) * w[p + "norm"].to(F64) * gate
    return stored(stored(y) @ w[p + "o"].to(F64).T)


# ------------------------------------------------------------------ feed-forwards

def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    a = stored(torch.relu(stored(h @ w[p + "up"].to(F64).T)) ** 2)
    return stored(a @ w[p + "down"].to(F64).T)


def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return stored(gelu_erf(stored(h @ w[p + "up"].to(F64).T))) @ w[p + "down"].to(F64).T


def route(h: torch.Tensor, w_router: torch.Tensor, r: dict):
    """Per token: the chosen experts and their weights."""
    s = torch.sigmoid(h @ w_router.to(F64).T)                       # [T, E]
    T, E = s.shape
    ng, keep, top = r["groups"]["count"], r["groups"]["keep"], r["top"]
    per = E // ng
    gs = s.view(T, ng, per)
    gscore = gs.topk(min(2, per), dim=-1).values.sum(-1)            # [T, ng]
    kept = gscore.topk(keep, dim=-1).indices                        # [T, keep]
    allowed = torch.zeros(T, ng, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = torch.where(allowed.repeat_interleave(per, dim=1), s, torch.full_like(s, -1.0))
    choice = masked.topk(top, dim=-1).indices                       # [T, top]
    return choice, s.gather(1, choice)


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    choice, weight = route(h, w[p + "router"], mlp["router"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, c in zip(choice[t].tolist(), weight[t].tolist()):
            out[t] += c * expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + expert(h, w, p + "shared.")
    return stored(out)


# ------------------------------------------------------------------ the model

def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[list] = None
            ) -> torch.Tensor:
    """Logits [T, vocab] (float64) of a whole sequence; ``layers_out`` collects the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"].to(F64)[list(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = stored(layer_norm(x, w[p + "norm1"].to(F64), eps))
        if layer["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "lightning":
            y = lightning_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, w[p + "norm1b"].to(F64), eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = stored(layer_norm(x, w[p + "norm2"].to(F64), eps))
            y = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, w, p + "mlp.", mlp)
            x = x + layer_norm(y, w[p + "norm2b"].to(F64), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = stored(layer_norm(x, w["final.norm"].to(F64), eps))
    return h @ w["embed"].to(F64).T


# ------------------------------------------------------------------ weights and files

def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W = cfg["width"]
    out: Dict[str, tuple] = {"embed": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        for n in ("norm1", "norm1b"):
            out[p + n] = (W,)
        m = layer["mixer"]
        if layer["type"] == "attention":
            H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * 2 * D, W), p + "mix.q.b": (H * 2 * D,), p + "mix.k": (G * 2 * D, W),
                        p + "mix.k.b": (G * 2 * D,), p + "mix.v": (G * DV, W), p + "mix.v.b": (G * DV,),
                        p + "mix.o": (W, H * DV)})
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[p + "mix." + n] = (D,)
        else:
            H, D, DV = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * D, W), p + "mix.k": (H * D, W), p + "mix.v": (H * DV, W),
                        p + "mix.g": (H * DV, W), p + "mix.o": (W, H * DV), p + "mix.norm": (H * DV,)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        for n in ("norm2", "norm2b"):
            out[p + n] = (W,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            for e in range(mlp["router"]["experts"]):
                out.update({f"{p}mlp.e{e}.up": (mlp["expert"]["ff"], W), f"{p}mlp.e{e}.down": (W, mlp["expert"]["ff"])})
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            if mlp.get("shared"):
                out.update({p + "mlp.shared.up": (mlp["shared"]["ff"], W), p + "mlp.shared.down": (W, mlp["shared"]["ff"])})
    out["final.norm"] = (W,)
    return out


def random_weights(cfg: dict, seed: int, sharpen: float = 3.0) -> Dict[str, torch.Tensor]:
    """Seeded weights (float32 values that bfloat16 holds exactly): matrices N(0, 1/fan_in), q and k
    scaled up so that attention is not flat, router rows scaled so that scores spread, norm weights
    around 1, biases and the lambda vectors small."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if len(shape) == 2:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if leaf in ("q", "k") and ".mix." in name:
                t = t * sharpen
            if leaf == "router":
                t = t * 4.0
            if leaf == "embed":
                t = torch.randn(shape, generator=g)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = torch.randn(shape, generator=g) * 0.3
        elif leaf == "b":
            t = torch.randn(shape, generator=g) * 0.2
        else:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16).float()
    return out


_ST = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}


def write_model_dir(path: str, cfg: dict, weights: Dict[str, torch.Tensor], dtype=torch.bfloat16) -> None:
    """config.json and one model.safetensors (8-byte length, JSON header, data), written by hand."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, t in weights.items():
        t = t.to(dtype).contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
