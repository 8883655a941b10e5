"""Plain, slow implementation of the Pufevik decoder: the oracle of its tests.

Whole sequences, no cache, no batching, float64, one function per mechanism.  It shares no code with
``redline_b200``: it reads the configuration dictionary itself, draws its own random weights and writes
its own safetensors file.

The model in this file's notation (x_t is the stream at token t, W applied as W x, h = x_t):

  embedding:  x = table[token] * embedding.scale
  layer:      x += N_1(mixer(x));  x += N_2(ff(x))       N = RMS norm with a weight; the sublayers read x itself
  attention:  grouped-query heads; q and k are RMS-normed per head (one weight of the head's size for all
              heads), then the first rot.dims entries of every head are rotated in neighbouring pairs
              (2i, 2i+1) by the angle pos * base^(-2i / rot.dims); s = scale * (q . k); causal softmax;
              in layers with v_mix other than the first such layer, v <- (1 - lam) v + lam v_first, v_first
              the first such layer's values of the same token; the joined heads are multiplied by
              sigmoid(W_g h) element by element; output projection
  parallel:   left_scale * left(h) + right_scale * right(h)
    left:     attention whose q and k are RMS-normed over the whole projection (all heads at once, weights of
              that size), rotated as above, seen through a sliding window (i sees j when 0 <= i - j < size),
              with exp(sink_h) added to the softmax's denominator; head h's output is multiplied by
              sigmoid(W_g h)_h (one number per head); output projection
    right:    a matrix memory per head: q = W_q h / sqrt(dim), k = W_k h, v = W_v h;
              i = cap * tanh((W_i h + b_i) / cap), f = logsigmoid(cap * tanh((W_f h + b_f) / cap));
              m_t = max(f + m_(t-1), i) with m_0 = 0;
              S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T, n_t the same with k alone;
              o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6); every head's o is divided by its root mean
              square, the joined heads multiplied by a weight and by sigmoid(W_g h); output projection
  dense ff:   W_down (gelu_tanh(W_gate h) * (W_up h))
  output:     N_final, logits = head x
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
DENOMINATOR_FLOOR = 1e-6        # added to the matrix memory's denominator

# When set to a 16-bit type, what a 16-bit engine stores in that type is rounded here as well (the
# sublayers' inputs, projections and activations, cached keys and values, mixer and feed-forward
# outputs); the stream, scores, states, gates of the recurrence and the norms' arithmetic stay double.
STORE_DTYPE: Optional[torch.dtype] = None


def stored(x: torch.Tensor) -> torch.Tensor:
    return x if STORE_DTYPE is None else x.to(STORE_DTYPE).to(F64)


# ------------------------------------------------------------------ small pieces

def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -(torch.clamp(-z, min=0.0) + torch.log1p(torch.exp(-z.abs())))


def rotate_pairs(x: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [tokens, heads, size]: entries (2i, 2i+1), i < dims / 2, of every head turn by pos * base^(-2i/dims)."""
    T = x.shape[0]
    out = x.clone()
    pos = torch.arange(T, dtype=F64)
    for i in range(dims // 2):
        a = pos * (base ** (-2.0 * i / dims))
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0,
                      sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, DV] -> [T, H, DV].  Token i sees j <= i, and with a window only
    i - j < window; ``sink`` [H] adds exp(sink_h) to head h's denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if window <= 0 else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            mx = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - mx)
            den = e.sum() if sink is None else e.sum() + torch.exp(sink[h] - mx)
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


# ------------------------------------------------------------------ mixers

def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                    shared: dict) -> torch.Tensor:
    """``shared`` carries the first value-mixing layer's values to the later ones."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    q = stored(h @ w[p + "q"].T).view(T, H, D)
    k = stored(h @ w[p + "k"].T).view(T, G, D)
    v = stored(h @ w[p + "v"].T).view(T, G, DV)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q, k = rotate_pairs(q, rot["base"], rot["dims"]), rotate_pairs(k, rot["base"], rot["dims"])
    if m.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v
        else:
            lam = w[p + "vmix"].reshape(())
            v = (1.0 - lam) * v + lam * shared["v_first"]
    o = softmax_attention(stored(q), stored(k), stored(v), m["scale"])
    gate = sigmoid(stored(h @ w[p + "g"].T))
    return stored(stored(o.reshape(T, H * DV) * gate) @ w[p + "o"].T)


def window_sink_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, DV = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    q = rms_norm(stored(h @ w[p + "q"].T), w[p + "q.norm"], eps).view(T, H, D)
    k = rms_norm(stored(h @ w[p + "k"].T), w[p + "k.norm"], eps).view(T, G, D)
    v = stored(h @ w[p + "v"].T).view(T, G, DV)
    rot = m.get("rot")
    if rot:
        q, k = rotate_pairs(q, rot["base"], rot["dims"]), rotate_pairs(k, rot["base"], rot["dims"])
    o = softmax_attention(stored(q), stored(k), v, m["scale"], window=m["mask"]["size"], sink=w[p + "sink"])
    gate = sigmoid(stored(h @ w[p + "g"].T))                     # [T, H]
    return stored(stored((o * gate[:, :, None]).reshape(T, H * DV)) @ w[p + "o"].T)


def matrix_memory(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ig: torch.Tensor, fg: torch.Tensor,
                  state: Optional[dict] = None) -> torch.Tensor:
    """One head.  q (already scaled), k [T, D]; v [T, DV]; ig, fg [T] the logarithms of the input and forget
    gates.  ``state`` (S, n, m) is read and left behind if given; the start is S = 0, n = 0, m = 0."""
    T, D = q.shape
    DV = v.shape[1]
    S = torch.zeros(D, DV, dtype=F64) if state is None or "S" not in state else state["S"]
    n = torch.zeros(D, dtype=F64) if state is None or "n" not in state else state["n"]
    m = 0.0 if state is None or "m" not in state else state["m"]
    out = torch.zeros(T, DV, dtype=F64)
    for t in range(T):
        m_new = max(float(fg[t]) + m, float(ig[t]))
        a, b = math.exp(float(fg[t]) + m - m_new), math.exp(float(ig[t]) - m_new)
        S = a * S + b * torch.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        den = max(abs(float(n @ q[t])), math.exp(-m)) + DENOMINATOR_FLOOR
        out[t] = (S.T @ q[t]) / den
    if state is not None:
        state.update(S=S, n=n, m=m)
    return out


def memory_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, DV, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = stored(h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = stored(h @ w[p + "k"].T).view(T, H, D)
    v = stored(h @ w[p + "v"].T).view(T, H, DV)
    ig = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    fg = log_sigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    o = torch.stack([matrix_memory(q[:, a], k[:, a], v[:, a], ig[:, a], fg[:, a]) for a in range(H)], dim=1)
    o = rms_norm(o, None, eps).reshape(T, H * DV) * w[p + "norm"]
    return stored(stored(o * sigmoid(stored(h @ w[p + "g"].T))) @ w[p + "o"].T)


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    return (m["left_scale"] * window_sink_mixer(h, w, p + "left.", m["left"], eps)
            + m["right_scale"] * memory_mixer(h, w, p + "right.", m["right"], eps))


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    a = stored(gelu_tanh(stored(h @ w[p + "gate"].T)) * stored(h @ w[p + "up"].T))
    return stored(a @ w[p + "down"].T)


# ------------------------------------------------------------------ the model

def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[list] = None
            ) -> torch.Tensor:
    """Logits [tokens, vocab] (float64) of one whole sequence.  ``layers_out`` receives the stream after every
    layer."""
    w = {k: v.to(F64) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)] * cfg["embedding"]["scale"]
    shared: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = stored(x)
        if layer["type"] == "attention":
            a = attention_mixer(h, w, p + "mix.", layer["mixer"], eps, shared)
        elif layer["type"] == "parallel":
            a = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"layer type {layer['type']}")
        x = x + rms_norm(a, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(dense_ff(stored(x), w, p + "mlp."), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return stored(rms_norm(x, w["final.norm"], eps)) @ w["head"].T


# ------------------------------------------------------------------ weights and files

def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W = cfg["width"]
    out: Dict[str, tuple] = {"embed": (cfg["vocab"], W)}

    def softmax_heads(p: str, m: dict, whole_norm: bool, gate_rows: int) -> None:
        H, G, D, DV = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
        out.update({p + "q": (H * D, W), p + "k": (G * D, W), p + "v": (G * DV, W),
                    p + "q.norm": (H * D if whole_norm else D,), p + "k.norm": (G * D if whole_norm else D,),
                    p + "g": (gate_rows, W), p + "o": (W, H * DV)})

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        out[p + "norm1"] = (W,)
        m = layer["mixer"]
        if layer["type"] == "attention":
            softmax_heads(p + "mix.", m, False, m["heads"] * m["vdim"])
            if m.get("v_mix"):
                out[p + "mix.vmix"] = ()          # (the first such layer has the number too and does not use it)
        else:
            l, r = m["left"], m["right"]
            softmax_heads(p + "mix.left.", l, True, l["heads"])
            out[p + "mix.left.sink"] = (l["heads"],)
            H, D, DV = r["heads"], r["dim"], r["vdim"]
            q = p + "mix.right."
            out.update({q + "q": (H * D, W), q + "k": (H * D, W), q + "v": (H * DV, W), q + "g": (H * DV, W),
                        q + "o": (W, H * DV), q + "norm": (H * DV,), q + "i": (H, W), q + "i.b": (H,),
                        q + "f": (H, W), q + "f.b": (H,)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            out.update({p + "norm2": (W,), p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    out["final.norm"] = (W,)
    out["head"] = (cfg["vocab"], W)
    return out


def random_weights(cfg: dict, seed: int, sharpen: float = 2.0) -> Dict[str, torch.Tensor]:
    """Seeded weights as the float32 values that bfloat16 holds.  Matrices N(0, 1 / fan_in), query and key
    projections ``sharpen`` times larger in their norms' weights so that attention is not flat, norm weights
    around 1, sinks, biases and mixing numbers of moderate size."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith(("q.norm", "k.norm")):
            t = math.sqrt(sharpen) * (1.0 + 0.1 * torch.randn(shape, generator=g))
        elif last in ("norm1", "norm2") or name.endswith(("final.norm", "right.norm")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last == "sink":
            t = torch.randn(shape, generator=g)
        elif last == "vmix":
            t = 0.2 + 0.5 * torch.rand(shape, generator=g)
        elif name.endswith("i.b"):
            t = torch.randn(shape, generator=g)
        elif name.endswith("f.b"):
            t = 2.0 + torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).float()
    return out


def write_model_dir(path: str, cfg: dict, weights: Dict[str, torch.Tensor], dtype=torch.bfloat16) -> None:
    """config.json and model.safetensors (8-byte length, JSON header, raw data), written by hand."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    code = {torch.bfloat16: "BF16", torch.float32: "F32"}[dtype]
    header, blobs, off = {}, [], 0
    for name, t in weights.items():
        raw = t.to(dtype).contiguous()
        data = raw.view(torch.uint8).numpy().tobytes() if raw.dim() > 0 else raw.reshape(1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": code, "shape": list(t.shape), "data_offsets": [off, off + len(data)]}
        blobs.append(data)
        off += len(data)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def read_model_dir(path: str):
    """(cfg, weights as float32) of a folder written by ``write_model_dir`` or any file of that format."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        buf = bytearray(data[a:b])
        if e["dtype"] == "BF16":
            t = torch.frombuffer(buf, dtype=torch.bfloat16).float()
        elif e["dtype"] == "F32":
            t = torch.frombuffer(buf, dtype=torch.float32).clone()
        elif e["dtype"] == "I32":
            t = torch.frombuffer(buf, dtype=torch.int32).clone()
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = t.reshape(e["shape"])
    return cfg, out
