"""The Kapitar tests' own small configurations (config.json dictionaries).

MIX has every mechanism with sizes that differ from layer to layer: grouped and ungrouped attention
heads, key and value sizes that are equal or not, windows shorter and longer than the test sequences,
with and without kept first tokens, one or several expert groups with one or several kept, top 1 and
top 3, with and without a shared expert, a layer without a feed-forward, a single-head lightning
layer.  PLAIN is MIX without routed layers (for 16-bit comparisons, where a router's close call
between two experts would decide the result).  ATTN has attention layers only (no state: its decoding
runs as CUDA graphs), LIGHT lightning layers only (no cache).
"""

import copy


def attention(heads, kv_heads, dim, vdim, size, keep_first, softcap, diff, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "softcap": softcap,
            "scale": scale if scale is not None else dim ** -0.5, "mask": {"size": size, "keep_first": keep_first}}


def lightning(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, count, keep, ff, shared=0):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


MIX = {
    "architecture": "Kapitar", "vocab": 157, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": attention(4, 2, 16, 32, 24, 3, 12.0, 0.35, 0.3), "mlp": dense(160)},
        {"type": "lightning", "mixer": lightning(3, 16, 24, (0.5, 0.9, 0.99)), "mlp": moe(8, 3, 4, 2, 40, 56)},
        {"type": "attention", "mixer": attention(3, 3, 24, 16, 7, 0, 30.0, 0.8), "mlp": None},
        {"type": "lightning", "mixer": lightning(1, 32, 64, (0.97,)), "mlp": dense(64)},
        {"type": "attention", "mixer": attention(2, 1, 64, 64, 500, 5, 8.0, 0.5), "mlp": moe(6, 1, 1, 1, 32)},
    ],
}

PLAIN = copy.deepcopy(MIX)
PLAIN["layers"][1]["mlp"] = dense(72)
PLAIN["layers"][4]["mlp"] = dense(200)

ATTN = {
    "architecture": "Kapitar", "vocab": 131, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": attention(2, 2, 32, 32, 20, 2, 10.0, 0.6), "mlp": dense(128)},
        {"type": "attention", "mixer": attention(4, 1, 16, 48, 33, 0, 25.0, 0.2), "mlp": moe(4, 2, 2, 2, 24, 16)},
    ],
}

LIGHT = {
    "architecture": "Kapitar", "vocab": 90, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "lightning", "mixer": lightning(2, 24, 40, (0.8, 0.95)), "mlp": dense(96)},
        {"type": "lightning", "mixer": lightning(4, 8, 16, (0.3, 0.6, 0.9, 0.999)), "mlp": None},
    ],
}


# Sizes that are multiples of neither 8 nor 16: the kernels' 16-byte and tensor-core forms do not apply and
# their plain forms must take over (also in the products).
ODD = {
    "architecture": "Kapitar", "vocab": 77, "width": 100, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": attention(3, 1, 20, 12, 9, 2, 15.0, 0.25), "mlp": moe(6, 2, 3, 2, 28, 36)},
        {"type": "lightning", "mixer": lightning(2, 10, 20, (0.7, 0.98)), "mlp": dense(84)},
        {"type": "attention", "mixer": attention(2, 2, 8, 4, 300, 0, 50.0, 0.7), "mlp": None},
    ],
}
ODD_PLAIN = copy.deepcopy(ODD)
ODD_PLAIN["layers"][0]["mlp"] = dense(52)


def one_attention_layer(size, keep_first, heads=2, kv_heads=1, dim=32, vdim=32, softcap=40.0, diff=0.3, vocab=64, width=64):
    """A single attention layer without a feed-forward: what a position sees decides its logits."""
    return {"architecture": "Kapitar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": attention(heads, kv_heads, dim, vdim, size, keep_first, softcap, diff),
                        "mlp": None}]}


ALL = {"mix": MIX, "plain": PLAIN, "attn": ATTN, "light": LIGHT, "odd": ODD, "odd_plain": ODD_PLAIN}
