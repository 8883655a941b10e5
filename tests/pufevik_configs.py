"""The Pufevik tests' own small configurations (config.json dictionaries).

MIX has every mechanism with sizes that differ from layer to layer: grouped and ungrouped heads, key and
value sizes that are equal or not, a rotation of all of a head, of a part of it and of two entries only,
windows shorter and longer than the test sequences and a window of one token, three layers that share
values (of one shape; the first provides them) beside an attention layer that does not, a layer without a feed-forward,
a single-head matrix memory, scales of the two sides that are 1 or not, a model that begins with an
attention layer.  ODD has sizes that are multiples of neither 8 nor 16 (no 16-byte pieces, no tensor-core
tiles).  ATTN has attention layers only (no state), MEM one pair whose window is a single token, so that
nearly everything comes through the memory.
"""

import copy


def attention(heads, kv_heads, dim, vdim, rot_dims, base=10000.0, v_mix=False, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "v_mix": v_mix,
            "scale": scale if scale is not None else dim ** -0.5, "rot": {"base": base, "dims": rot_dims}}


def windowed(heads, kv_heads, dim, vdim, rot_dims, size, base=200000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size},
            "scale": scale if scale is not None else dim ** -0.5, "rot": {"base": base, "dims": rot_dims}}


def memory(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def pair(left, right, left_scale, right_scale):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


def dense(ff):
    return {"kind": "dense", "ff": ff}


MIX = {
    "architecture": "Pufevik", "vocab": 149, "width": 96, "norm": {"eps": 3e-6}, "embedding": {"scale": 0.7},
    "layers": [
        {"type": "attention", "mixer": attention(4, 2, 32, 16, 32, v_mix=True, scale=0.3), "mlp": dense(160)},
        {"type": "parallel", "mixer": pair(windowed(4, 2, 16, 32, 8, 24), memory(3, 16, 24, 12.0), 0.9, 0.4), "mlp": dense(72)},
        {"type": "attention", "mixer": attention(2, 2, 48, 16, 2, base=500.0, v_mix=True), "mlp": None},
        {"type": "parallel", "mixer": pair(windowed(3, 3, 32, 16, 32, 7, base=100.0), memory(1, 32, 64, 4.0), 1.0, 1.0), "mlp": dense(64)},
        {"type": "attention", "mixer": attention(3, 3, 16, 48, 8, v_mix=False), "mlp": dense(40)},
        {"type": "attention", "mixer": attention(8, 2, 16, 16, 16, v_mix=True), "mlp": dense(200)},
        {"type": "parallel", "mixer": pair(windowed(2, 1, 64, 64, 16, 500), memory(4, 8, 16, 30.0), 0.3, 1.7), "mlp": None},
    ],
}

ODD = {
    "architecture": "Pufevik", "vocab": 61, "width": 100, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "layers": [
        {"type": "parallel", "mixer": pair(windowed(3, 1, 20, 12, 6, 11), memory(2, 10, 20, 8.0), 1.2, 0.6), "mlp": dense(28)},
        {"type": "attention", "mixer": attention(2, 2, 10, 6, 10, v_mix=True), "mlp": dense(36)},
        {"type": "attention", "mixer": attention(4, 2, 13, 6, 4, v_mix=True), "mlp": None},
    ],
}

ATTN = {
    "architecture": "Pufevik", "vocab": 101, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.6},
    "layers": [
        {"type": "attention", "mixer": attention(4, 2, 16, 16, 8, v_mix=False), "mlp": dense(96)},
        {"type": "attention", "mixer": attention(2, 2, 32, 32, 32, v_mix=True), "mlp": dense(96)},
        {"type": "attention", "mixer": attention(4, 2, 16, 32, 4, v_mix=True), "mlp": None},
    ],
}

MEM = {
    "architecture": "Pufevik", "vocab": 83, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
    "layers": [
        {"type": "parallel", "mixer": pair(windowed(2, 2, 16, 16, 8, 1), memory(2, 32, 40, 10.0), 0.2, 1.0), "mlp": dense(96)},
        {"type": "parallel", "mixer": pair(windowed(2, 1, 16, 16, 8, 1), memory(4, 16, 16, 20.0), 0.2, 1.0), "mlp": None},
    ],
}

ALL = {"mix": MIX, "odd": ODD, "attn": ATTN, "mem": MEM}


def one_windowed_layer(size, heads=2, kv_heads=1, dim=32, vdim=32, rot_dims=8):
    """One pair whose memory side is switched off by its scale: what the window shows decides the logits."""
    return {"architecture": "Pufevik", "vocab": 67, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": [{"type": "parallel", "mlp": None,
                        "mixer": pair(windowed(heads, kv_heads, dim, vdim, rot_dims, size), memory(1, 8, 8, 9.0), 1.0, 0.0)}]}


def one_attention_layer(heads=4, kv_heads=2, dim=16, vdim=48, rot_dims=4):
    return {"architecture": "Pufevik", "vocab": 67, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": [{"type": "attention", "mlp": None, "mixer": attention(heads, kv_heads, dim, vdim, rot_dims)}]}


def clone(cfg):
    return copy.deepcopy(cfg)


def random_config(seed, big=False):
    """A configuration drawn from a seed: two to five layers of either kind with sizes of their own (``big``: head
    sizes of 128 to 256), windows from one token to longer than the test sequences, layers with and without a
    feed-forward; the layers that share values have one value shape."""
    import random
    rng = random.Random(seed)
    width = rng.choice([256, 320] if big else [64, 96, 128, 160])
    shared = None

    def heads(window):
        kv = rng.choice([1, 2, 3])
        dim = rng.choice([128, 192, 256] if big else [16, 24, 32, 48, 64, 80])
        m = {"heads": kv * rng.choice([1, 2, 4]), "kv_heads": kv, "dim": dim,
             "vdim": rng.choice([128, 176, 256] if big else [8, 16, 24, 40, 64, 96]),
             "scale": dim ** -0.5 * rng.choice([0.7, 1.0, 1.3]),
             "rot": {"base": rng.choice([100.0, 10000.0, 1e6]), "dims": max(2, rng.choice([2, dim // 4 * 2, dim // 2 * 2]))}}
        if window:
            m["mask"] = {"size": rng.choice([1, 3, 17, 64, 100, 300])}
        return m

    layers = []
    for _ in range(rng.randint(2, 5)):
        if rng.random() < 0.5:
            m = heads(False)
            m["v_mix"] = rng.random() < 0.7
            if m["v_mix"] and shared is None:
                shared = (m["kv_heads"], m["vdim"])
            elif m["v_mix"]:
                m["kv_heads"], m["vdim"] = shared
                m["heads"] = shared[0] * rng.choice([1, 2])
            layer = {"type": "attention", "mixer": m}
        else:
            right = memory(rng.choice([1, 2, 3, 5]), rng.choice([128, 256] if big else [8, 16, 32, 64]),
                           rng.choice([128, 256] if big else [8, 20, 48, 64, 130]), rng.choice([3.0, 10.0, 25.0]))
            layer = {"type": "parallel", "mixer": pair(heads(True), right, rng.choice([0.3, 1.0, 1.4]), rng.choice([0.5, 1.0, 2.0]))}
        layer["mlp"] = None if rng.random() < 0.25 else dense(rng.choice([40, 96, 200, 264]))
        layers.append(layer)
    return {"architecture": "Pufevik", "vocab": rng.choice([50, 131, 300]), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5])},
            "embedding": {"scale": rng.choice([0.4, 1.0, 2.0])}, "layers": layers}
