"""Helpers of the Kapitar GPU tests: model folders, engines, comparisons with the plain implementation."""

from __future__ import annotations

import os
from typing import Dict, Optional, Sequence

import numpy as np
import torch

import plain_kapitar as K
from gpu_utils import F32_REL, rel_max


def make_model(tmp, cfg: dict, seed: int, sharpen: float = 3.0, patch=None):
    """Writes a model folder with seeded weights; returns (folder, weights as float32 values bfloat16 holds)."""
    w = K.random_weights(cfg, seed, sharpen)
    if patch is not None:
        patch(w)
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    d = os.path.join(str(tmp), f"kapitar_{seed}_{abs(hash(str(cfg))) % 10**8}")
    K.write_model_dir(d, cfg, w)
    return d, w


def engine_for(model_dir: str, dtype: str, **kw):
    from redline_b200.engine.engine import Engine
    opts = dict(dtype=dtype, kv_cache_tokens=1024, max_seq_len=1024, max_num_seqs=4, max_num_batched_tokens=512,
                max_logit_rows=512, cuda_graphs=False, async_scheduling=False)
    opts.update(kw)
    return Engine(model_dir, **opts)


def oracle(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], rounded: Optional[torch.dtype] = None) -> np.ndarray:
    K.STORE_DTYPE = rounded
    try:
        return K.forward(cfg, w, list(tokens)).numpy()
    finally:
        K.STORE_DTYPE = None


class Reference:
    """The plain implementation's logits of a sequence: exact (float64), and for a 16-bit engine also with
    everything rounded that such an engine stores in 16 bits."""

    def __init__(self, cfg: dict, w, tokens: Sequence[int], dtype: str):
        self.exact = oracle(cfg, w, tokens)
        self.rounded = oracle(cfg, w, tokens, torch.bfloat16) if dtype != "float32" else None
        self.main = self.exact if self.rounded is None else self.rounded


def row_rms(d: np.ndarray) -> np.ndarray:
    d = d - d.mean(axis=-1, keepdims=True)
    return np.sqrt((d * d).mean(axis=-1))


# A 16-bit engine against the exact logits: a row may be off by up to this many times what rounding alone
# does to the plain implementation on the same sequence (its worst row).  Faults of logic (a key one
# position off, a lost state) are tens of times larger, and the 32-bit runs hold them to 1e-4.
BF16_NOISE_FACTOR = 3.0


_model_noise: Dict[int, float] = {}


def model_noise(cfg: dict, w) -> float:
    """What rounding alone does to the plain implementation's logits on a 64-token sequence of this model
    (worst row): the floor under the level of a short sequence, whose own worst row is a poor estimate."""
    key = id(w)
    if key not in _model_noise:
        toks = np.random.RandomState(0).randint(0, cfg["vocab"], size=64).tolist()
        _model_noise[key] = float(row_rms(oracle(cfg, w, toks, torch.bfloat16) - oracle(cfg, w, toks)).max())
    return _model_noise[key]


def check(got: np.ndarray, cfg: dict, w, tokens: Sequence[int], dtype: str, rows=None, ref: Optional[Reference] = None) -> float:
    """float32: rel-max against the exact logits below 1e-4.  bfloat16: every row's error (root mean square,
    mean removed) against the exact logits within BF16_NOISE_FACTOR times the rounding error of the plain
    implementation itself."""
    rows = list(range(len(tokens))) if rows is None else list(rows)
    ref = ref or Reference(cfg, w, tokens, dtype)
    if dtype == "float32":
        want = ref.exact[rows]
        err = rel_max(got, want)
        assert err < F32_REL, (f"float32 logits differ: rel-max {err:.3e}, worst row "
                               f"{rows[int(np.abs(got - want).max(axis=1).argmax())]}")
        return err
    level = max(float(row_rms(ref.rounded - ref.exact).max()), model_noise(cfg, w))
    err = row_rms(got - ref.exact[rows])
    worst = int(err.argmax())
    assert err[worst] <= BF16_NOISE_FACTOR * level, (f"bfloat16 logits differ: row {rows[worst]} is off by {err[worst]:.3e}, "
                                                     f"rounding alone gives {level:.3e}")
    return float(err[worst] / level)
