"""Pufevik without a GPU: its configuration (keys, errors, round trip), the tensor names the model expects
against the plain implementation's own list, cache groups and states per layer, the random-weights writer,
and the plain implementation against closed forms of its own mechanisms (the matrix memory without its
stabiliser, carried across a cut; the sink; the rotation; the window)."""

import copy
import json
import math
import os

import pytest
import torch

import plain_pufevik as P
import pufevik_configs as C


def test_configuration_round_trip_and_registry(tmp_path):
    from redline_b200.config.model_config import PufevikConfig
    from redline_b200.config.registry import config_from_dict, load_config
    for name, cfg in C.ALL.items():
        c = config_from_dict(cfg)
        assert isinstance(c, PufevikConfig) and c.architecture == "Pufevik"
        assert c.vocab_size == cfg["vocab"] and c.hidden_size == cfg["width"] and c.norm_eps == cfg["norm"]["eps"]
        assert c.embedding_scale == cfg["embedding"]["scale"]
        assert c.to_hf()["layers"] == cfg["layers"], name
        c.save(str(tmp_path / name))
        assert load_config(str(tmp_path / name)) == c
    m = config_from_dict(C.MIX)
    assert m.layers[0].mixer.v_mix and not m.layers[4].mixer.v_mix and m.layers[2].ff == 0
    assert m.layers[1].mixer.left.window == 24 and m.layers[1].mixer.right.gate_cap == 12.0
    assert m.layers[3].mixer.left.rot.base == 100.0 and m.layers[6].mixer.right_scale == 1.7


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "conv"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 24), "v_mix"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "moe"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].__setitem__("eps", 0.0), "eps"),
])
def test_configuration_errors_name_the_key(edit, word):
    from redline_b200.config.model_config import ConfigError
    from redline_b200.config.registry import config_from_dict
    cfg = copy.deepcopy(C.MIX)
    edit(cfg)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


def _model(cfg):
    from redline_b200.config.registry import config_from_dict, model_spec
    from redline_b200.engine.model import DecoderModel
    from redline_b200.parts.base import Runtime
    rt = Runtime(device=torch.device("cpu"), dtype=torch.float32, max_tokens=8, max_seqs=2, max_seq_len=64, page_size=16)
    return DecoderModel(model_spec(config_from_dict(cfg)), rt)


@pytest.mark.parametrize("name", list(C.ALL))
def test_expected_tensors_are_the_plain_implementations(name):
    model = _model(C.ALL[name])
    exp = {n: tuple(s.shape) for n, s in model.expected_tensors().items()}
    assert exp == P.tensor_shapes(C.ALL[name])


def test_cache_groups_and_states_follow_the_layers():
    model = _model(C.MIX)
    groups = model.cache_groups()
    got = sorted((g.spec.kind, g.spec.window, tuple(t.shape for t in g.spec.tensors), tuple(g.owners)) for g in groups)
    assert got == sorted([
        ("full", 0, ((2, 32), (2, 16)), (0,)), ("window", 24, ((2, 16), (2, 32)), (1,)),
        ("full", 0, ((2, 48), (2, 16)), (2,)), ("window", 7, ((3, 32), (3, 16)), (3,)),
        ("full", 0, ((3, 16), (3, 48)), (4,)), ("full", 0, ((2, 16), (2, 16)), (5,)),
        ("window", 500, ((1, 64), (1, 64)), (6,))])
    # a pair's state: [heads, dim, vdim + 1] and a stabiliser per head
    assert {i: s.shape for i, s in model.state_specs().items()} == {
        1: (3 * 16 * 25 + 3,), 3: (32 * 65 + 1,), 6: (4 * 8 * 17 + 4,)}
    assert not _model(C.ATTN).state_specs()
    # which layer provides the shared values and which blend them in
    mixes = [b.mixer.params.value_mix for b in model.blocks if hasattr(b.mixer.params, "value_mix")]
    assert mixes == ["keep", "blend", "none", "blend"]
    # a model whose same layers recur shares groups
    cfg = C.clone(C.MEM)
    cfg["layers"][1]["mixer"]["left"] = copy.deepcopy(cfg["layers"][0]["mixer"]["left"])
    assert [g.owners for g in _model(cfg).cache_groups()] == [[0, 1]]


def test_random_weights_writer(tmp_path):
    from redline_b200.config.registry import config_from_dict
    from redline_b200.weights.random_init import write_random_model
    from redline_b200.weights.safetensors_io import CheckpointReader
    d = write_random_model(str(tmp_path / "m"), config_from_dict(C.MIX), seed=3)
    r = CheckpointReader(d)
    assert {n: tuple(r.info(n)[1]) for n in r.names()} == P.tensor_shapes(C.MIX)
    assert json.load(open(os.path.join(d, "config.json")))["architecture"] == "Pufevik"
    w = {n: r.tensor(n).float() for n in r.names()}
    assert torch.isfinite(P.forward(C.MIX, w, [1, 5, 9, 2])).all()
    cfg2, w2 = P.read_model_dir(d)                # the plain reader reads the framework's file
    assert cfg2["layers"] == C.MIX["layers"] and all(torch.equal(w[n], w2[n]) for n in w)


# ------------------------------------------------------------------ the plain implementation itself

def test_plain_memory_is_the_gated_sum():
    """Without the stabiliser, in double precision and with small gates: S_t = sum_s (prod_{s<r<=t} F_r) I_s k_s v_s^T,
    the denominator max(|n . q|, 1) e^m-free form: o = num / max(|den|, 1) when every quantity is rescaled by e^m."""
    g = torch.Generator().manual_seed(0)
    T, D, DV = 11, 4, 6
    q, k = torch.randn(T, D, generator=g, dtype=P.F64), torch.randn(T, D, generator=g, dtype=P.F64)
    v = torch.randn(T, DV, generator=g, dtype=P.F64)
    ig = torch.randn(T, generator=g, dtype=P.F64)
    fg = P.log_sigmoid(torch.randn(T, generator=g, dtype=P.F64) + 2.0)
    got = P.matrix_memory(q, k, v, ig, fg)
    for t in range(T):
        num, den = torch.zeros(DV, dtype=P.F64), 0.0
        for s in range(t + 1):
            wgt = math.exp(float(ig[s] + fg[s + 1:t + 1].sum()))
            num += wgt * float(k[s] @ q[t]) * v[s]
            den += wgt * float(k[s] @ q[t])
        # the stabilised form divides numerator and denominator by e^m; its floor exp(-m) is then 1
        m = 0.0
        for s in range(t + 1):
            m = max(float(fg[s]) + m, float(ig[s]))
        want = (num / math.exp(m)) / (max(abs(den) / math.exp(m), math.exp(-m)) + P.DENOMINATOR_FLOOR)
        assert torch.allclose(got[t], want, atol=1e-12), t


def test_plain_memory_carries_its_state_across_a_cut():
    g = torch.Generator().manual_seed(1)
    T, D, DV = 30, 3, 5
    q, k = torch.randn(T, D, generator=g, dtype=P.F64), torch.randn(T, D, generator=g, dtype=P.F64)
    v = torch.randn(T, DV, generator=g, dtype=P.F64)
    ig, fg = 3 * torch.randn(T, generator=g, dtype=P.F64), P.log_sigmoid(3 * torch.randn(T, generator=g, dtype=P.F64))
    whole = P.matrix_memory(q, k, v, ig, fg)
    state: dict = {}
    parts = [P.matrix_memory(q[a:b], k[a:b], v[a:b], ig[a:b], fg[a:b], state) for a, b in ((0, 7), (7, 9), (9, 10), (10, 30))]
    assert torch.allclose(torch.cat(parts), whole, atol=1e-13)
    # the stabiliser starts at 0, not at minus infinity: a first token with a very negative input gate
    first = P.matrix_memory(q[:1], k[:1], v[:1], torch.tensor([-9.0], dtype=P.F64), fg[:1])
    n_q = math.exp(-9.0) * float(k[0] @ q[0])
    want = math.exp(-9.0) * float(k[0] @ q[0]) * v[0] / (max(abs(n_q), 1.0) + P.DENOMINATOR_FLOOR)
    assert torch.allclose(first[0], want, atol=1e-15)


def test_plain_sink_window_and_groups():
    q = torch.zeros(5, 2, 4, dtype=P.F64)
    k = torch.zeros(5, 1, 4, dtype=P.F64)
    v = torch.arange(5, dtype=P.F64).view(5, 1, 1).expand(5, 1, 3).contiguous()
    # equal scores: the mean of the visible values, the sink taking its share of the weight
    o = P.softmax_attention(q, k, v, 1.0)
    assert torch.allclose(o[4, 0], torch.full((3,), 2.0, dtype=P.F64))
    o = P.softmax_attention(q, k, v, 1.0, window=2)
    assert torch.allclose(o[4, 1], torch.full((3,), 3.5, dtype=P.F64)) and torch.allclose(o[0, 0], torch.zeros(3, dtype=P.F64))
    sink = torch.tensor([0.0, math.log(2.0)], dtype=P.F64)
    o = P.softmax_attention(q, k, v, 1.0, window=2, sink=sink)
    assert torch.allclose(o[4, 0], torch.full((3,), 7.0 / 3.0, dtype=P.F64))      # weights 1/3, 1/3 and the sink's 1/3
    assert torch.allclose(o[4, 1], torch.full((3,), 7.0 / 4.0, dtype=P.F64))      # the sink counts twice
    assert torch.allclose(o[0, 1], torch.zeros(3, dtype=P.F64))


def test_plain_rotation_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1, 1, 12, generator=g, dtype=P.F64).expand(9, 1, 12).contiguous()
    y = torch.randn(1, 1, 12, generator=g, dtype=P.F64).expand(9, 1, 12).contiguous()
    rx, ry = P.rotate_pairs(x, 100.0, 8), P.rotate_pairs(y, 100.0, 8)
    assert torch.equal(rx[:, :, 8:], x[:, :, 8:]) and torch.allclose(rx[0], x[0])
    dots = torch.einsum("ihd,jhd->ij", rx, ry)
    for d in range(1, 5):
        assert torch.allclose(dots.diagonal(d), dots.diagonal(d)[0].expand(9 - d), atol=1e-12)
        assert torch.allclose(dots.diagonal(-d), dots.diagonal(-d)[0].expand(9 - d), atol=1e-12)
    # the pair (u, v) = (1, 0) at position p of pair 1 points at the angle p * base^(-2/8)
    e = torch.zeros(4, 1, 12, dtype=P.F64)
    e[:, 0, 2] = 1.0
    r = P.rotate_pairs(e, 100.0, 8)
    a = torch.arange(4, dtype=P.F64) * 100.0 ** (-2.0 / 8)
    assert torch.allclose(r[:, 0, 2], torch.cos(a)) and torch.allclose(r[:, 0, 3], torch.sin(a))
