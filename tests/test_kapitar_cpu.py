"""Kapitar without a GPU: its configuration (keys, errors, round trip, the registry's singular key), the
tensor names the model expects against the plain implementation's own list, the random-weights writer,
window groups that keep the pages of their first tokens, and the plain implementation against closed
forms of its own mechanisms."""

import copy
import json
import os

import pytest
import torch

import kapitar_configs as C
import plain_kapitar as K


def test_configuration_round_trip_and_registry(tmp_path):
    from redline_b200.config.model_config import KapitarConfig
    from redline_b200.config.registry import config_from_dict, load_config
    for name, cfg in C.ALL.items():
        c = config_from_dict(cfg)
        assert isinstance(c, KapitarConfig) and c.architecture == "Kapitar"
        assert c.vocab_size == cfg["vocab"] and c.hidden_size == cfg["width"] and c.norm_eps == cfg["norm"]["eps"]
        assert c.to_hf()["layers"] == cfg["layers"], name
        c.save(str(tmp_path / name))
        assert load_config(str(tmp_path / name)) == c
    m = config_from_dict(C.MIX)
    assert m.layers[0].mixer.mask.keep_first == 3 and m.layers[2].mlp is None
    assert m.layers[1].mlp.groups == 4 and m.layers[1].mlp.groups_keep == 2 and m.layers[1].mlp.shared_ff == 56
    assert m.layers[4].mlp.shared_ff == 0 and m.layers[3].mixer.decay == (0.97,)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "conv"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5]), "decays"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("experts", 7), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 5), "top"),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), "mask"),
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
    assert exp == K.tensor_shapes(C.ALL[name])


def test_cache_groups_and_states_follow_the_layers():
    model = _model(C.MIX)
    groups = model.cache_groups()
    assert [(g.spec.kind, g.spec.window, g.spec.keep_first, g.owners) for g in groups] == [
        ("window", 24, 3, [0]), ("window", 7, 0, [2]), ("window", 500, 5, [4])]
    assert [t.shape for t in groups[0].spec.tensors] == [(4, 16), (2, 32)]       # two maps of keys, one of values
    assert {i: s.shape for i, s in model.state_specs().items()} == {1: (3, 16, 24), 3: (1, 32, 64)}
    assert not _model(C.LIGHT).cache_groups() and not _model(C.ATTN).state_specs()


def test_random_weights_writer(tmp_path):
    from redline_b200.config.registry import config_from_dict
    from redline_b200.weights.random_init import write_random_model
    from redline_b200.weights.safetensors_io import CheckpointReader
    d = write_random_model(str(tmp_path / "m"), config_from_dict(C.MIX), seed=3)
    r = CheckpointReader(d)
    assert {n: tuple(r.info(n)[1]) for n in r.names()} == K.tensor_shapes(C.MIX)
    assert json.load(open(os.path.join(d, "config.json")))["architecture"] == "Kapitar"
    # the plain implementation runs on them
    w = {n: r.tensor(n).float() for n in r.names()}
    assert torch.isfinite(K.forward(C.MIX, w, [1, 5, 9, 2])).all()


def test_window_groups_keep_the_pages_of_their_first_tokens():
    from redline_b200.cache.manager import CacheManager, GroupInfo
    from redline_b200.parts.spec import CacheSpec, CacheTensor
    t = (CacheTensor("k", (1, 8)),)
    groups = [GroupInfo(CacheSpec("window", t, 24, 20), [0]), GroupInfo(CacheSpec("window", t, 24, 0), [1]),
              GroupInfo(CacheSpec("full", t), [2])]
    m = CacheManager(groups, [40, 40, 40], 16, 2)
    rc = m.open("a")
    assert m.reserve(rc, 200)
    first = [rc.table(g)[:2] for g in range(3)]
    m.release_passed(rc, 200)                       # keys 0 .. 176 are behind every window
    tabs = rc.tables
    assert tabs[0][:2] == first[0] and all(p == 0 for p in tabs[0][2:11]) and all(p > 0 for p in tabs[0][11:])
    assert all(p == 0 for p in tabs[1][:11]) and all(p > 0 for p in tabs[1][11:])
    assert all(p > 0 for p in tabs[2])
    m.check_invariants()
    assert m.num_free_pages(0) == 39 - 13 + 9 and m.num_free_pages(1) == 39 - 13 + 11 and m.num_free_pages(2) == 39 - 13
    # a short sequence whose window never leaves the kept blocks releases nothing
    rb = m.open("b")
    assert m.reserve(rb, 30)
    assert m.release_passed(rb, 30) == 0
    m.check_invariants()
    m.close("a")
    m.close("b")
    m.check_invariants()
    assert [m.num_free_pages(g) for g in range(3)] == [39, 39, 39]
    # pages come back in use by the next request
    rc = m.open("c")
    assert m.reserve(rc, 39 * 16) and not m.reserve(rc, 40 * 16)
    m.close("c")


def test_plain_recurrence_is_the_decayed_sum():
    g = torch.Generator().manual_seed(0)
    cfg = {"heads": 2, "dim": 4, "vdim": 6, "decay": [0.7, 0.95]}
    W = 10
    w = {"q": torch.randn(8, W, generator=g), "k": torch.randn(8, W, generator=g), "v": torch.randn(12, W, generator=g),
         "g": torch.randn(12, W, generator=g), "o": torch.eye(12), "norm": torch.ones(12)}
    h = torch.randn(9, W, generator=g, dtype=torch.float64)
    got = K.lightning_mixer(h, w, "", cfg, 1e-6)
    q, k, v = (K.silu(h @ w[n].double().T) for n in "qkv")
    o = torch.zeros(9, 12, dtype=torch.float64)
    for t in range(9):
        for hd, d in enumerate(cfg["decay"]):
            for s in range(t + 1):
                o[t, hd * 6:(hd + 1) * 6] += d ** (t - s) * (q[t, hd * 4:(hd + 1) * 4] @ k[s, hd * 4:(hd + 1) * 4]) * v[s, hd * 6:(hd + 1) * 6]
    want = K.unit_rms(o, 1e-6) * torch.sigmoid(h @ w["g"].double().T)
    assert torch.allclose(got, want, atol=1e-12)


def test_plain_router_keeps_groups_by_their_two_best():
    s = torch.tensor([[0.9, 0.15, 0.1, 0.1, 0.6, 0.6, 0.1, 0.1, 0.5, 0.5, 0.5, 0.5]], dtype=torch.float64)
    z = torch.log(s / (1 - s))
    r = {"groups": {"count": 3, "keep": 1}, "top": 2}
    choice, weight = K.route(torch.eye(12, dtype=torch.float64)[:1] * 0 + z, torch.eye(12), r)
    # group sums of the two best: 1.05, 1.2, 1.0 -> the middle group, although the best expert is elsewhere
    assert sorted(choice[0].tolist()) == [4, 5] and torch.allclose(weight, torch.tensor([[0.6, 0.6]], dtype=torch.float64))
    r = {"groups": {"count": 3, "keep": 2}, "top": 3}
    choice, weight = K.route(z, torch.eye(12), r)
    assert sorted(choice[0].tolist()) == [0, 4, 5]


def test_plain_mask():
    assert K.visible(10, 10, 1, 0) and not K.visible(10, 9, 1, 0) and not K.visible(3, 4, 9, 9)
    assert K.visible(30, 7, 24, 0) and not K.visible(31, 7, 24, 0) and K.visible(31, 2, 24, 3) and not K.visible(31, 3, 24, 3)
