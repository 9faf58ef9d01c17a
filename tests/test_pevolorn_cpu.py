"""Pevolorn without a GPU: the configuration read from its own keys and back, the model description (blocks, parts,
tensor names, which layers share a cache, what the cache manager has to provide), and the plain implementation's
mechanisms on cases small enough to check by hand."""
import json
import math

import pytest
import torch

import plain_pevolorn as plain
from tiny_pevolorn import PEVOLORNS, make_folder, requests_for

from tiny_llm_infer_b200.config import ConfigError, config_from_dict, describe_model, load_config
from tiny_llm_infer_b200.config.pevolorn import PevolornConfig
from tiny_llm_infer_b200.models.model import Model, expected_tensors


@pytest.mark.parametrize("name", sorted(PEVOLORNS))
def test_config_round_trip(name, tmp_path):
    tiny = PEVOLORNS[name]
    folder = make_folder(tiny, tmp_path)
    raw = json.loads((folder / "config.json").read_text())
    assert raw["architecture"] == "Pevolorn"
    cfg = load_config(folder)
    assert isinstance(cfg, PevolornConfig) and cfg == tiny["cfg"]
    assert config_from_dict(cfg.to_dict()).to_dict() == raw


def test_description_blocks_and_caches():
    tiny = PEVOLORNS["V1"]
    desc = describe_model(tiny["cfg"])
    assert [l.block for l in desc.layers] == ["postnorm_mixer_ffn", "postnorm_pair_ffn", "postnorm_mixer",
                                              "postnorm_pair_ffn", "postnorm_mixer_ffn"]
    assert desc.layers[1].params == {"alpha": 2.0, "mixer_weights": (1.2, 0.9)} and desc.layers[0].params == {"alpha": 2.0}
    # the two borrowers read the first layer's cache and write nothing
    assert [(e.layer, e.cache, e.writes_cache) for e in desc.order] == [
        (0, 0, True), (1, (1, 2), True), (2, 0, False), (3, (4, 5), True), (4, 0, False)]
    names, _ = expected_tensors(desc)
    assert {"embed", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.dkv", "l0.mix.dkv.norm", "l0.mix.uk",
            "l0.mix.g", "l0.mlp.router", "l0.mlp.correction", "l0.mlp.e5.up", "l0.mlp.shared.down", "l1.mix.left.q.b",
            "l1.mix.left.o.b", "l1.mix.left.g", "l1.mix.right.in", "l1.mix.right.conv.b", "l1.mix.right.A_log",
            "l1.mix.right.D", "l2.mix.uk", "l2.norm1"} <= set(names)
    for absent in ("l2.mix.dkv", "l2.mix.dkv.norm", "l4.mix.dkv", "l2.norm2", "l2.mlp.router", "l1.mlp.shared.up",
                   "l0.mlp.e6.up", "l0.mix.dq", "l0.mix.sink", "lm_head.weight"):
        assert absent not in names, absent
    assert names["l0.mix.g"].shape == (4, 128) and names["l1.mix.left.g"].shape == (4, 128)
    assert names["l0.mlp.router"].shape == (8, 128) and names["l0.mlp.correction"].shape == (8,)
    assert names["l0.mix.q"].shape == (4 * 40, 128) and names["l0.mix.dkv"].shape == (64, 128)
    assert names["l1.mix.right.in"].shape == (2 * 32 + 2 * 16 + 4, 128) and names["l1.mix.right.conv"].shape == (64, 4)
    assert names["l3.mix.right.in"].shape == (2 * 48 + 2 * 2 * 32 + 2, 128)
    model = Model(desc, torch.float32, None)
    needs = model.cache_needs()
    assert sorted(needs) == [0, 1, 2, 4, 5]
    assert needs[0][0].planes == ((1, 64),) and needs[0][1] is None and needs[0][0].window is None
    assert needs[1][0].planes == ((2, 32), (2, 24)) and needs[2][0] is None
    assert needs[2][1].shape == (4 * 16 * 8 + 3 * 64,) and needs[5][1].shape == (2 * 32 * 24 + 1 * (48 + 128),)


def test_config_errors():
    raw = PEVOLORNS["V2"]["cfg"].to_dict()
    for path, value, text in ((("layers", 0, "type"), "window", "not a layer"),
                              (("layers", 1, "mixer", "rot", "dims"), 8, "rot.dims"),
                              (("layers", 0, "mixer", "left", "rot", "dims"), 7, "rot.dims"),
                              (("layers", 2, "mixer", "left", "kv_heads"), 2, "multiple of kv_heads"),
                              (("layers", 0, "mixer", "right", "groups"), 2, "multiple of groups"),
                              (("layers", 0, "mixer", "right", "norm_groups"), 4, "norm_groups"),
                              (("layers", 3, "mixer", "kv_from"), 0, "kv_from"),
                              (("layers", 3, "mixer", "kv_from"), 3, "kv_from"),
                              (("layers", 3, "mixer", "kv_rank"), 24, "must equal layer 1"),
                              (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups"),
                              (("layers", 1, "mlp", "router", "top"), 3, "router.top"),
                              (("layers", 1, "mlp", "kind"), "dense", "not 'moe'"),
                              (("norm", "eps"), 0.0, "norm.eps")):
        bad = json.loads(json.dumps(raw))
        at = bad
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=text):
            config_from_dict(bad)


def test_router_by_hand():
    """Six outputs, the last two identity experts, three groups of two of which two are kept, top 2.  The correction
    lifts expert 5 into the choice without changing its weight; group 0 holds the largest score and still loses
    its second expert to the rule that both choices come from kept groups only."""
    h = torch.eye(6, dtype=torch.float64)[:1]
    z = torch.tensor([2.0, 1.9, 0.0, 0.1, -1.0, 0.5], dtype=torch.float64)
    w = {"r.router": z.view(6, 1) * torch.ones(1, 6, dtype=torch.float64) * torch.eye(6, dtype=torch.float64)[0],
         "r.correction": torch.tensor([0.0, -0.5, 0.0, 0.0, 0.0, 0.4], dtype=torch.float64)}
    r = {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 2}}
    chosen, weights = plain.route(h, w, "r.", r)
    s = torch.softmax(z, 0)
    # choice scores: group 0 = max(s0, s1 - 0.5) = s0, group 1 = s3, group 2 = s5 + 0.4: groups 0 and 2 stay
    assert sorted(chosen[0].tolist()) == [0, 5]
    assert torch.allclose(weights[0].sort().values, torch.stack([s[5], s[0]]).sort().values)
    out = plain.mixture(h, {**w, "r.e0.up": torch.ones(3, 6, dtype=torch.float64), "r.e0.down": torch.ones(6, 3, dtype=torch.float64)},
                        "r.", {"router": r})
    # expert 0: relu(1)^2 summed over three units = 3 in every column; identity expert 5 returns h itself
    assert torch.allclose(out[0], s[0] * 3.0 + s[5] * h[0])
    margin = plain.router_margin(h, w, "r.", r)
    assert margin.shape == (1,) and margin[0] > 0


def test_rotation_convolution_and_state_space_by_hand():
    x = torch.arange(1.0, 7.0, dtype=torch.float64).view(1, 1, 6)
    out = plain.rotate_half(x.expand(2, 1, 6), torch.tensor([0, 3]), 100.0, 4)
    assert torch.equal(out[0], x[0])                                      # position 0 turns nothing
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert torch.allclose(out[1, 0], torch.tensor([1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                                                   3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1),
                                                   5.0, 6.0], dtype=torch.float64))
    seq = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    conv = plain.causal_conv(seq, torch.tensor([[0.5, 10.0]], dtype=torch.float64), torch.tensor([1.0], dtype=torch.float64))
    assert torch.allclose(conv[:, 0], torch.tensor([11.0, 21.5, 42.0], dtype=torch.float64))
    # one head, one state row, one column, no convolution to speak of (one tap of weight one, no bias), weights
    # chosen so that every factor can be followed: S_t = a_t S_(t-1) + dt_t B_t u_t, y_t = S_t C_t + D u_t
    m = dict(heads=1, vdim=1, state=1, groups=1, conv=1, norm_groups=1)
    w = {"s.in": torch.tensor([[0.0, 1.0], [1.0, 0.0], [1.0, 0.0], [1.0, 0.0], [0.0, 0.0]], dtype=torch.float64),
         "s.conv": torch.ones(3, 1, dtype=torch.float64), "s.conv.b": torch.zeros(3, dtype=torch.float64),
         "s.dt_bias": torch.tensor([0.3], dtype=torch.float64), "s.A_log": torch.tensor([-1.0], dtype=torch.float64),
         "s.D": torch.tensor([0.5], dtype=torch.float64), "s.norm": torch.ones(1, dtype=torch.float64),
         "s.o": torch.ones(1, 1, dtype=torch.float64)}
    xs = torch.tensor([[1.0, 2.0], [-0.5, 1.0]], dtype=torch.float64)
    got = plain.state_space(xs, w, "s.", m, 1e-12)
    dt = math.log1p(math.exp(0.3))
    silu = lambda v: v / (1 + math.exp(-v))
    u0, u1 = silu(1.0), silu(-0.5)
    S0 = dt * u0 * u0
    y0 = (S0 * u0 + 0.5 * u0) * silu(2.0)
    S1 = math.exp(-math.exp(-1.0) * dt) * S0 + dt * u1 * u1
    y1 = (S1 * u1 + 0.5 * u1) * silu(1.0)
    assert torch.allclose(got[:, 0], torch.tensor([y0 / abs(y0), y1 / abs(y1)], dtype=torch.float64), atol=1e-9)


@pytest.mark.parametrize("name", sorted(PEVOLORNS))
def test_a_missing_mechanism_would_show(name, tmp_path):
    """The weights of the tiny models make every mechanism matter: the plain implementation with another residual
    factor, rotation, cap, scale or mixing weight, without the correction, the groups, the identity experts, the
    biases, the gates or the convolution's bias, with the borrowed cache replaced by the layer's own input, or
    without the first tokens moves the logits far beyond the tolerances of the comparisons with the engine."""
    import numpy as np
    from tiny_llm_infer_b200.weights.safetensors_io import SafetensorsFile
    tiny = PEVOLORNS[name]
    folder = make_folder(tiny, tmp_path)
    cfg = json.loads((folder / "config.json").read_text())
    f = SafetensorsFile(folder / "model.safetensors")
    w = {n: f.read(n).clone() for n in f.tensors}
    f.close()
    toks = max(requests_for(tiny).values(), key=len)[:120]
    ref = plain.forward(cfg, w, toks).numpy()

    def moved(changed_cfg=None, changed_w=None, tokens=None):
        got = plain.forward(changed_cfg or cfg, changed_w or w, tokens or toks).numpy()
        d = got[-40:] - ref[-40:]
        return float((np.sqrt(((d - d.mean(1, keepdims=True)) ** 2).mean(1)) / ref[-40:].std(1)).max())

    def with_weights(fn):
        return {k: fn(k, v) for k, v in w.items()}

    def with_layers(fn):
        c = json.loads(json.dumps(cfg))
        for layer in c["layers"]:
            fn(layer)
        return c

    def set_(d, path, f_):
        for key in path[:-1]:
            d = d.get(key) or {}
        if d.get(path[-1]) is not None:
            d[path[-1]] = f_(d[path[-1]])

    floor = 2e-3
    for suffix in (".correction", ".q.b", ".k.b", ".v.b", ".o.b", ".conv.b", ".dt_bias", ".D", ".g", "mix.right.norm"):
        assert moved(changed_w=with_weights(lambda k, v: torch.zeros_like(v) if k.endswith(suffix) else v)) > floor, suffix
    for path, f_ in ((("mixer", "rot", "base"), lambda v: v / 50), (("mixer", "scale"), lambda v: v * 1.5),
                     (("mixer", "left", "rot", "base"), lambda v: v * 2), (("mixer", "left", "rot", "dims"), lambda v: v - 2),
                     (("mixer", "left", "softcap"), lambda v: v * 0.3), (("mixer", "left", "scale"), lambda v: v * 1.5),
                     (("mixer", "left_scale"), lambda v: v + 0.3), (("mixer", "right_scale"), lambda v: v + 0.3),
                     (("mixer", "right", "norm_groups"), lambda v: 1 if v > 1 else v),
                     (("mlp", "router", "groups"), lambda g: {"count": g["count"], "keep": g["count"]})):
        changed = with_layers(lambda layer: set_(layer, path, f_))
        if changed != cfg:
            assert moved(changed_cfg=changed) > floor, path
    changed = json.loads(json.dumps(cfg))
    changed["postln_alpha"] = cfg["postln_alpha"] * 1.5
    assert moved(changed_cfg=changed) > floor
    assert moved(tokens=toks[40:]) > floor                       # the first forty tokens forgotten
