"""Tetodra without a GPU: the configuration read from its own keys and back, the sizes that only the checkpoint's
shapes give, the model description (blocks, parts, tensor names, what the cache manager has to provide), and the
table of distance buckets against the plain implementation's formula."""
import json

import pytest
import torch

import plain_tetodra as plain
from tiny_tetodra import TETODRAS, make_folder

from tiny_llm_infer_b200.config import ConfigError, config_from_dict, describe_model, load_config
from tiny_llm_infer_b200.config.tetodra import TetodraConfig
from tiny_llm_infer_b200.models.model import Model, expected_tensors
from tiny_llm_infer_b200.parts.attention_biased import distance_buckets


@pytest.mark.parametrize("name", sorted(TETODRAS))
def test_config_round_trip_and_sizes_from_the_checkpoint(name, tmp_path):
    tiny = TETODRAS[name]
    folder = make_folder(tiny, tmp_path)
    raw = json.loads((folder / "config.json").read_text())
    assert raw["architecture"] == "Tetodra" and "bias_rows" not in json.dumps(raw) and "decay_rank" not in json.dumps(raw)
    cfg = load_config(folder)
    assert isinstance(cfg, TetodraConfig) and cfg == tiny["cfg"]          # rows and ranks came back from the shapes
    assert config_from_dict(cfg.to_dict()).to_dict() == raw


def test_description_blocks_and_caches():
    tiny = TETODRAS["T1"]
    desc = describe_model(tiny["cfg"])
    assert [l.block for l in desc.layers] == ["parallel_pair_ffn", "parallel_mixer", "parallel_pair_ffn", "parallel_pair"]
    assert desc.layers[0].params == {"residual_mult": 0.6, "mixer_weights": (0.8, 1.3)}
    names, _ = expected_tensors(desc)
    assert {"embed", "final.norm", "l0.ls1", "l0.ls2", "l0.mix.left.q.norm", "l0.mix.left.rel", "l0.mix.left.sink",
            "l0.mix.right.i.b", "l1.mix.a", "l1.mix.dt_bias", "l1.mix.q.conv", "l2.mix.right.a2.b", "l2.mix.left.v",
            "l3.mix.right.norm"} <= set(names)
    assert "l0.mix.left.v" not in names and "l1.ls2" not in names and "l3.mlp.up" not in names
    assert names["l0.mix.left.rel"].shape == (12, 4) and names["l2.mix.right.a1"].shape == (16, 128)
    assert names["l1.mix.a"].shape == (4, 128) and names["l1.mix.dt_bias"].shape == (4,)
    assert names["l0.mix.right.norm"].shape == (80,) and names["l2.mix.right.norm"].shape == (32,)
    model = Model(desc, torch.float32, None)
    needs = model.cache_needs()
    assert len(needs) == 7                        # three pairs with two memories each, one delta rule
    pages = [spec for spec, _ in needs.values() if spec is not None]
    states = [state for _, state in needs.values() if state is not None]
    assert len(pages) == 3 and len(states) == 4 and all(spec.window is None for spec in pages)
    assert pages[0].planes == ((2, 32), (2, 32)) and pages[1].planes == ((3, 40), (3, 24))


def test_config_errors():
    raw = TETODRAS["T2"]["cfg"].to_dict()
    for path, value, text in ((("layers", 0, "type"), "window", "not a layer"),
                              (("layers", 1, "mixer", "left", "vdim"), 12, "vdim must equal dim"),
                              (("layers", 0, "mixer", "left", "rot", "dims"), 7, "rot.dims"),
                              (("layers", 2, "mixer", "kv_heads"), 2, "multiple of kv_heads"),
                              (("layers", 1, "mixer", "left", "q_temp", "every"), 0, "temp_every"),
                              (("norm", "eps"), 0.0, "norm.eps")):
        bad = json.loads(json.dumps(raw))
        at = bad
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=text):
            config_from_dict(bad)


@pytest.mark.parametrize("rows,far", [(16, 100.0), (6, 9.0), (32, 256.0), (12, 50.0), (8, 64.0), (20, 1000.5)])
def test_distance_buckets(rows, far):
    table = distance_buckets(rows, far)
    for n in range(3 * int(far)):
        assert table[min(n, len(table) - 1)] == plain.distance_bucket(n, rows, far), n
    assert table[-1] == rows - 1 and table[:rows // 2] == list(range(rows // 2))
    with pytest.raises(ValueError):
        distance_buckets(rows, rows / 2)


@pytest.mark.parametrize("name", sorted(TETODRAS))
def test_a_missing_mechanism_would_show(name, tmp_path):
    """The weights of the tiny models make every mechanism matter: the plain implementation without the sink,
    with the distance table shifted by one row or reaching further, without the temperature, with another cap,
    decay exponent or rotation, with the pair's weights swapped, without the layer scale, or without the first
    tokens' state moves the logits far beyond the tolerances of the comparisons with the engine."""
    import numpy as np
    from tiny_tetodra import requests_for
    from tiny_llm_infer_b200.weights.safetensors_io import SafetensorsFile
    tiny = TETODRAS[name]
    folder = make_folder(tiny, tmp_path)
    cfg = json.loads((folder / "config.json").read_text())
    f = SafetensorsFile(folder / "model.safetensors")
    w = {n: f.read(n).clone() for n in f.tensors}
    f.close()
    toks = max(requests_for(tiny).values(), key=len)[:150]
    ref = plain.forward(cfg, w, toks).numpy()

    def moved(changed_cfg=None, changed_w=None, tokens=None):
        got = plain.forward(changed_cfg or cfg, changed_w or w, tokens or toks).numpy()
        d = got[-40:] - ref[-40:]
        return float((np.sqrt(((d - d.mean(1, keepdims=True)) ** 2).mean(1)) / ref[-40:].std(1)).max())

    def with_weights(fn):
        return {k: fn(k, v) for k, v in w.items()}

    def with_mixers(fn):
        c = json.loads(json.dumps(cfg))
        for layer in c["layers"]:
            fn(layer["type"], layer["mixer"])
        return c

    def set_(d, path, f_):
        for key in path[:-1]:
            d = d.get(key, {})
        if path[-1] in d:
            d[path[-1]] = f_(d[path[-1]])

    floor = 2e-3
    assert moved(changed_w=with_weights(lambda k, v: torch.full_like(v, -80.0) if k.endswith(".sink") else v)) > floor
    assert moved(changed_w=with_weights(lambda k, v: torch.roll(v, 1, 0) if k.endswith(".rel") else v)) > floor
    assert moved(changed_w=with_weights(lambda k, v: torch.ones_like(v) if k.endswith(".ls1") else v)) > floor
    assert moved(changed_w=with_weights(lambda k, v: torch.ones_like(v) if k.endswith(".q.norm") else v)) > floor
    for path, f_ in ((("left", "bias_max"), lambda v: v * 1.5), (("left", "q_temp", "coef"), lambda v: v + 0.5),
                     (("left", "q_temp", "every"), lambda v: v + 1), (("left", "rot", "base"), lambda v: v * 2),
                     (("left", "rot", "dims"), lambda v: v - 2), (("right", "gate_cap"), lambda v: v * 0.5),
                     (("right", "tau"), lambda v: v * 1.5), (("left_scale",), lambda v: v + 0.3)):
        changed = with_mixers(lambda kind, m: set_(m, path, f_))
        if changed != cfg:
            assert moved(changed_cfg=changed) > floor, path
    assert moved(tokens=toks[40:]) > floor                       # the first forty tokens forgotten
