"""Tetodra as data: which registered parts each layer is made of.

The stream starts as the scaled embedding.  Every layer is a ``parallel_*`` block: one layer norm (a gain, no bias),
whose output every sub-layer reads; the mixers' outputs times a learned vector ``ls1`` and the feed-forward's times
``ls2`` are added to the stream, times the model's residual multiplier.  The mixer is

* a pair of ``biased_attention`` with normed queries and keys, the keys as values, a query temperature, a table of
  distance biases and a learned sink, beside ``matrix_memory`` (layer type ``parallel``);
* a pair of ``biased_attention`` with a rotation of part of every head and plain softmax, beside ``gated_linear``
  (layer type ``parallel_2``); a pair's outputs are mixed with two weights of the layer;
* ``channel_delta`` with one decay per head and a SiLU gate from a full projection (layer type ``delta``);

then, where the layer has one, a ``swiglu`` feed-forward with SiLU.  The model's last norm is a layer norm too and
the head is the embedding table itself.  Tensor names: ``embed``, ``l<i>.norm1|ls1|ls2``,
``l<i>.mix.left.q|k|v|o|q.norm|k.norm|rel|sink``, ``l<i>.mix.right.q|k|v|g|o|norm|i|i.b|f|f.b|a1|a2|a2.b``,
``l<i>.mix.q|k|v`` (+ ``.conv``) ``|b|A_log|norm|a|dt_bias|g|o``, ``l<i>.mlp.gate|up|down``, ``final.norm``.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.tetodra import (ARCHITECTURE, DEFAULT_BIAS_ROWS, GatedDeltaConfig, KeyValueAttentionConfig,
                              MatrixMemoryConfig, TetodraConfig, default_rank)
from ..parts.spec import ExecEntry, LayerSpec, ModelDescription, PartSpec

UNIT_EPS = 1e-6               # under the root when the delta rule's q and k are made unit vectors
MEMORY_FLOOR_EPS = 1e-6       # added to the matrix memory's divisor
GATED_NAMES = ("gate", "up", "down")
ATTENTION_NAMES = ("q", "k", "v", "o", "g")
DELTA_NAMES = ("q", "k", "v", "b", "A_log", "norm", "a", "a.unused", "dt_bias", "g", "g.unused", "o")


def describe_tetodra(cfg: TetodraConfig) -> ModelDescription:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        parts = {"norm1": PartSpec("layernorm", dict(width=cfg.width, eps=cfg.norm_eps, name="norm1"), p),
                 "ls1": PartSpec("column_scale", dict(width=cfg.width, name="ls1"), p)}
        params = dict(residual_mult=cfg.residual_mult)
        if isinstance(m, GatedDeltaConfig):
            block = "parallel_mixer"
            parts["mixer"] = PartSpec("channel_delta", dict(
                hidden_size=cfg.width, heads=m.heads, kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim,
                conv_taps=m.conv, decay_rank=0, gate_rank=0, norm_eps=cfg.norm_eps, unit_eps=UNIT_EPS,
                names=DELTA_NAMES, decay_per_head=True, full_gate=True, gate_act="silu"), p + "mix.")
        else:
            block = "parallel_pair"
            params["mixer_weights"] = (m.left_scale, m.right_scale)
            a, r = m.left, m.right
            common = dict(hidden_size=cfg.width, q_heads=a.heads, kv_heads=a.kv_heads, key_dim=a.dim, value_dim=a.vdim,
                          scale=a.scale, names=ATTENTION_NAMES)
            if isinstance(a, KeyValueAttentionConfig):
                common.update(unit_norm_eps=cfg.norm_eps, qk_gains=True, values_are_keys=True,
                              q_temperature=(a.temp_coef, a.temp_every),
                              distance_bias=(a.bias_rows or DEFAULT_BIAS_ROWS, a.bias_max), sink=True, learned_sink=True)
            else:
                common.update(position=PartSpec("rotary_half", dict(head_dim=a.dim, theta=a.rot_base, rotary_dim=a.rot_dims)))
            parts["left"] = PartSpec("biased_attention", common, p + "mix.left.")
            if isinstance(r, MatrixMemoryConfig):
                parts["right"] = PartSpec("matrix_memory", dict(
                    hidden_size=cfg.width, heads=r.heads, key_dim=r.dim, value_dim=r.vdim, gate_cap=r.gate_cap,
                    norm_eps=cfg.norm_eps, floor_eps=MEMORY_FLOOR_EPS), p + "mix.right.")
            else:
                parts["right"] = PartSpec("gated_linear", dict(
                    hidden_size=cfg.width, heads=r.heads, key_dim=r.dim, value_dim=r.vdim,
                    decay_rank=r.decay_rank or default_rank(cfg.width), tau=r.tau, norm_eps=cfg.norm_eps), p + "mix.right.")
        if layer.mlp is not None:
            block += "_ffn"
            parts["ffn"] = PartSpec("swiglu", dict(hidden_size=cfg.width, intermediate_size=layer.mlp.ff,
                                                   activation="silu", names=GATED_NAMES), p + "mlp.")
            parts["ls2"] = PartSpec("column_scale", dict(width=cfg.width, name="ls2"), p)
        layers.append(LayerSpec(block, parts, params))
    return ModelDescription(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=cfg.width,
                                                   scale=cfg.embedding_scale, name="embed"), ""),
        layers=tuple(layers),
        order=tuple(ExecEntry(i) for i in range(len(cfg.layers))),
        final_norm=PartSpec("layernorm", dict(width=cfg.width, eps=cfg.norm_eps, name="norm"), "final."),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tied=True), "lm_head."),
    )


register_architecture(ARCHITECTURE, TetodraConfig, describe_tetodra, model_types=("tetodra",))
