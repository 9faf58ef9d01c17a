"""Pevolorn as data: which registered parts each layer is made of.

The stream starts as the embedding.  Every layer norms after its sums, and the norm's result is the stream
(``postnorm_*`` blocks): x <- N1(alpha x + mixer(x)), then, where the layer has a feed-forward, x <- N2(alpha x +
ffn(x)), with N an RMS norm whose stored weight is the gain minus one.  The mixer is

* ``latent_attention`` with directly projected queries, the rotation that pairs an element with the one half a
  rotated width away, plain causal softmax and one sigmoid gate per head; a layer whose configuration says
  ``kv_from`` has no compression of its own and reads (without writing) the cache of the layer named there;
* a pair of ``biased_attention`` (biases on its projections, a rotation of part of every head, unit queries and
  keys, a capped score, one gate per head) beside ``state_space``, mixed with two weights of the layer;

then a ``moe`` feed-forward: a softmax over all experts, a learned correction for the choice, groups of experts of
which only the best may be chosen from, identity experts, plain experts with the squared ReLU, the weights the
scores as they are, and a shared expert of the same form.  The model's last norm has the same form and the head is
the embedding table itself.  Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.q|dkv|dkv.norm|uk|uv|g|o``,
``l<i>.mix.left.q|k|v|o`` (+ ``.b``) ``|g``, ``l<i>.mix.right.in|conv|conv.b|dt_bias|A_log|D|norm|o``,
``l<i>.mlp.router|correction|e<j>.up|e<j>.down|shared.up|shared.down``, ``final.norm``.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.pevolorn import ARCHITECTURE, LatentConfig, PevolornConfig
from ..parts.spec import ExecEntry, LayerSpec, ModelDescription, PartSpec

EXPERT_ACTIVATION = "relu2"       # the design's experts: W_down relu(W_up x)^2
LATENT_NAMES = ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "sink", "g", "o")
ATTENTION_NAMES = ("q", "k", "v", "o", "g")


def _norm(cfg: PevolornConfig, name: str, prefix: str) -> PartSpec:
    return PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, name=name, offset=1.0), prefix)


def describe_pevolorn(cfg: PevolornConfig) -> ModelDescription:
    layers, order = [], []
    mixers_before = 0                 # cache ids: one per mixer, in layer order
    first_cache = {}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        parts = {"norm1": _norm(cfg, "norm1", p)}
        params = dict(alpha=cfg.postln_alpha)
        first_cache[i] = mixers_before
        if isinstance(m, LatentConfig):
            block = "postnorm_mixer"
            parts["mixer"] = PartSpec("latent_attention", dict(
                hidden_size=cfg.width, heads=m.heads, plain_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, q_rank=0,
                kv_rank=m.kv_rank, scale=m.scale, norm_eps=cfg.norm_eps, rot_base=m.rot_base, rot_dims=m.rot_dims,
                rotation="half", output_gate=True, gate_per_head=True, borrows_cache=m.kv_from is not None,
                names=LATENT_NAMES, q_name="q"), p + "mix.")
            if m.kv_from is None:
                order.append(ExecEntry(i, cache=mixers_before))
            else:
                order.append(ExecEntry(i, cache=first_cache[m.kv_from], writes_cache=False))
            mixers_before += 1        # a borrowing layer's id stays unused: ids follow the layers
        else:
            block = "postnorm_pair"
            params["mixer_weights"] = (m.left_scale, m.right_scale)
            a, r = m.left, m.right
            parts["left"] = PartSpec("biased_attention", dict(
                hidden_size=cfg.width, q_heads=a.heads, kv_heads=a.kv_heads, key_dim=a.dim, value_dim=a.vdim,
                scale=a.scale, unit_norm_eps=cfg.norm_eps, softcap=a.softcap, output_gate=True, gate_per_head=True,
                biases=True, defer_output_bias=True, names=ATTENTION_NAMES,
                position=PartSpec("rotary_half", dict(head_dim=a.dim, theta=a.rot_base, rotary_dim=a.rot_dims))),
                p + "mix.left.")
            parts["right"] = PartSpec("state_space", dict(
                hidden_size=cfg.width, heads=r.heads, head_dim=r.vdim, state=r.state, groups=r.groups, conv_taps=r.conv,
                norm_groups=r.norm_groups, norm_eps=cfg.norm_eps), p + "mix.right.")
            order.append(ExecEntry(i, cache=(mixers_before, mixers_before + 1)))
            mixers_before += 2
        if layer.mlp is not None:
            f = layer.mlp
            block += "_ffn"
            shared = None
            if f.shared_ff is not None:
                shared = PartSpec("mlp", dict(hidden_size=cfg.width, intermediate_size=f.shared_ff,
                                              activation=EXPERT_ACTIVATION, names=("up", "down")), "shared.")
            parts["ffn"] = PartSpec("moe", dict(
                hidden_size=cfg.width, experts=f.experts, top=f.top, expert_size=f.expert_ff, activation=EXPERT_ACTIVATION,
                router_scores="softmax_all", weight_on="output", shared=shared, gated=False, names=("up", "down"),
                correction=True, groups=(f.group_count, f.group_keep), identity=f.identity), p + "mlp.")
            parts["norm2"] = _norm(cfg, "norm2", p)
        layers.append(LayerSpec(block, parts, params))
    return ModelDescription(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, scale=1.0, name="embed"), ""),
        layers=tuple(layers),
        order=tuple(order),
        final_norm=_norm(cfg, "norm", "final."),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tied=True), "lm_head."),
    )


register_architecture(ARCHITECTURE, PevolornConfig, describe_pevolorn, model_types=("pevolorn",))
