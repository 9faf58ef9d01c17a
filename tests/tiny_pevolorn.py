"""Tiny Pevolorn configurations for the tests.  They differ in every size and constant and take values that hide
nothing: layers in every order (a pair first, a latent layer that borrows from a layer other than the first, two
borrowers of one cache), layers without a feed-forward, fewer key/value heads than query heads and one head alone,
key and value widths that differ and that are no multiples of four, a rotation of part of the rotated width and of
all of it, a layer without a cap, one to four groups of state-space heads, one to five taps, norms in one to four
parts, routers with and without identity experts, with one group and with several, top 1 to 4, with and without a
shared expert, a residual factor of one and others, widths the tensor-core kernels take and widths they do not.
Routers are made decisive and half of the state-space heads slow, so that what was written hundreds of tokens
ago still shows in the read-out."""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tiny_llm_infer_b200.config.pevolorn import (GroupedAttentionConfig, LatentConfig, MixtureConfig, PairConfig,
                                                  PevolornConfig, PevolornLayerConfig, StateSpaceConfig)
from tiny_llm_infer_b200.weights import write_random_model
from tiny_llm_infer_b200.weights.safetensors_io import SafetensorsFile, save_file


def latent(heads, dim, rot_dim, vdim, rank, scale, base, dims, kv_from=None, mlp=None):
    return PevolornLayerConfig("latent_attention", LatentConfig(heads, dim, rot_dim, vdim, rank, scale, base, dims, kv_from), mlp)


def pair(att, ssm, weights=(1.2, 0.9), mlp=None):
    """att: heads, kv_heads, dim, vdim, scale, softcap, base, dims; ssm: heads, vdim, state, groups, conv, norm_groups."""
    return PevolornLayerConfig("parallel", PairConfig(GroupedAttentionConfig(*att), StateSpaceConfig(*ssm), *weights), mlp)


def moe(ff, experts, top, identity, count, keep, shared):
    return MixtureConfig(ff, experts, top, identity, count, keep, shared)


# widths of eight: the vector kernels; a latent of 48 + 16 (tensor-core attention in bfloat16); two borrowers
V1 = dict(cfg=PevolornConfig(vocab=320, width=128, norm_eps=1e-5, postln_alpha=2.0, layers=(
    latent(4, 24, 16, 32, 48, 0.2, 10000.0, 16, mlp=moe(48, 6, 2, 2, 4, 2, 64)),
    pair((4, 2, 32, 24, 0.9, 12.0, 50000.0, 16), (4, 8, 16, 1, 4, 2), mlp=moe(40, 8, 3, 0, 2, 1, None)),
    latent(2, 16, 16, 8, 48, 0.3, 10000.0, 16, kv_from=0),
    pair((2, 2, 48, 48, 0.7, None, 300.0, 48), (2, 24, 32, 2, 2, 1), weights=(0.8, 1.3), mlp=moe(24, 4, 1, 0, 1, 1, 56)),
    latent(4, 8, 16, 16, 48, 0.25, 10000.0, 16, kv_from=0, mlp=moe(32, 9, 4, 3, 4, 3, 32)),
)), seed=51, std=0.08, norm_range=(0.7, 1.3), page_size=16, lengths=(70, 97, 130, 41, 66, 35))
# nothing a multiple of eight, little a multiple of four; one head alone; pages of 8; a pair first; a borrower of layer 1
V2 = dict(cfg=PevolornConfig(vocab=401, width=100, norm_eps=3e-6, postln_alpha=1.0, layers=(
    pair((3, 1, 10, 6, 1.1, None, 77.0, 4), (5, 6, 10, 5, 2, 3), weights=(1.0, 1.0), mlp=moe(30, 5, 3, 0, 1, 1, None)),
    latent(3, 10, 6, 6, 20, 0.35, 5000.0, 4, mlp=moe(12, 4, 2, 2, 3, 1, 50)),
    pair((1, 1, 20, 12, 0.8, 5.0, 250000.0, 20), (3, 10, 6, 1, 5, 1), weights=(0.6, 1.5)),
    latent(1, 6, 6, 10, 20, 0.4, 5000.0, 4, kv_from=1, mlp=moe(20, 7, 2, 1, 2, 2, 10)),
)), seed=52, std=0.12, norm_range=(0.6, 1.4), page_size=8, lengths=(70, 97, 41, 35, 66))
# the tensor-core kernels' own widths (a latent of 96 + 32, keys of 128 with values of 64, 64 and 64), pages of 32,
# prompts of hundreds of tokens, a latent wider than the tensor-core kernels take (136 + 8)
V3 = dict(cfg=PevolornConfig(vocab=512, width=224, norm_eps=1e-6, postln_alpha=0.5, layers=(
    latent(4, 64, 32, 64, 96, 0.1, 20000.0, 32, mlp=moe(64, 9, 4, 3, 4, 3, 136)),
    pair((8, 2, 128, 64, 1.0, 15.0, 400000.0, 64), (4, 64, 64, 2, 3, 4), mlp=moe(56, 12, 2, 0, 3, 2, 96)),
    latent(2, 32, 8, 40, 136, 0.15, 1000.0, 8, mlp=moe(64, 8, 1, 0, 1, 1, None)),
    pair((2, 1, 64, 64, 1.2, 30.0, 10000.0, 32), (8, 16, 128, 4, 4, 2), weights=(1.1, 1.1)),
    latent(8, 32, 32, 32, 96, 0.12, 20000.0, 32, kv_from=0, mlp=moe(32, 14, 3, 2, 2, 1, 48)),
)), seed=53, std=0.07, norm_range=(0.8, 1.2), page_size=32, lengths=(70, 230, 130, 41, 150, 35))
PEVOLORNS = {"V1": V1, "V2": V2, "V3": V3}


def make_folder(tiny, folder=None, dtype=torch.bfloat16) -> Path:
    """Random weights, then: routers made decisive, their corrections of the size of a score, and half of every
    state space's heads slow."""
    folder = Path(folder or tempfile.mkdtemp(prefix="tllm_pevo_"))
    write_random_model(folder, tiny["cfg"], tiny["seed"], tiny["std"], tiny["norm_range"], dtype=dtype)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {name: f.read(name).clone() for name in f.tensors}
    f.close()

    def change(name, fn):
        tensors[name] = fn(tensors[name].float()).to(dtype)

    for i, layer in enumerate(tiny["cfg"].layers):
        p = f"l{i}."
        if layer.type == "parallel":
            def slow(a):
                a[::2] -= 5.0                      # a decay of exp(-0.005 dt): a memory of hundreds of tokens
                return a
            change(p + "mix.right.A_log", slow)
            change(p + "mix.right.conv", lambda c: c * 1.2)
        if layer.mlp is not None:
            change(p + "mlp.router", lambda r: r * (5.0 / tiny["std"] / r.shape[1] ** 0.5))     # logits of order five
            change(p + "mlp.correction", lambda c: c * 2.0)
    save_file(tensors, folder / "model.safetensors")
    return folder


def prompt(seed: int, length: int, vocab: int):
    g = torch.Generator().manual_seed(7000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def requests_for(tiny):
    return {str(i): prompt(i, n, tiny["cfg"].vocab) for i, n in enumerate(tiny["lengths"])}
