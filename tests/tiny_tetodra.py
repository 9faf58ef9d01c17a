"""Tiny Tetodra configurations for the tests.  They differ in every size and constant and take values that hide
nothing: fewer key/value heads than query heads and one head alone, key and value widths that differ and that are
no multiples of four, two to five taps, tables of distance biases of six to twenty rows reaching 9 to 200 tokens,
temperatures that step every 3 to 64 positions, rotations of part of a head and of all of it, layers in every
order with and without a feed-forward, mixing weights and a residual multiplier other than one, widths the
tensor-core kernels take and widths they do not.  Sinks and distance biases are spread out; half of the matrix
memories' keep gates, of the gated linear attention's channels and of the delta rule's heads are made slow, so
that what was written hundreds of tokens ago still shows in the read-out."""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tiny_llm_infer_b200.config.tetodra import (DenseConfig, GatedDeltaConfig, GatedLinearConfig, KeyValueAttentionConfig,
                                                 MatrixMemoryConfig, PairConfig, RotaryAttentionConfig, TetodraConfig,
                                                 TetodraLayerConfig)
from tiny_llm_infer_b200.weights import write_random_model
from tiny_llm_infer_b200.weights.safetensors_io import SafetensorsFile, save_file


def keyed(heads, kv, dim, scale, far, coef, every, rows, mem, weights=(0.8, 1.3), ff=None):
    """A ``parallel`` layer: attention whose values are its keys beside a matrix memory (heads, dim, vdim, cap)."""
    pair = PairConfig(KeyValueAttentionConfig(heads, kv, dim, dim, scale, far, coef, every, rows),
                      MatrixMemoryConfig(*mem), *weights)
    return TetodraLayerConfig("parallel", pair, None if ff is None else DenseConfig(ff))


def rotary(heads, kv, dim, vdim, scale, base, dims, gla, weights=(1.2, 0.7), ff=None):
    """A ``parallel_2`` layer: attention with a rotation beside gated linear attention (heads, dim, vdim, tau, rank)."""
    pair = PairConfig(RotaryAttentionConfig(heads, kv, dim, vdim, scale, base, dims), GatedLinearConfig(*gla), *weights)
    return TetodraLayerConfig("parallel_2", pair, None if ff is None else DenseConfig(ff))


def delta(heads, kv, dim, vdim, conv, ff=None):
    return TetodraLayerConfig("delta", GatedDeltaConfig(heads, kv, dim, vdim, conv), None if ff is None else DenseConfig(ff))


# widths of eight: the vector kernels; keys of 32 and 40 with values of 24 (tensor-core attention in bfloat16)
T1 = dict(cfg=TetodraConfig(vocab=320, width=128, embedding_scale=6.0, norm_eps=1e-5, residual_mult=0.6, layers=(
    keyed(4, 2, 32, 0.3, 50.0, 0.4, 16, 12, (2, 24, 40, 8.0), ff=160),
    delta(4, 2, 16, 24, 4),
    rotary(6, 3, 40, 24, 0.25, 10000.0, 16, (3, 24, 32, 4.0, 16), ff=96),
    keyed(2, 2, 48, 0.2, 110.0, 0.2, 64, 20, (4, 16, 16, 20.0)),
)), seed=41, std=0.08, norm_range=(0.7, 1.3), page_size=16, lengths=(70, 97, 130, 41, 66, 35))
# nothing a multiple of eight, little a multiple of four; one head alone; pages of 8; a table of 6 rows reaching 9
T2 = dict(cfg=TetodraConfig(vocab=401, width=100, embedding_scale=1.0, norm_eps=3e-6, residual_mult=1.0, layers=(
    rotary(3, 1, 10, 6, 0.4, 77.0, 4, (5, 6, 10, 1.5, 9), weights=(1.0, 1.0)),
    keyed(1, 1, 20, 0.35, 9.0, 1.0, 3, 6, (1, 10, 6, 3.0), ff=50),
    delta(3, 1, 10, 6, 2, ff=30),
    delta(2, 2, 6, 10, 5),
    rotary(5, 5, 12, 20, 0.3, 250000.0, 12, (2, 20, 12, 32.0, 8), ff=64),
)), seed=42, std=0.12, norm_range=(0.6, 1.4), page_size=8, lengths=(70, 97, 41, 35, 66))
# keys and values of 64 and 128 (the tensor-core kernels' own widths), pages of 32, prompts of hundreds of tokens;
# a table reaching 200 tokens and a temperature that steps every 50
T3 = dict(cfg=TetodraConfig(vocab=512, width=224, embedding_scale=12.0, norm_eps=1e-6, residual_mult=0.8, layers=(
    rotary(4, 2, 128, 128, 0.09, 400000.0, 64, (2, 64, 64, 12.0, 24), ff=256),
    keyed(8, 2, 64, 0.125, 200.0, 0.35, 50, 16, (2, 128, 64, 14.0), ff=256),
    delta(2, 1, 128, 128, 3, ff=128),
    keyed(2, 1, 128, 0.09, 64.0, 0.5, 100, 8, (3, 40, 72, 6.0)),
)), seed=43, std=0.07, norm_range=(0.8, 1.2), page_size=32, lengths=(70, 300, 130, 41, 210, 35))
TETODRAS = {"T1": T1, "T2": T2, "T3": T3}


def make_folder(tiny, folder=None, dtype=torch.bfloat16) -> Path:
    """Random weights, then: sinks and distance biases spread out, and half of every memory made slow."""
    folder = Path(folder or tempfile.mkdtemp(prefix="tllm_teto_"))
    write_random_model(folder, tiny["cfg"], tiny["seed"], tiny["std"], tiny["norm_range"], dtype=dtype)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {name: f.read(name).clone() for name in f.tensors}
    f.close()

    def change(name, fn):
        tensors[name] = fn(tensors[name].float()).to(dtype)

    for i, layer in enumerate(tiny["cfg"].layers):
        p = f"l{i}.mix."
        if layer.type == "delta":
            def slow(b):
                b[::2] -= 6.0                      # softplus near 0.003: a memory of hundreds of tokens
                return b
            change(p + "dt_bias", slow)
        elif layer.type == "parallel":
            change(p + "left.sink", lambda s: s * 3.0)
            change(p + "left.rel", lambda r: r * 2.5)

            def keep(b):
                b[::2] += 5.0                      # keep gates near one
                return b
            change(p + "right.f.b", keep)
        else:
            def channels(b):
                b[::2] += 4.0
                return b
            change(p + "right.a2.b", channels)
    save_file(tensors, folder / "model.safetensors")
    return folder


def prompt(seed: int, length: int, vocab: int):
    g = torch.Generator().manual_seed(5000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def requests_for(tiny):
    return {str(i): prompt(i, n, tiny["cfg"].vocab) for i, n in enumerate(tiny["lengths"])}
