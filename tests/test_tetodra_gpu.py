"""Tetodra on the GPU against the plain implementation (``plain_tetodra.py``).

Each mechanism alone, as the registered part with sizes of its own: the scaled sum of several outputs fused with
the layer norm; the attention whose values are its keys (gains, temperature, table of distance biases, learned
sink) and the attention with a rotation of part of a head, over scrambled pages that hold other requests'
leftovers, with inputs shaped so that single keys far back, at page borders and next to the query stand out;
the matrix memory, the gated linear attention and the delta rule with a decay per head, whole, in portions down
to one token, side by side and in slots that are used again, with gates slow enough that the first tokens still
show at the end.  Then whole models through ``bin/trace_run`` in every way of cutting, the first tokens one by
one, long decoding, and greedy generation through the engine's entry point under budgets and starved pools.

Tolerances, as a row's root-mean-square difference (its mean taken off) over the row's own spread: float32 2e-4
against the plain implementation and between the ways of cutting; bfloat16 three times what a B200 shows per
configuration."""
import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_tetodra as plain
import replay
from tiny_tetodra import TETODRAS, make_folder, prompt, requests_for

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
F64 = torch.float64


def read_model(folder):
    from tiny_llm_infer_b200.weights.safetensors_io import SafetensorsFile
    cfg = json.loads((Path(folder) / "config.json").read_text())
    f = SafetensorsFile(Path(folder) / "model.safetensors")
    w = {name: f.read(name).clone() for name in f.tensors}
    f.close()
    return cfg, w


def make_ctx(rows):
    """rows: (slot, first position, count) per portion -> the step's context, as the runner lays it out."""
    from tiny_llm_infer_b200.engine.batch import StepContext
    pos, slots, seg, tiles, dec, row = [], [], [], [], [], 0
    for s, (slot, p0, n) in enumerate(rows):
        pos += list(range(p0, p0 + n))
        slots += [slot] * n
        seg.append([slot, row, n, p0])
        if n == 1:
            dec.append(row)
        else:
            tiles += [[s, off] for off in range(0, n, 64)]
        row += n
    # blocks at multiples of 256 rows first, then those at other multiples of 128 (the tcgen05 kernel's lists)
    tiles.sort(key=lambda t: (t[1] % 256 != 0, t[1] % 128 != 0, -(rows[t[0]][1] + t[1])))
    i32 = dict(dtype=torch.int32, device=DEV)
    return StepContext(tokens=row, token_ids=None, positions=torch.tensor(pos, **i32),
                       token_slot=torch.tensor(slots, **i32), want_rows=None, segments=[],
                       seg_info=torch.tensor(seg, **i32),
                       dec_rows=torch.tensor(dec, **i32) if dec and len(dec) < row else None, n_dec=len(dec),
                       pf_tiles=torch.tensor(tiles, **i32).view(-1, 2), n_tiles=len(tiles),
                       n_tiles128=sum(1 for t in tiles if t[1] % 128 == 0),
                       n_tiles256=sum(1 for t in tiles if t[1] % 256 == 0),
                       decode_only=all(n == 1 for _, _, n in rows), max_context=max(p0 + n for _, p0, n in rows),
                       max_segment=max(n for _, _, n in rows))


def build_part(kind, params, dtype, seed, change=None, stds=None):
    """The registered mixer with random weights of its own -> (part, float64 weights under the prefix ``m.``)."""
    from tiny_llm_infer_b200.parts.registry import lookup
    cls = lookup("mixer", kind)
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, spec in cls.param_specs(**params).items():
        if spec.init == "norm":
            w[name] = torch.rand(spec.shape, generator=g) * 0.8 + 0.6
        else:
            w[name] = torch.randn(spec.shape, generator=g) * (stds or {}).get(name, 0.5 if spec.init == "unit" else 0.25)
    if change:
        change(w)
    w = {k: v.to(dtype) for k, v in w.items()}
    part = cls(dtype=dtype, device=DEV, **params)
    part.load({k: v.to(DEV) for k, v in w.items()})
    return part, {"m." + k: v.double() for k, v in w.items()}


class Bench:
    """A cache of the part's own: scrambled pages full of leftovers, a state per slot; ``step`` runs portions of
    several requests as one batch and returns the worst difference from what is expected."""

    def __init__(self, part, dtype, xs, want, page=16, slots=4, seed=3):
        from tiny_llm_infer_b200.cache.manager import LayerCacheView
        self.part, self.xs, self.want, self.dtype = part, xs, want, dtype
        longest = max(x.shape[0] for x in xs)
        spec, st = part.cache_spec(), part.state_spec()
        planes, table = (), None
        if spec is not None:
            per = -(-longest // page)
            g = torch.Generator().manual_seed(seed)
            order = torch.randperm(slots * per + 3, generator=g)
            table = order[:slots * per].view(slots, per).to(torch.int32).to(DEV)
            # the planes of a page lie one behind the other, as in the cache manager's pools
            sizes = [heads * page * width for heads, width in spec.planes]
            flat = (torch.randn(slots * per + 3, sum(sizes), generator=g) * 2.0).to(dtype).to(DEV)
            planes, at = [], 0
            for (heads, width), size in zip(spec.planes, sizes):
                planes.append(flat[:, at:at + size].unflatten(1, (heads, page, width)))
                at += size
            planes = tuple(planes)
        self.state = torch.zeros(slots, st.shape[0], device=DEV) if st is not None else None
        self.view = LayerCacheView(kv=None, block_table=table, page_size=page, writes=True, state=self.state,
                                   window=None, planes=planes)

    def step(self, rows):
        """rows: (request, slot, first position, count)."""
        x = torch.cat([self.xs[r][p0:p0 + n] for r, _, p0, n in rows]).to(self.dtype).to(DEV)
        got = self.part.forward(x, make_ctx([(slot, p0, n) for _, slot, p0, n in rows]), self.view).double().cpu()
        assert torch.isfinite(got).all()
        expect = torch.cat([self.want[r][p0:p0 + n] for r, _, p0, n in rows])
        return ((got - expect).abs().max() / expect.abs().max()).item()

    def free(self, slot):
        if self.state is not None:
            self.state[slot].zero_()          # as the cache manager does at admission


SIZES = [1, 1, 2, 1, 3, 2, 17, 2, 1, 16, 33, 1, 64, 5]


def whole_then_portions(bench, lengths):
    """Request 0 whole beside 1 and 2; then, in slots and pages that were used, 0 again in portions of every size
    down to one token beside 1, which sits some steps out."""
    worst_whole = bench.step([(0, 2, 0, lengths[0]), (1, 0, 0, lengths[1]), (2, 3, 0, lengths[2])])
    bench.free(2)
    bench.free(0)
    at0 = at1 = k = 0
    worst = 0.0
    while at0 < lengths[0]:
        n0 = min(SIZES[k % len(SIZES)], lengths[0] - at0)
        rows = [(0, 0, at0, n0)]
        if at1 < lengths[1] and k % 3 != 1:
            n1 = min(SIZES[(k + 5) % len(SIZES)], lengths[1] - at1)
            rows.append((1, 2, at1, n1))
            at1 += n1
        worst = max(worst, bench.step(rows))
        at0 += n0
        k += 1
    assert at1 == lengths[1]
    return worst_whole, worst


# ----------------------------------------------------------------------------- the sum and the layer norm
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,n", [(100, 3), (192, 2), (4104, 1), (36, 0)])
def test_scaled_sum_with_layer_norm(dtype, width, n):
    from tiny_llm_infer_b200 import ops
    torch.manual_seed(width)
    h = torch.randn(11, width, device=DEV) * 3 + 1.5
    deltas = [(torch.randn(11, width, device=DEV) * 4).to(dtype) for _ in range(n)]
    scales = [torch.randn(width, device=DEV) for _ in range(n)]
    gain = (torch.rand(width, device=DEV) + 0.5).to(dtype)
    total = h.double()
    for d, s in zip(deltas, scales):
        total = total + s.double() * d.double()
    want = plain.layer_norm(total, gain.double(), 3e-6)
    tol = 2e-5 if dtype == torch.float32 else 0.03
    rows = torch.tensor([7, 0, -1, 10], dtype=torch.int32, device=DEV)
    before = h.clone()
    out = torch.empty(4, width, dtype=dtype, device=DEV)
    ops.scaled_add_layernorm(h, deltas, scales, gain, 3e-6, out, rows)      # chosen rows: the stream is not written
    assert torch.equal(h, before) and out[2].abs().max() == 0
    assert (out[[0, 1, 3]].double() - want[[7, 0, 10]]).abs().max() < tol
    out = torch.empty(11, width, dtype=dtype, device=DEV)
    ops.scaled_add_layernorm(h, deltas, scales, gain, 3e-6, out)
    assert (h.double() - total).abs().max() < 2e-5                           # the stream itself stays float32
    assert (out.double() - want).abs().max() < tol


# ----------------------------------------------------------------------------- the two attentions as parts
def turn(hidden, seed=99):
    """A fixed orthogonal matrix of the rows' width."""
    g = torch.Generator().manual_seed(seed)
    return torch.linalg.qr(torch.randn(hidden, hidden, generator=g, dtype=F64)).Q.float()


def echo_inputs(lengths, hidden, page, seed):
    """Random rows in which chosen queries are the turned row (``turn``) of one key: the first token, the second,
    the keys on both sides of page borders far back, a key in the middle and the key next to the query.  With
    keys projected like the first query head of their group after the same turn, that one score stands out among
    all others (and the query's own key does not)."""
    g = torch.Generator().manual_seed(seed)
    R = turn(hidden)
    xs = []
    for L in lengths:
        x = torch.randn(L, hidden, generator=g)
        for i in range(5, L - 1, 11):
            x[i] = R @ x[i - 1]                            # the key next to the query
        targets = [0, 1, page - 1, page, 2 * page - 1, 2 * page, L // 2, L // 2 + 1]
        i = L - 1
        for n, j in enumerate(targets * 3):
            if i <= j + 1 or i < 2:
                break
            x[i] = R @ x[j]
            i -= 2 + n % 3
        xs.append(x)
    return xs


def tie_keys_to_queries(H, G, dk, hidden):
    R = turn(hidden)

    def change(w):
        for kv in range(G):
            first = kv * (H // G)
            w["k"][kv * dk:(kv + 1) * dk] = w["q"][first * dk:(first + 1) * dk] @ R
    return change


KEYED_CASES = [dict(H=4, G=2, dk=32, scale=0.3, far=50.0, coef=0.4, every=16, rows=12, page=16),
               dict(H=1, G=1, dk=20, scale=0.35, far=9.0, coef=1.0, every=3, rows=6, page=8),
               dict(H=8, G=2, dk=64, scale=0.125, far=200.0, coef=0.35, every=50, rows=16, page=32),
               dict(H=6, G=6, dk=128, scale=0.09, far=64.0, coef=0.5, every=100, rows=8, page=16),
               dict(H=3, G=1, dk=44, scale=0.2, far=1000.5, coef=0.0, every=1, rows=20, page=16)]


@pytest.mark.parametrize("case", KEYED_CASES, ids=lambda c: f"h{c['H']}g{c['G']}k{c['dk']}r{c['rows']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_keys_as_values(case, dtype):
    from tiny_llm_infer_b200.engine.runner import strict_float32
    strict_float32()
    H, G, dk, hidden = case["H"], case["G"], case["dk"], 104
    params = dict(hidden_size=hidden, q_heads=H, kv_heads=G, key_dim=dk, value_dim=dk, scale=case["scale"],
                  unit_norm_eps=2e-6, qk_gains=True, values_are_keys=True, q_temperature=(case["coef"], case["every"]),
                  distance_bias=(case["rows"], case["far"]), sink=True, learned_sink=True)

    def change(w):
        tie_keys_to_queries(H, G, dk, hidden)(w)
        w["rel"] *= 4.0                                      # rows of the table that differ by whole units
        w["sink"] *= 4.0
    part, w64 = build_part("biased_attention", params, dtype, seed=dk, change=change)
    lengths = (290, 75, 1)
    xs = [x.to(dtype) for x in echo_inputs(lengths, hidden, case["page"], seed=H)]
    m = dict(heads=H, kv_heads=G, dim=dk, vdim=dk, scale=case["scale"], bias_max=case["far"],
             q_temp=dict(coef=case["coef"], every=case["every"]))
    want = [plain.attention_keys_as_values(x.double(), w64, "m.", m, 2e-6) for x in xs]
    # the echoes do take the weight: without the far keys the answer at the last query differs
    cut = plain.attention_keys_as_values(xs[0][40:].double(), w64, "m.", m, 2e-6)
    assert (cut[-1] - want[0][-1]).abs().max() > 0.05 * want[0].abs().max()
    whole, cutup = whole_then_portions(Bench(part, dtype, xs, want, page=case["page"]), lengths)
    limit = 3e-5 if dtype == torch.float32 else 0.06
    assert whole < limit and cutup < limit, (whole, cutup)


ROTARY_CASES = [dict(H=6, G=3, dk=40, dv=24, scale=0.25, base=10000.0, dims=16, page=16),
                dict(H=3, G=1, dk=10, dv=6, scale=0.4, base=77.0, dims=4, page=8),
                dict(H=4, G=2, dk=128, dv=128, scale=0.09, base=400000.0, dims=64, page=32),
                dict(H=5, G=5, dk=12, dv=20, scale=0.3, base=250000.0, dims=12, page=16),
                dict(H=8, G=2, dk=80, dv=176, scale=0.1, base=1e6, dims=80, page=16),
                dict(H=2, G=2, dk=64, dv=64, scale=0.125, base=300.0, dims=2, page=16)]


@pytest.mark.parametrize("case", ROTARY_CASES, ids=lambda c: f"h{c['H']}g{c['G']}k{c['dk']}v{c['dv']}r{c['dims']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_a_rotation_of_part_of_the_head(case, dtype):
    from tiny_llm_infer_b200.engine.runner import strict_float32
    from tiny_llm_infer_b200.parts.spec import PartSpec
    strict_float32()
    H, G, dk, dv, hidden = case["H"], case["G"], case["dk"], case["dv"], 88
    params = dict(hidden_size=hidden, q_heads=H, kv_heads=G, key_dim=dk, value_dim=dv, scale=case["scale"],
                  position=PartSpec("rotary_half", dict(head_dim=dk, theta=case["base"], rotary_dim=case["dims"])))
    part, w64 = build_part("biased_attention", params, dtype, seed=dk + dv, change=tie_keys_to_queries(H, G, dk, hidden),
                           stds={"q": 0.3, "k": 0.3})
    lengths = (290, 75, 1)
    xs = [x.to(dtype) for x in echo_inputs(lengths, hidden, case["page"], seed=G)]
    m = dict(heads=H, kv_heads=G, dim=dk, vdim=dv, scale=case["scale"], rot=dict(base=case["base"], dims=case["dims"]))
    want = [plain.attention_rotary(x.double(), w64, "m.", m) for x in xs]
    whole, cutup = whole_then_portions(Bench(part, dtype, xs, want, page=case["page"]), lengths)
    limit = 3e-5 if dtype == torch.float32 else 0.06
    assert whole < limit and cutup < limit, (whole, cutup)
    # the angles are the positions': a request that starts later in the cache's numbering would differ
    moved = plain.rotate_half(torch.ones(1, 1, dk, dtype=F64), torch.tensor([257]), case["base"], case["dims"])
    assert (moved - 1).abs().max() > 0.1


@pytest.mark.parametrize("splits_forced", [None, 1])
@pytest.mark.parametrize("H,G,table_rows,sink", [(4, 2, 300, True), (3, 3, 64, True), (2, 1, 1500, False), (2, 2, 0, False)])
def test_planes_attention_on_tcgen05_over_a_long_request(H, G, table_rows, sink, splits_forced, monkeypatch):
    """Width 128 on both sides: prompt portions take the tcgen05 kernel over the two planes.  One portion of 2500
    tokens behind 900 in the cache (the rings of tiles and every barrier wrap; few blocks, so the keys of a block
    are shared out and summed again), with a table of biases whose end falls inside a tile, a sink, and one key
    900 or more tokens back made to stand out for sampled rows.  Against float64 and against the mma.sync kernel."""
    from tiny_llm_infer_b200 import ops
    d, page, have, new = 128, 16, 900, 2500
    n, pages = have + new, -(-(have + new) // page)
    g = torch.Generator().manual_seed(H * 10 + G)
    flat = (torch.randn(pages + 5, 2 * G * page * d, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    k_plane = flat[:, :G * page * d].unflatten(1, (G, page, d))
    v_plane = flat[:, G * page * d:].unflatten(1, (G, page, d))
    table = torch.randperm(pages + 5, generator=g)[:pages].to(torch.int32).view(1, -1).to(DEV)
    q = (torch.randn(new, H, d, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    keys_of = lambda plane: plane[table[0].long()].double().permute(1, 0, 2, 3).reshape(G, pages * page, d)[:, :n]
    K, V = keys_of(k_plane), keys_of(v_plane)
    sample = torch.cat([torch.arange(0, new, 41), torch.tensor([127, 128, 255, 256, new - 1])])
    for i, r in enumerate(sample.tolist()):                   # a far key that carries the answer of these rows
        q[r, :, :] = (K[:, (7 * i) % have].repeat_interleave(H // G, 0) * 4.0).to(torch.bfloat16)
    bias = sinks = None
    if table_rows:
        bias = (torch.randn(H, table_rows, generator=g) * 1.5).to(DEV)
        bias[:, -1] = 2.0                                      # what the far keys get
    if sink:
        sinks = (torch.randn(H, generator=g) * 2.0 + 4.0).to(DEV)
    ctx = make_ctx([(0, have, new)])
    if splits_forced:
        monkeypatch.setattr(ops, "prefill_splits", lambda blocks, ctx_len: splits_forced)
    else:
        pairs = ops.prefill_tcgen05_block_rows(H, G) == 128
        assert ops.prefill_splits(ctx.n_tiles128 * H // 2 if pairs else ctx.n_tiles256 * H, n) > 1
    outs = {}
    for fast in (True, False):
        monkeypatch.setattr(ops, "PREFILL_TCGEN05", fast)
        before = ops.tcgen05_calls
        out = torch.zeros(new, H * d, dtype=torch.bfloat16, device=DEV)
        ops.attention_biased(q.view(new, -1), k_plane, v_plane, ctx.positions, ctx.token_slot, table, page, H, G, d, d,
                             0.11, out, sink=sink, sink_logits=sinks, distance_bias=bias, ctx=ctx)
        ops.check_error_word(torch.device(DEV))
        assert (ops.tcgen05_calls > before) == fast
        outs[fast] = out.double().view(new, H, d)
    pos = have + sample.to(DEV)
    keys = torch.arange(n, device=DEV)
    mask = keys[None, :] <= pos[:, None]
    for h in range(H):
        s = q[sample.to(DEV), h].double() @ K[h // (H // G)].T * 0.11
        if bias is not None:
            s = s + bias[h].double()[(pos[:, None] - keys[None, :]).clamp(0, table_rows - 1)]
        s = s.masked_fill(~mask, float("-inf"))
        top = s.max(-1, keepdim=True).values
        e = torch.exp(s - top)
        den = e.sum(-1, keepdim=True) + (torch.exp(sinks[h].double() - top) if sink else 0.0)
        want = (e / den) @ V[h // (H // G)]
        # the far key holds most of the weight of its row
        held = (e / den)[torch.arange(len(sample)), [(7 * i) % have for i in range(len(sample))]]
        assert held.median() > 0.9 and held.min() > 0.05
        for fast in (True, False):
            err = (outs[fast][sample.to(DEV), h] - want).abs().max().item()
            assert err < 0.02 * want.abs().max().item() + 0.01, (h, fast, err)
    assert (outs[True] - outs[False]).abs().max() < 0.03


# ----------------------------------------------------------------------------- the three recurrences as parts
def recurrence_run(part, w64, plain_fn, dtype, hidden, lengths=(230, 61, 1), seed=5, reach=200):
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(L, hidden, generator=g).to(dtype) for L in lengths]
    want = [plain_fn(x.double()) for x in xs]
    # old tokens still show at the end: without the state carried over ``reach`` tokens the answer differs
    # (200 where the gates can stay open that long; a low cap on the gates or a narrow key forgets sooner)
    short = plain_fn(xs[0][lengths[0] - reach:].double())
    assert (short[-1] - want[0][-1]).abs().max() > 1e-3 * want[0].abs().max()
    return whole_then_portions(Bench(part, dtype, xs, want), lengths)


MEMORY_CASES = [dict(H=2, dk=24, dv=40, cap=8.0), dict(H=1, dk=10, dv=6, cap=3.0, reach=40), dict(H=2, dk=128, dv=64, cap=14.0),
                dict(H=3, dk=40, dv=72, cap=6.0), dict(H=4, dk=16, dv=16, cap=20.0), dict(H=5, dk=7, dv=2, cap=1.5, reach=20)]


@pytest.mark.parametrize("case", MEMORY_CASES, ids=lambda c: f"h{c['H']}k{c['dk']}v{c['dv']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_matrix_memory(case, dtype):
    """Gate logits of several units, so that the cap bends them; keep gates near one on every second head."""
    from tiny_llm_infer_b200.engine.runner import strict_float32
    strict_float32()
    H, dk, dv, hidden = case["H"], case["dk"], case["dv"], 96
    params = dict(hidden_size=hidden, heads=H, key_dim=dk, value_dim=dv, gate_cap=case["cap"], norm_eps=1e-5, floor_eps=1e-6)

    def change(w):
        w["i"] *= 2.0
        w["f"] *= 0.2
        w["f.b"] += 5.0
        w["f.b"][1::2] -= 3.0
        w["i.b"] -= 1.0
    part, w64 = build_part("matrix_memory", params, dtype, seed=dk, change=change)
    m = dict(heads=H, dim=dk, vdim=dv, gate_cap=case["cap"])
    raw = (torch.randn(50, hidden, dtype=F64) @ w64["m.i"].T).abs().max().item()
    assert raw > case["cap"] * 0.5                                           # the cap does bend
    whole, cutup = recurrence_run(part, w64, lambda x: plain.matrix_memory(x, w64, "m.", m, 1e-5), dtype, hidden,
                                  reach=case.get("reach", 200))
    limit = 3e-5 if dtype == torch.float32 else 0.06
    assert whole < limit and cutup < limit, (whole, cutup)


LINEAR_CASES = [dict(H=3, dk=24, dv=32, tau=4.0, rank=16), dict(H=5, dk=6, dv=10, tau=1.5, rank=9),
                dict(H=2, dk=64, dv=64, tau=16.0, rank=24), dict(H=2, dk=20, dv=12, tau=32.0, rank=8),
                dict(H=4, dk=56, dv=24, tau=12.0, rank=12), dict(H=1, dk=130, dv=3, tau=2.0, rank=5)]


@pytest.mark.parametrize("case", LINEAR_CASES, ids=lambda c: f"h{c['H']}k{c['dk']}v{c['dv']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_linear_attention(case, dtype):
    from tiny_llm_infer_b200.engine.runner import strict_float32
    strict_float32()
    H, dk, dv, hidden = case["H"], case["dk"], case["dv"], 72
    params = dict(hidden_size=hidden, heads=H, key_dim=dk, value_dim=dv, decay_rank=case["rank"], tau=case["tau"], norm_eps=2e-6)

    def change(w):
        w["a2.b"][::2] += 4.0                                # every second key channel forgets slowly
    part, w64 = build_part("gated_linear", params, dtype, seed=dk + 1, change=change)
    m = dict(heads=H, dim=dk, vdim=dv, tau=case["tau"])
    whole, cutup = recurrence_run(part, w64, lambda x: plain.gated_linear_attention(x, w64, "m.", m, 2e-6), dtype, hidden)
    limit = 3e-5 if dtype == torch.float32 else 0.06
    assert whole < limit and cutup < limit, (whole, cutup)


HEAD_DELTA_CASES = [dict(H=4, G=2, dk=16, dv=24, taps=4), dict(H=3, G=1, dk=10, dv=6, taps=2, reach=120), dict(H=2, G=2, dk=6, dv=10, taps=5, reach=50),
                    dict(H=2, G=1, dk=128, dv=128, taps=3), dict(H=2, G=1, dk=36, dv=72, taps=1), dict(H=6, G=3, dk=40, dv=8, taps=3)]


@pytest.mark.parametrize("case", HEAD_DELTA_CASES, ids=lambda c: f"h{c['H']}g{c['G']}k{c['dk']}v{c['dv']}t{c['taps']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_delta_rule_with_a_decay_per_head(case, dtype):
    from tiny_llm_infer_b200.engine.runner import strict_float32
    from tiny_llm_infer_b200.models.tetodra import DELTA_NAMES
    strict_float32()
    H, G, dk, dv, hidden = case["H"], case["G"], case["dk"], case["dv"], 80
    params = dict(hidden_size=hidden, heads=H, kv_heads=G, key_dim=dk, value_dim=dv, conv_taps=case["taps"], decay_rank=0,
                  gate_rank=0, norm_eps=1e-5, unit_eps=1e-6, names=DELTA_NAMES, decay_per_head=True, full_gate=True,
                  gate_act="silu")

    def change(w):
        w["a"] *= 0.2
        w["dt_bias"][::2] -= 6.0                             # every second head forgets slowly
    part, w64 = build_part("channel_delta", params, dtype, seed=dk + dv, change=change)
    m = dict(heads=H, kv_heads=G, dim=dk, vdim=dv, conv=case["taps"])
    whole, cutup = recurrence_run(part, w64, lambda x: plain.gated_delta(x, w64, "m.", m, 1e-5), dtype, hidden,
                                  reach=case.get("reach", 200))
    limit = 3e-5 if dtype == torch.float32 else 0.06
    assert whole < limit and cutup < limit, (whole, cutup)


# ----------------------------------------------------------------------------- whole models, every way of cutting
BF16_RMS = {"T1": 0.3, "T2": 0.3, "T3": 0.3}


@pytest.fixture(scope="module", params=sorted(TETODRAS))
def case(request, tmp_path_factory):
    name = request.param
    tiny = TETODRAS[name]
    folder = make_folder(tiny, tmp_path_factory.mktemp(name))
    cfg, w = read_model(folder)
    reqs = requests_for(tiny)
    want = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    tb = replay.TraceBuilder()
    replay.whole(tb, reqs)
    replay.tail_one_by_one(tb, reqs)
    replay.portions(tb, reqs)
    replay.mixed(tb, reqs, seed=11)
    return name, tiny, folder, cfg, w, want, tb, reqs


def run_tool(folder, dtype, out, tb, page_size):
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", str(out), "--max-tokens", str(tb.max_tokens), "--page-size", str(page_size), "--max-requests", "4"]
    res = subprocess.run(cmd, input=tb.text(), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    done = [l for l in res.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(tb.steps))]


def relative_rows(out, tb, want, vocab):
    """Per way of cutting every row's root-mean-square difference from the plain implementation (the mean taken
    off) over the row's own spread, and the same between each way and the whole-request run."""
    errors, base, spread, rows_of = {}, {}, {}, {}
    for step, rows in tb.expect.items():
        got = replay.read_logits(out, step, vocab).astype(np.float64)
        assert np.isfinite(got).all()
        for r, (name, pos) in enumerate(rows):
            rows_of[(name, pos)] = got[r]
            ref = want[name[1:]][pos]
            d = got[r] - ref
            errors.setdefault(name[0], []).append(float(np.sqrt(np.mean((d - d.mean()) ** 2)) / ref.std()))
            if name[0] == "w":
                base[(name[1:], pos)] = got[r]
    for (name, pos), row in rows_of.items():
        if name[0] != "w" and (name[1:], pos) in base:
            ref = base[(name[1:], pos)]
            spread.setdefault(name[0], []).append(float(np.sqrt(np.mean((row - ref) ** 2)) / ref.std()))
    return {k: np.array(v) for k, v in errors.items()}, {k: np.array(v) for k, v in spread.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_all_ways_of_cutting(case, dtype, tmp_path):
    name, tiny, folder, cfg, w, want, tb, reqs = case
    out = tmp_path / "out"
    run_tool(folder, dtype, out, tb, tiny["page_size"])
    errors, spread = relative_rows(out, tb, want, cfg["vocab"])
    assert set(errors) == {"w", "t", "p", "m"}
    summary = {k: (round(float(np.percentile(v, 50)), 6), round(float(v.max()), 6)) for k, v in errors.items()}
    between = {k: (round(float(np.percentile(v, 50)), 6), round(float(v.max()), 6)) for k, v in spread.items()}
    print(f"\n[{name} {dtype}] against plain (median, max) {summary}; between the ways (median, max) {between}")
    limit = 2e-4 if dtype == "float32" else BF16_RMS[name]
    assert max(v.max() for v in errors.values()) < limit, summary
    assert max(v.max() for v in spread.values()) < limit, between


def test_first_tokens_one_by_one_and_long_decoding(case, tmp_path):
    """One token at a time from an empty cache and empty states (the convolution's first taps, the memories'
    first writes, the temperature's and the distance table's first steps), beside a second request that decodes
    from the middle of a page; then the last 140 tokens of the longest request one by one."""
    name, tiny, folder, cfg, w, want, _, reqs = case
    a, b = reqs["0"], reqs["1"]
    tb = replay.TraceBuilder()
    tb.step([("f1", b[:29])])
    for i in range(len(a)):
        extra = [("f1", b[29 + i:30 + i])] if 29 + i < len(b) else []
        tb.step([("f0", a[i:i + 1])] + extra)
    tb.step([], end=["f0", "f1"])
    long_one = max(reqs, key=lambda r: len(reqs[r]))
    replay.tail_one_by_one(tb, {long_one: reqs[long_one]}, tail=min(140, len(reqs[long_one]) - 3), tag="f")
    out = tmp_path / "out"
    run_tool(folder, "float32", out, tb, tiny["page_size"])
    errors, _ = relative_rows(out, tb, want, cfg["vocab"])
    assert errors["f"].max() < 2e-4, errors["f"].max()


# ----------------------------------------------------------------------------- generation through the entry point
def plain_greedy(cfg, w, prompt_ids, n):
    ids = list(prompt_ids)
    for _ in range(n):
        ids.append(int(plain.forward(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt_ids):]


@pytest.mark.parametrize("name", ["T1", "T2"])
@pytest.mark.parametrize("budget,blocks", [(256, 64), (8, 64), (7, 14)])
def test_greedy_generation_equals_plain(name, budget, blocks, tmp_path):
    """Budgets down to seven tokens a step and a pool so small that requests are preempted and computed again
    (their states start from zero again), with decode steps replayed as CUDA graphs."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = TETODRAS[name]
    folder = make_folder(tiny, tmp_path)
    cfg, w = read_model(folder)
    prompts = [prompt(i, n, cfg["vocab"]) for i, n in enumerate((5, 27, 53, 1))]
    want = [plain_greedy(cfg, w, p, 12) for p in prompts]
    llm = LLM(str(folder), dtype="float32", max_model_len=128, num_kv_blocks=blocks, block_size=tiny["page_size"],
              max_num_batched_tokens=budget, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    llm.cache.audit()
    assert all(v == blocks for v in llm.cache.free_pages().values())


def test_a_model_of_recurrent_layers_alone(tmp_path):
    """No attention: the cache manager has no group of pages at all and only the state slots."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    from tiny_tetodra import delta
    from tiny_llm_infer_b200.config.tetodra import TetodraConfig
    tiny = dict(cfg=TetodraConfig(vocab=150, width=64, embedding_scale=1.5, norm_eps=1e-5, residual_mult=0.9, layers=(
        delta(2, 1, 24, 16, 3, ff=80), delta(4, 4, 8, 8, 2))), seed=31, std=0.1, norm_range=(0.7, 1.3))
    folder = make_folder(tiny, tmp_path)
    cfg, w = read_model(folder)
    prompts = [prompt(i, n, cfg["vocab"]) for i, n in enumerate((19, 3, 40))]
    want = [plain_greedy(cfg, w, p, 10) for p in prompts]
    llm = LLM(str(folder), dtype="float32", max_model_len=96, num_kv_blocks=8, block_size=16,
              max_num_batched_tokens=16, max_num_seqs=2)
    assert not llm.cache.groups
    outs = llm.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    llm.cache.audit()


def test_long_decoding_in_bfloat16_through_graphs(tmp_path):
    """Sixty tokens each for three requests, decode steps replayed as CUDA graphs, bfloat16 kernels: every token
    is the plain implementation's choice given the same beginning, or within a near-tie of it."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = TETODRAS["T3"]
    folder = make_folder(tiny, tmp_path)
    cfg, w = read_model(folder)
    prompts = [prompt(i, n, cfg["vocab"]) for i, n in enumerate((60, 9, 190))]
    llm = LLM(str(folder), dtype="bfloat16", max_model_len=256, num_kv_blocks=24, block_size=32,
              max_num_batched_tokens=64, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=60, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ids = list(p) + list(o.token_ids)
        logits = plain.forward(cfg, w, ids[:-1]).numpy()
        near = [logits[len(p) - 1 + i][tok] >= logits[len(p) - 1 + i].max() - 0.15 * logits[len(p) - 1 + i].std()
                for i, tok in enumerate(o.token_ids)]
        assert sum(near) >= 0.9 * len(near), near


def test_command_line_writes_and_runs_a_model(tmp_path):
    """``bin/model_main``: a random Tetodra model from its config.json, greedy tokens equal to the plain
    implementation's in float32, and seeded sampling that repeats itself."""
    tiny = TETODRAS["T2"]
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny["cfg"].to_dict()))
    folder = tmp_path / "model"
    tool = [sys.executable, str(ROOT / "bin" / "model_main")]
    res = subprocess.run(tool + ["--write-random-model", str(folder), "--config", str(cfg_path), "--random-weights", "21",
                                 "--weight-std", "0.07"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    cfg, w = read_model(folder)
    prompts = [prompt(40 + i, n, cfg["vocab"]) for i, n in enumerate((9, 31))]
    ids = [a for p in prompts for a in ("--prompt-ids", ",".join(map(str, p)))]
    common = tool + ["--infer", "--model", str(folder), "--max-seq-len", "128", "--max-new-tokens", "7"] + ids
    res = subprocess.run(common + ["--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    got = [[int(x) for x in line.split(",")] for line in res.stdout.strip().splitlines()[-2:]]
    assert got == [plain_greedy(cfg, w, p, 7) for p in prompts]
    draws = []
    for _ in range(2):
        res = subprocess.run(common + ["--dtype", "bfloat16", "--temperature", "0.8", "--top-p", "0.9", "--seed", "5"],
                             capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stderr[-2000:]
        draws.append(res.stdout.strip().splitlines()[-2:])
    assert draws[0] == draws[1]
