"""Pevolorn on the GPU against the plain implementation (``plain_pevolorn.py``).

Each mechanism alone, as the registered part or kernel with sizes of its own: the norm of a weighted sum that
becomes the stream; the router over all experts with correction, groups and identity experts, and the mixture
around it on every product kernel; the latent attention with direct queries, a writer and a layer that borrows
its cache; the attention with biases, a rotation of part of a head, unit queries and keys, a capped score and a
gate per head, over scrambled pages that hold other requests' leftovers, with inputs shaped so that single keys
far back, at page borders and next to the query stand out; the state space, whole, in portions down to one
token, side by side and in slots that are used again, with heads slow enough that the first tokens still show at
the end.  Then whole models through ``bin/trace_run`` in every way of cutting, the first tokens one by one, long
decoding, and greedy generation through the engine's entry point under budgets and starved pools.

Tolerances, as a row's root-mean-square difference (its mean taken off) over the row's own spread: float32 2e-4
against the plain implementation and between the ways of cutting; bfloat16 three times what a B200 shows per
configuration."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_pevolorn as plain
import replay
from test_tetodra_gpu import (Bench, build_part, echo_inputs, make_ctx, read_model, relative_rows, run_tool,
                              tie_keys_to_queries, whole_then_portions)
from tiny_pevolorn import PEVOLORNS, make_folder, prompt, requests_for

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
F64 = torch.float64


# ----------------------------------------------------------------------------- the norm of a sum as the stream
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,n,bias", [(100, 2, True), (192, 1, False), (4104, 2, True), (36, 0, False), (328, 3, False)])
def test_norm_of_a_weighted_sum_becomes_the_stream(dtype, width, n, bias):
    from tiny_llm_infer_b200 import ops
    torch.manual_seed(width)
    h = torch.randn(11, width, device=DEV) * 3 + 1.5
    deltas = [(torch.randn(11, width, device=DEV) * 4).to(dtype) for _ in range(n)]
    coefs = [1.2, -0.7, 0.4][:n]
    gain = torch.rand(width, device=DEV) + 0.5
    b = torch.randn(width, device=DEV) if bias else None
    total = 2.5 * h.double()
    for d, c in zip(deltas, coefs):
        total = total + c * d.double()
    if bias:
        total = total + b.double()
    want = plain.rms_unit(total, 3e-6) * gain.double()
    out = torch.empty(11, width, dtype=dtype, device=DEV)
    ops.sum_rmsnorm(h, deltas, coefs, 2.5, gain, 3e-6, out, bias=b)
    assert (h.double() - want).abs().max() < 2e-5                           # the stream itself stays float32
    assert (out.double() - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.03)


def test_blocks_that_norm_after_the_sum_hand_the_stream_on():
    """The part's own face: a gain stored around zero, the stream copy between blocks, and the last norm that
    takes the copy for nothing left to add."""
    from tiny_llm_infer_b200.parts.norm import RMSNorm, StreamCopy
    norm = RMSNorm(72, 1e-5, torch.bfloat16, DEV, name="n", offset=1.0)
    w = torch.randn(72) * 0.2
    norm.load({"n": w.to(torch.bfloat16).to(DEV)})
    h = torch.randn(5, 72, device=DEV)
    d = torch.randn(5, 72, device=DEV).to(torch.bfloat16)
    want = plain.offset_norm(3.0 * h.double() + d.double(), w.to(torch.bfloat16).double().to(DEV), 1e-5)
    x = norm.of_sum(h, 3.0, [d], [1.0])
    assert (h.double() - want).abs().max() < 2e-5 and (x.double() - want).abs().max() < 0.03
    last = norm.forward(h, StreamCopy(x), rows=torch.tensor([4, 1], dtype=torch.int32, device=DEV))
    again = plain.offset_norm(want, w.to(torch.bfloat16).double().to(DEV), 1e-5)
    assert (last.double() - again[[4, 1]]).abs().max() < 0.03


# ----------------------------------------------------------------------------- the router and the mixture
ROUTER_CASES = [dict(E=6, I=2, top=2, count=4, keep=2), dict(E=5, I=0, top=3, count=1, keep=1),
                dict(E=15, I=3, top=3, count=6, keep=2), dict(E=4, I=2, top=2, count=3, keep=1),
                dict(E=61, I=3, top=8, count=8, keep=4), dict(E=250, I=6, top=6, count=16, keep=3),
                dict(E=7, I=1, top=1, count=2, keep=2)]


@pytest.mark.parametrize("case", ROUTER_CASES, ids=lambda c: f"e{c['E']}i{c['I']}t{c['top']}g{c['count']}k{c['keep']}")
def test_router_over_all_experts(case):
    """The kernel's choice against the plain router on rows of logits of several units, corrections as large as
    the scores (so that the choice and the weights part ways) and negative choice scores."""
    from tiny_llm_infer_b200 import ops
    total = case["E"] + case["I"]
    g = torch.Generator().manual_seed(total)
    z = torch.randn(700, total, generator=g, dtype=F64) * 2.0
    corr = torch.randn(total, generator=g, dtype=F64) * (2.0 / total) - 1.0 / total
    w = {"r.router": torch.eye(total, dtype=F64), "r.correction": corr}
    r = dict(experts=case["E"], identity=case["I"], top=case["top"], groups=dict(count=case["count"], keep=case["keep"]))
    z32 = z.float()
    chosen, weights = plain.route(z32.double(), w, "r.", r)
    margin = plain.router_margin(z32.double(), w, "r.", r)
    ids, wts = ops.moe_route_grouped(z32.to(DEV), case["top"], "softmax", corr.float().to(DEV), case["count"], case["keep"])
    sure = margin > 1e-4
    assert sure.float().mean() > 0.9
    got = ids.cpu().long().sort(-1)
    want = chosen.sort(-1)
    assert torch.equal(got.values[sure], want.values[sure])
    gw = torch.gather(wts.cpu().double(), 1, got.indices)
    ww = torch.gather(weights, 1, want.indices)
    assert (gw[sure] - ww[sure]).abs().max() < 1e-6
    assert (corr < 0).any() and (chosen >= case["E"]).any() == (case["I"] > 0)


MIXTURE_CASES = [dict(hidden=96, E=6, I=2, top=2, count=4, keep=2, ff=48, shared=64, rows=37),
                 dict(hidden=100, E=5, I=0, top=3, count=1, keep=1, ff=30, shared=None, rows=9),
                 dict(hidden=128, E=9, I=3, top=4, count=4, keep=3, ff=64, shared=136, rows=1500),
                 dict(hidden=64, E=4, I=2, top=2, count=3, keep=1, ff=12, shared=50, rows=3)]


@pytest.mark.parametrize("case", MIXTURE_CASES, ids=lambda c: f"h{c['hidden']}e{c['E']}i{c['I']}r{c['rows']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixture_with_identity_experts(case, dtype):
    """The registered part against the plain mixture: few rows (tiles of 64 on mma.sync, or one thread per output),
    many rows (the grouped tcgen05 product, squared ReLU in its epilogue), rows whose router is decisive."""
    from tiny_llm_infer_b200.engine.runner import strict_float32
    from tiny_llm_infer_b200.parts.registry import lookup
    from tiny_llm_infer_b200.parts.spec import PartSpec
    strict_float32()
    hidden = case["hidden"]
    shared = None
    if case["shared"]:
        shared = PartSpec("mlp", dict(hidden_size=hidden, intermediate_size=case["shared"], activation="relu2",
                                      names=("up", "down")), "shared.")
    params = dict(hidden_size=hidden, experts=case["E"], top=case["top"], expert_size=case["ff"], activation="relu2",
                  router_scores="softmax_all", weight_on="output", shared=shared, gated=False, names=("up", "down"),
                  correction=True, groups=(case["count"], case["keep"]), identity=case["I"])
    cls = lookup("feed_forward", "moe")
    g = torch.Generator().manual_seed(hidden + case["rows"])
    w = {}
    for name, spec in cls.param_specs(**params).items():
        scale = {"router": 3.0 / hidden ** 0.5, "correction": 0.1}.get(name, 0.25)
        w[name] = (torch.randn(spec.shape, generator=g) * scale).to(dtype)
    part = cls(dtype=dtype, device=DEV, **params)
    part.load({k: v.to(DEV) for k, v in w.items()})
    w64 = {"m." + k: v.double() for k, v in w.items()}
    x = torch.randn(case["rows"], hidden, generator=g).to(dtype)
    mlp = dict(router=dict(experts=case["E"], identity=case["I"], top=case["top"], groups=dict(count=case["count"], keep=case["keep"])),
               shared=dict(ff=case["shared"]) if case["shared"] else None)
    want = plain.mixture(x.double(), w64, "m.", mlp)
    sure = plain.router_margin(x.double(), w64, "m.", mlp["router"]) > (1e-4 if dtype == torch.float32 else 0.05)
    assert sure.float().mean() > 0.5
    got = part.forward(x.to(DEV), None).double().cpu()
    if case["rows"] >= 1024 and dtype == torch.bfloat16:
        from tiny_llm_infer_b200 import ops
        ops.check_error_word(torch.device(DEV))
    err = ((got - want)[sure].abs().max() / want.abs().max()).item()
    assert err < (3e-5 if dtype == torch.float32 else 0.03), err
    if case["I"] and case["rows"] >= 30:
        chosen, _ = plain.route(x.double(), w64, "m.", mlp["router"])
        assert (chosen >= case["E"]).any()


def test_squared_relu_in_the_products():
    """act = max(x, 0)^2 in the epilogues of the weight-streaming product (few rows), of the tcgen05 product (many)
    and in the kernel of its own (between them)."""
    from tiny_llm_infer_b200 import ops
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(512, 256, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    for rows in (3, 40, 2048):
        x = torch.randn(rows, 256, generator=g).to(torch.bfloat16).to(DEV)
        want = torch.clamp(x.double() @ w.double().T, min=0.0) ** 2
        got = ops.linear_act(x, w, "relu2", torch.bfloat16).double()
        assert (got - want).abs().max() < 0.02 * want.abs().max()
    ops.check_error_word(torch.device(DEV))


# ----------------------------------------------------------------------------- latent attention: a writer and a borrower
LATENT_CASES = [dict(H=4, dn=24, dr=16, dv=32, rank=48, dims=16, base=10000.0, scale=0.3, page=16, H2=2, dn2=16, dv2=8),
                dict(H=3, dn=10, dr=6, dv=6, rank=20, dims=4, base=5000.0, scale=0.6, page=8, H2=1, dn2=6, dv2=10),
                dict(H=4, dn=64, dr=32, dv=64, rank=96, dims=32, base=20000.0, scale=0.12, page=32, H2=8, dn2=32, dv2=32),
                dict(H=2, dn=32, dr=8, dv=40, rank=136, dims=8, base=1000.0, scale=0.13, page=16, H2=5, dn2=12, dv2=20)]


@pytest.mark.parametrize("case", LATENT_CASES, ids=lambda c: f"h{c['H']}n{c['dn']}r{c['dr']}k{c['rank']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_with_a_borrowed_cache(case, dtype):
    """One layer writes [latent | rotated key part] into scrambled pages; a second layer with other heads and
    widths and no compression of its own reads the same pages with its own matrices and its own input.  Whole
    requests side by side, then portions of every size in pages and slots that were used."""
    from tiny_llm_infer_b200.engine.runner import strict_float32
    from tiny_llm_infer_b200.cache.manager import LayerCacheView
    strict_float32()
    hidden = 88
    common = dict(hidden_size=hidden, rot_dim=case["dr"], q_rank=0, kv_rank=case["rank"], scale=case["scale"], norm_eps=2e-6,
                  rot_base=case["base"], rot_dims=case["dims"], rotation="half", output_gate=True, gate_per_head=True)
    writer, w_w = build_part("latent_attention", dict(common, heads=case["H"], plain_dim=case["dn"], value_dim=case["dv"]),
                             dtype, seed=case["rank"], stds={"q": 0.1, "dkv": 0.5})
    reader, w_r = build_part("latent_attention", dict(common, heads=case["H2"], plain_dim=case["dn2"], value_dim=case["dv2"],
                                                      borrows_cache=True), dtype, seed=case["rank"] + 1, stds={"q": 0.1})
    assert "dkv" not in type(reader).param_specs(**dict(common, heads=1, plain_dim=4, value_dim=4, borrows_cache=True))
    lengths = (200, 61, 1)
    g = torch.Generator().manual_seed(case["H"])
    xs = [torch.randn(L, hidden, generator=g).to(dtype) for L in lengths]
    ys = [torch.randn(L, hidden, generator=g).to(dtype) for L in lengths]          # the borrowing layer's own input
    m_w = dict(heads=case["H"], dim=case["dn"], rot_dim=case["dr"], vdim=case["dv"], kv_rank=case["rank"], scale=case["scale"],
               rot=dict(base=case["base"], dims=case["dims"]))
    m_r = dict(m_w, heads=case["H2"], dim=case["dn2"], vdim=case["dv2"])
    lat = [plain.latent_keys(x.double(), w_w, "m.", m_w, 2e-6) for x in xs]
    want_w = [plain.latent_attention(x.double(), w_w, "m.", m_w, 2e-6, l) for x, l in zip(xs, lat)]
    want_r = [plain.latent_attention(y.double(), w_r, "m.", m_r, 2e-6, l) for y, l in zip(ys, lat)]
    # far keys carry weight: without the first forty tokens the last answer differs
    cut = plain.latent_attention(xs[0][40:].double(), w_w, "m.", m_w, 2e-6, plain.latent_keys(xs[0][40:].double(), w_w, "m.", m_w, 2e-6))
    assert (cut[-1] - want_w[0][-1]).abs().max() > 1e-3 * want_w[0].abs().max()
    bench = Bench(writer, dtype, xs, want_w, page=case["page"])
    view_r = LayerCacheView(kv=None, block_table=bench.view.block_table, page_size=case["page"], writes=False, state=None,
                            window=None, planes=bench.view.planes)
    worst_r = [0.0]
    step = bench.step

    def both(rows):
        err = step(rows)                                        # the writer first, as the run order has it
        y = torch.cat([ys[r][p0:p0 + n] for r, _, p0, n in rows]).to(dtype).to(DEV)
        got = reader.forward(y, make_ctx([(slot, p0, n) for _, slot, p0, n in rows]), view_r).double().cpu()
        expect = torch.cat([want_r[r][p0:p0 + n] for r, _, p0, n in rows])
        worst_r[0] = max(worst_r[0], ((got - expect).abs().max() / expect.abs().max()).item())
        return err
    bench.step = both
    whole, cutup = whole_then_portions(bench, lengths)
    limit = 3e-5 if dtype == torch.float32 else 0.06
    assert whole < limit and cutup < limit and worst_r[0] < limit, (whole, cutup, worst_r[0])
    with pytest.raises(ValueError, match="must not write"):
        reader.forward(ys[2].to(DEV), make_ctx([(0, 0, 1)]), bench.view)


# ----------------------------------------------------------------------------- the attention beside the state space
GROUPED_CASES = [dict(H=4, G=2, dk=32, dv=24, scale=4.0, cap=12.0, base=50000.0, dims=16, page=16),
                 dict(H=3, G=1, dk=10, dv=6, scale=5.0, cap=None, base=77.0, dims=4, page=8),
                 dict(H=8, G=2, dk=128, dv=64, scale=6.0, cap=15.0, base=400000.0, dims=96, page=32),
                 dict(H=1, G=1, dk=20, dv=12, scale=3.0, cap=2.0, base=250000.0, dims=20, page=16),
                 dict(H=2, G=2, dk=64, dv=64, scale=8.0, cap=30.0, base=10000.0, dims=32, page=16),
                 dict(H=6, G=3, dk=44, dv=80, scale=5.0, cap=8.0, base=300.0, dims=2, page=16)]


@pytest.mark.parametrize("defer", [True, False], ids=["bias_in_the_sum", "bias_in_the_product"])
@pytest.mark.parametrize("case", GROUPED_CASES, ids=lambda c: f"h{c['H']}g{c['G']}k{c['dk']}v{c['dv']}r{c['dims']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_biases_unit_keys_cap_and_a_gate_per_head(case, dtype, defer):
    """Queries and keys are unit vectors, so a score is at most scale * dim: scales of several units and queries
    that echo one key let that key stand out (and the cap bends exactly those scores)."""
    from tiny_llm_infer_b200.engine.runner import strict_float32
    from tiny_llm_infer_b200.parts.spec import PartSpec
    strict_float32()
    if defer and case["H"] not in (4, 3, 8):
        pytest.skip("the other way of adding the output's bias is covered by the first cases")
    H, G, dk, dv, hidden = case["H"], case["G"], case["dk"], case["dv"], 104
    scale = case["scale"] / dk                                  # unit vectors have length sqrt(dk)
    params = dict(hidden_size=hidden, q_heads=H, kv_heads=G, key_dim=dk, value_dim=dv, scale=scale, unit_norm_eps=2e-6,
                  softcap=case["cap"], output_gate=True, gate_per_head=True, biases=True, defer_output_bias=defer,
                  position=PartSpec("rotary_half", dict(head_dim=dk, theta=case["base"], rotary_dim=case["dims"])))

    def change(w):
        tie_keys_to_queries(H, G, dk, hidden)(w)
        for kv in range(G):                                   # the biases tied like the matrices
            first = kv * (H // G)
            w["k.b"][kv * dk:(kv + 1) * dk] = w["q.b"][first * dk:(first + 1) * dk]
        w["q.b"] *= 0.3
        w["k.b"] *= 0.3
    part, w64 = build_part("biased_attention", params, dtype, seed=dk + dv, change=change, stds={"q": 0.3, "k": 0.3, "g": 0.5})
    lengths = (290, 75, 1)
    xs = [x.to(dtype) for x in echo_inputs(lengths, hidden, case["page"], seed=H)]
    m = dict(heads=H, kv_heads=G, dim=dk, vdim=dv, scale=scale, softcap=case["cap"], rot=dict(base=case["base"], dims=case["dims"]))
    want = [plain.gated_softcap_attention(x.double(), w64, "m.", m, 2e-6) for x in xs]
    if defer:                                                   # the block's sum kernel adds it: the part leaves it out
        assert part.deferred_bias is not None and part.out_bias is None
        want = [x - w64["m.o.b"] for x in want]
    cut = plain.gated_softcap_attention(xs[0][40:].double(), w64, "m.", m, 2e-6)
    full = plain.gated_softcap_attention(xs[0].double(), w64, "m.", m, 2e-6)
    if case["cap"] is None or case["cap"] > 4:                  # (a low cap flattens every score: no key stands out)
        assert (cut[-1] - full[-1]).abs().max() > 0.01 * full.abs().max()
    whole, cutup = whole_then_portions(Bench(part, dtype, xs, want, page=case["page"]), lengths)
    limit = 3e-5 if dtype == torch.float32 else 0.06
    assert whole < limit and cutup < limit, (whole, cutup)


SPACE_CASES = [dict(H=4, P=8, N=16, G=1, taps=4, parts=2), dict(H=5, P=6, N=10, G=5, taps=2, parts=3),
               dict(H=4, P=64, N=64, G=2, taps=3, parts=4), dict(H=3, P=10, N=6, G=1, taps=5, parts=1, reach=120),
               dict(H=8, P=16, N=128, G=4, taps=4, parts=2), dict(H=2, P=24, N=32, G=2, taps=1, parts=1),
               dict(H=8, P=32, N=48, G=2, taps=3, parts=1)]


@pytest.mark.parametrize("case", SPACE_CASES, ids=lambda c: f"h{c['H']}p{c['P']}n{c['N']}g{c['G']}t{c['taps']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_state_space(case, dtype):
    """Every second head decays by a few thousandths a token, so that the first tokens still show after hundreds;
    step sizes between a hundredth and several units (no clamp either way)."""
    from tiny_llm_infer_b200.engine.runner import strict_float32
    strict_float32()
    hidden = 80
    params = dict(hidden_size=hidden, heads=case["H"], head_dim=case["P"], state=case["N"], groups=case["G"],
                  conv_taps=case["taps"], norm_groups=case["parts"], norm_eps=1e-5)

    def change(w):
        w["A_log"][::2] -= 5.0
        w["dt_bias"] = w["dt_bias"] * 3.0
        w["in"][-case["H"]:] *= 2.0                          # the step sizes' logits
    part, w64 = build_part("state_space", params, dtype, seed=case["N"] + case["P"], change=change, stds={"in": 0.15, "conv": 0.6})
    m = dict(heads=case["H"], vdim=case["P"], state=case["N"], groups=case["G"], conv=case["taps"], norm_groups=case["parts"])
    fn = lambda x: plain.state_space(x, w64, "m.", m, 1e-5)
    lengths = (230, 61, 1)
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(L, hidden, generator=g).to(dtype) for L in lengths]
    want = [fn(x.double()) for x in xs]
    reach = case.get("reach", 200)
    short = fn(xs[0][lengths[0] - reach:].double())
    assert (short[-1] - want[0][-1]).abs().max() > 1e-3 * want[0].abs().max()
    dt = torch.nn.functional.softplus(xs[0].double() @ w64["m.in"][-case["H"]:].T + w64["m.dt_bias"])
    assert dt.min() < 0.05 and dt.max() > 3.0
    whole, cutup = whole_then_portions(Bench(part, dtype, xs, want), lengths)
    limit = 3e-5 if dtype == torch.float32 else 0.06
    assert whole < limit and cutup < limit, (whole, cutup)


# ----------------------------------------------------------------------------- whole models, every way of cutting
BF16_RMS = {"V1": 0.3, "V2": 0.3, "V3": 0.6}      # V3 (half the stream kept per sum, five layers) shows up to 0.2


@pytest.fixture(scope="module", params=sorted(PEVOLORNS))
def case(request, tmp_path_factory):
    name = request.param
    tiny = PEVOLORNS[name]
    folder = make_folder(tiny, tmp_path_factory.mktemp(name))
    cfg, w = read_model(folder)
    reqs = {rid: plain.decisive_tokens(cfg, w, toks, seed=int(rid)) for rid, toks in requests_for(tiny).items()}
    want = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    tb = replay.TraceBuilder()
    replay.whole(tb, reqs)
    replay.tail_one_by_one(tb, reqs)
    replay.portions(tb, reqs)
    replay.mixed(tb, reqs, seed=11)
    return name, tiny, folder, cfg, w, want, tb, reqs


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
    """One token at a time from an empty cache and empty states (the convolution's first taps, the state's first
    writes, the rotation's first angles), beside a second request that decodes from the middle of a page; then the
    last 140 tokens of the longest request one by one."""
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


def decisive_greedy(cfg, w, seeds_and_lengths, n):
    """Prompts whose greedy continuation of ``n`` tokens meets no near-tie of a router or of the last argmax."""
    prompts, wants = [], []
    for seed, length in seeds_and_lengths:
        for attempt in range(40):
            p = plain.decisive_tokens(cfg, w, prompt(seed + 100 * attempt, length, cfg["vocab"]), seed=seed)
            out = plain_greedy(cfg, w, p, n)
            gaps = []
            logits = plain.forward(cfg, w, p + out, gaps_out=gaps)[len(p) - 1:-1]
            top2 = logits.topk(2, dim=-1).values
            if (top2[:, 0] - top2[:, 1]).min() > 1e-3 and torch.stack(gaps).min() > 1e-3:
                break
        prompts.append(p)
        wants.append(out)
    return prompts, wants


@pytest.mark.parametrize("name", ["V1", "V2"])
@pytest.mark.parametrize("budget,blocks", [(256, 64), (8, 64), (7, 14)])
def test_greedy_generation_equals_plain(name, budget, blocks, tmp_path):
    """Budgets down to seven tokens a step and a pool so small that requests are preempted and computed again
    (their states start from zero again), with decode steps replayed as CUDA graphs."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = PEVOLORNS[name]
    folder = make_folder(tiny, tmp_path)
    cfg, w = read_model(folder)
    prompts, want = decisive_greedy(cfg, w, [(0, 5), (1, 27), (2, 53), (3, 1)], 12)
    llm = LLM(str(folder), dtype="float32", max_model_len=128, num_kv_blocks=blocks, block_size=tiny["page_size"],
              max_num_batched_tokens=budget, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    llm.cache.audit()
    assert all(v == blocks for v in llm.cache.free_pages().values())


def test_long_decoding_in_bfloat16_through_graphs(tmp_path):
    """Sixty tokens each for three requests, decode steps replayed as CUDA graphs, bfloat16 kernels: every token
    is the plain implementation's choice given the same beginning, or within a near-tie of it."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = PEVOLORNS["V3"]
    folder = make_folder(tiny, tmp_path)
    cfg, w = read_model(folder)
    prompts = [prompt(i, n, cfg["vocab"]) for i, n in enumerate((60, 9, 150))]
    llm = LLM(str(folder), dtype="bfloat16", max_model_len=256, num_kv_blocks=24, block_size=32,
              max_num_batched_tokens=64, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=60, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ids = list(p) + list(o.token_ids)
        logits = plain.forward(cfg, w, ids[:-1]).numpy()
        near = [logits[len(p) - 1 + i][tok] >= logits[len(p) - 1 + i].max() - 0.15 * logits[len(p) - 1 + i].std()
                for i, tok in enumerate(o.token_ids)]
        assert sum(near) >= 0.85 * len(near), near


def test_command_line_writes_and_runs_a_model(tmp_path):
    """``bin/model_main``: a random Pevolorn model from its config.json, greedy tokens equal to the plain
    implementation's in float32, and seeded sampling that repeats itself."""
    tiny = PEVOLORNS["V2"]
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny["cfg"].to_dict()))
    folder = tmp_path / "model"
    tool = [sys.executable, str(ROOT / "bin" / "model_main")]
    res = subprocess.run(tool + ["--write-random-model", str(folder), "--config", str(cfg_path), "--random-weights", "21",
                                 "--weight-std", "0.07"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    cfg, w = read_model(folder)
    prompts, want = decisive_greedy(cfg, w, [(40, 9), (41, 31)], 7)
    ids = [a for p in prompts for a in ("--prompt-ids", ",".join(map(str, p)))]
    common = tool + ["--infer", "--model", str(folder), "--max-seq-len", "128", "--max-new-tokens", "7"] + ids
    res = subprocess.run(common + ["--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    got = [[int(x) for x in line.split(",")] for line in res.stdout.strip().splitlines()[-2:]]
    assert got == want
    draws = []
    for _ in range(2):
        res = subprocess.run(common + ["--dtype", "bfloat16", "--temperature", "0.8", "--top-p", "0.9", "--seed", "5"],
                             capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stderr[-2000:]
        draws.append(res.stdout.strip().splitlines()[-2:])
    assert draws[0] == draws[1]
