#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode and prefill throughput of a Qwen3-8B-shaped
model with random weights, in bfloat16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference] [--model 8b|0.6b|32b] [--mixed]

A "step" is one decode step of a batch of 8 requests.  The headline ``value`` is decoded
tokens per second timed on the device (CUDA events around each step); ``e2e`` is the same
through the Python entry point (``LLMEngine.step``), host token ids in and out, timed by
the wall clock.  One JSON line is printed.  The sizes are those of Qwen3-8B
(the benchmark configuration); every request stands at a context of about 4096 tokens while it decodes
(the prompts are really prefilled, in portions of 2048 tokens, outside the timed region).

Beside the headline, in ``points`` (flat, numbers only): decode at batch 1 and 64 at the same context;
the reference's own benchmark workload (``p128_*``: 128-token prompts, 128 outputs, batch 1 / 8 / 64:
the decode steps alone timed on the device with their share of the HBM peak, and output tokens per
second end to end with the prompts inside the timed region, median of five runs after three
warm-ups); the mixed continuous-batching run that goes with the Qwen3-0.6B sizes.  ``prefill`` is one
prompt of 2048 tokens.  ``check``: the logits of the model that was timed, bfloat16 kernels against
the float32 path under four ways of cutting; a mismatch ends the run with an error line and code 1.

``--impl reference`` runs the unmodified reference (built by baseline/reference_arm/build.py into
baseline/_ref/) on the same sizes and the same decode workload through its own LLMEngine, and its own
``model_main --bench`` on the 128-token workload; it prints the same line with ``"impl": "reference"``,
or ``{"impl": "reference", "unavailable": why}``.

For more than one GPU this engine has nothing to run: it prints one line and exits 2.
"""
import argparse
import json
import math
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# the benchmark configuration: Qwen3-8B shape, random weights N(0, 0.02), untied head, page 16
QWEN3_8B = dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, vocab_size=151936, max_position_embeddings=40960,
                rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
# the two other sizes the reference is quoted on: the 0.6B shape (tied head) and the 32B shape (--model)
QWEN3_06B = dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=128, vocab_size=151936, max_position_embeddings=40960,
                 rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)
QWEN3_32B = dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                 num_key_value_heads=8, head_dim=128, vocab_size=151936, max_position_embeddings=40960,
                 rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
MODELS = {"8b": ("Qwen3-8B shape", QWEN3_8B), "0.6b": ("Qwen3-0.6B shape", QWEN3_06B),
          "32b": ("Qwen3-32B shape", QWEN3_32B)}
CONTEXT = 4096
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                   "source": "measured"}
            if raw.get("bf16_tflops_sustained"):          # a seconds-long loop under the power cap
                out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            return out
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,clocks.mem,power.draw")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self, windows):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        mhz, max_mhz, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for a, b, what in windows:                 # per timed region, for the log
            lines = [[p.strip() for p in line.split(",")] for t, line in self.samples if a <= t <= b]
            inside = [int(p[0]) for p in lines if p[0].isdigit()]
            if inside:
                mem = sorted({p[6] for p in lines if len(p) > 7})
                watts = [float(p[7]) for p in lines if len(p) > 7 and p[7].replace(".", "", 1).isdigit()]
                print(f"[bench] clocks during {what}: SM median {int(statistics.median(inside))} MHz, min {min(inside)}; "
                      f"memory {'/'.join(mem)} MHz; {int(statistics.median(watts)) if watts else '?'} W; {len(inside)} samples",
                      file=sys.stderr, flush=True)
        for t, line in self.samples:
            if windows and not any(a <= t <= b for a, b, _ in windows):
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                mhz.append(int(parts[0]))
                max_mhz = max(max_mhz, int(parts[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, parts[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max_mhz or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ---------------------------------------------------------------------- the reference arm
REF_BIN = ROOT / "baseline" / "_ref" / "bin"


def _unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def _reference_binaries():
    """The reference built by baseline/reference_arm/build.py (its sources unchanged, three stand-in
    headers); built now if its sources are at hand and the binaries are not."""
    need = [REF_BIN / "decode_main", REF_BIN / "model_main"]
    if all(p.is_file() for p in need):
        return need, None
    import os
    src = Path(os.environ.get("TLLM_REFERENCE", str(ROOT.parent / "reference")))    # or a folder beside this one
    if not (src / "model" / "model_main.cpp").is_file():
        return None, (f"the reference is not built (no {REF_BIN}) and its sources are not at {src}: "
                      "run baseline/reference_arm/build.py where they are")
    res = subprocess.run([sys.executable, str(ROOT / "baseline" / "reference_arm" / "build.py"), "--reference", str(src)],
                         capture_output=True, text=True)
    if res.returncode != 0 or not all(p.is_file() for p in need):
        return None, "building the reference failed: " + (res.stderr or res.stdout).strip().splitlines()[-1][:200]
    return need, None


def _write_reference_model(folder: Path, sizes: dict, seed: int = 0):
    """config.json, tokenizer.json and model.safetensors (FP16, the reference's storage type) of the
    given sizes with random weights N(0, 0.02) and norm gains U[0.8, 1.2], written with torch and the
    safetensors library alone.  The reference's tokenizer must know every id it may have to print
    (layers/src/encode.cpp:311-315): the vocabulary is t0, t1, ..."""
    import torch
    from safetensors.torch import save_file
    folder.mkdir(parents=True, exist_ok=True)
    cfg = dict(sizes, model_type="qwen3", architectures=["Qwen3ForCausalLM"], torch_dtype="float16")
    (folder / "config.json").write_text(json.dumps(cfg))
    vocab, hidden, inter = sizes["vocab_size"], sizes["hidden_size"], sizes["intermediate_size"]
    q = sizes["num_attention_heads"] * sizes["head_dim"]
    kv = sizes["num_key_value_heads"] * sizes["head_dim"]
    (folder / "tokenizer.json").write_text(json.dumps(
        {"model": {"vocab": {f"t{i}": i for i in range(vocab)}, "merges": []}, "added_tokens": []}))
    gen = torch.Generator(device="cuda").manual_seed(seed)

    def normal(*shape):
        return (torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32) * 0.02).to(torch.float16).cpu()

    def gain(n):
        return (torch.rand(n, generator=gen, device="cuda") * 0.4 + 0.8).to(torch.float16).cpu()

    tensors = {"model.embed_tokens.weight": normal(vocab, hidden), "model.norm.weight": gain(hidden)}
    if not sizes.get("tie_word_embeddings"):
        tensors["lm_head.weight"] = normal(vocab, hidden)     # present as in a real checkpoint; the reference never reads it
    for i in range(sizes["num_hidden_layers"]):
        p = f"model.layers.{i}."
        tensors.update({
            p + "input_layernorm.weight": gain(hidden), p + "post_attention_layernorm.weight": gain(hidden),
            p + "self_attn.q_proj.weight": normal(q, hidden), p + "self_attn.k_proj.weight": normal(kv, hidden),
            p + "self_attn.v_proj.weight": normal(kv, hidden), p + "self_attn.o_proj.weight": normal(hidden, q),
            p + "self_attn.q_norm.weight": gain(sizes["head_dim"]), p + "self_attn.k_norm.weight": gain(sizes["head_dim"]),
            p + "mlp.gate_proj.weight": normal(inter, hidden), p + "mlp.up_proj.weight": normal(inter, hidden),
            p + "mlp.down_proj.weight": normal(hidden, inter)})
    save_file(tensors, str(folder / "model.safetensors"))
    del tensors
    torch.cuda.empty_cache()


def _standing_prompt_len(batch: int, steps: int, warmup: int, budget: int = 256) -> int:
    """Longest prompt with which decode_main's requests (which keep decoding while the other prompts
    are computed) stay inside CONTEXT until the timed steps are over."""
    n = CONTEXT
    while n > 1:
        budget_steps = -(-batch * n // budget)
        if n + warmup + steps + budget_steps + budget_steps // 8 + 16 <= CONTEXT:
            return n
        n -= 1
    return 1


def reference_arm(args, model_name: str, model_sizes: dict) -> int:
    """The unmodified reference on the same sizes and workload: decode steps of ``--batch`` requests
    standing at a context of about 4096 through its LLMEngine (``value`` and ``e2e``: its step() takes
    host token ids in and gives host token ids out, so the two are one number), and its own
    ``model_main --bench`` on 128-token prompts with 128 outputs (``points``)."""
    import os
    import shutil
    import tempfile
    if args.gpus != 1:
        print(f"bench.py: the reference runs on one GPU; --gpus {args.gpus} has nothing to measure")
        return 2
    bins, why = _reference_binaries()
    if bins is None:
        return _unavailable(why)
    try:
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device")
    except ImportError:
        return _unavailable("torch is needed to write the random model file")
    args.warmup = max(args.warmup, 3)
    layers = args.layers or model_sizes["num_hidden_layers"]
    sizes = dict(model_sizes, num_hidden_layers=layers)
    need_bytes = 2.2 * (layers * _layer_params(sizes) + 2 * sizes["vocab_size"] * sizes["hidden_size"]) + (1 << 30)
    base = None
    for cand in ("/dev/shm", tempfile.gettempdir()):
        try:
            if shutil.disk_usage(cand).free > need_bytes:
                base = cand
                break
        except OSError:
            continue
    if base is None:
        return _unavailable("no room for the reference's model file")
    work = Path(tempfile.mkdtemp(prefix="tllm_ref_", dir=base))
    pk = peaks()
    try:
        t0 = time.perf_counter()
        _write_reference_model(work, sizes)
        print(f"[bench] reference model written to {work} in {time.perf_counter() - t0:.1f} s", file=sys.stderr, flush=True)
        clocks = ClockSampler()
        clocks.start()
        windows = []
        vocab = sizes["vocab_size"]
        prompt_len = _standing_prompt_len(args.batch, args.steps, args.warmup)
        blocks = args.batch * (CONTEXT // PAGE) + 64
        cmd = [str(bins[0]), str(work / "model.safetensors"), str(work / "tokenizer.json"), str(args.batch),
               str(prompt_len), str(args.warmup), str(args.steps), str(CONTEXT), str(blocks), str(vocab - 1), "0"]
        w0 = time.perf_counter()
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
        windows.append((w0, time.perf_counter(), "reference decode"))
        sys.stderr.write(res.stderr[-2000:])
        if res.returncode != 0:
            return _unavailable(f"the reference's decode run ended with {res.returncode}: "
                                + (res.stderr.strip().splitlines() or ["no message"])[-1][:200])
        dec = json.loads(res.stdout.strip().splitlines()[-1])
        print(f"[bench] reference decode: {dec}", file=sys.stderr, flush=True)

        points = {}
        for b in ([1, 8, 64] if args.ref_all else [args.batch]):
            cmd = [str(bins[1]), "--bench", "--tokenizer", str(work / "tokenizer.json"), "--model",
                   str(work / "model.safetensors"), "--device", "cuda", "--num-seqs", str(b), "--min-input-len", "128",
                   "--max-input-len", "128", "--min-output-len", "128", "--max-output-len", "128", "--warmup", "3",
                   "--repeats", "5", "--max-seq-len", str(CONTEXT), "--num-kv-blocks", str(b * (256 // PAGE) + 16),
                   "--max-token-id", str(vocab - 1), "--seed", "0"]
            w0 = time.perf_counter()
            res = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
            windows.append((w0, time.perf_counter(), f"reference 128/128 b{b}"))
            rates = [float(part.split("=")[1]) for line in res.stdout.splitlines() if line.startswith("run=")
                     for part in line.split() if part.startswith("output_tokens_per_second=")]
            if res.returncode != 0 or len(rates) != 5:
                print(f"[bench] reference model_main --bench b{b} ended with {res.returncode}: {res.stderr[-400:]}",
                      file=sys.stderr, flush=True)
                continue
            points[f"p128_e2e_b{b}"] = round(statistics.median(rates), 1)
            print(f"[bench] reference 128/128 b{b}: {points[f'p128_e2e_b{b}']} output tok/s (median of 5)",
                  file=sys.stderr, flush=True)
    finally:
        shutil.rmtree(work, ignore_errors=True)

    weight_bytes = 2 * (layers * _layer_params(sizes) + vocab * sizes["hidden_size"])
    kv_per_token = 2 * sizes["num_key_value_heads"] * sizes["head_dim"] * 2 * layers
    # request i has decoded about (batch - 1 - i) / batch of the prompt steps' tokens before the timed steps
    prefill_steps = dec.get("prefill_steps", 0)
    mean_ctx = prompt_len + prefill_steps / 2.0 + args.warmup + (args.steps + 1) / 2.0
    achieved = (weight_bytes + args.batch * mean_ctx * kv_per_token) / dec["seconds"] * args.steps / 1e9
    table_entries = CONTEXT // PAGE
    record = {
        "impl": "reference",
        "metric": f"decode tok/s @ batch {args.batch} ({model_name}, context 4096, 1 B200)",
        "value": round(dec["tokens_per_second"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dec["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp16",
        "data": "synthetic (random weights N(0,0.02), uniform random token ids); the reference multiplies by the "
                "embedding matrix for the head whatever tie_word_embeddings says",
        "config": _config(model_name, args.batch, layers, model_sizes, sizes, mean_ctx, weight_bytes, pk),
        "e2e": {"value": round(dec["tokens_per_second"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": args.batch * (8 + 4 * table_entries + 20), "d2h_bytes_per_step": args.batch * 4},
        "gpu_launches": (17 * layers + 6) * args.steps,
        "prefill": None,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.stop(windows),
    }
    print(json.dumps(record))
    return 0


def _layer_params(sizes: dict) -> int:
    q = sizes["num_attention_heads"] * sizes["head_dim"]
    kv = sizes["num_key_value_heads"] * sizes["head_dim"]
    h = sizes["hidden_size"]
    return (q + 2 * kv) * h + h * q + 3 * h * sizes["intermediate_size"]


def _config(model_name, batch, layers, model_sizes, sizes, mean_ctx, weight_bytes, pk) -> dict:
    """The ``config`` of the record, the same for both arms (flat, at most 20 keys)."""
    return {"model": model_name, "global_batch": batch, "seq_len": CONTEXT, "parallelism": "single GPU",
            "layers": layers, "layers_of_model": model_sizes["num_hidden_layers"],
            "hidden_size": sizes["hidden_size"], "intermediate_size": sizes["intermediate_size"],
            "q_heads": sizes["num_attention_heads"], "kv_heads": sizes["num_key_value_heads"],
            "head_dim": sizes["head_dim"], "vocab_size": sizes["vocab_size"], "page_size": PAGE,
            "decode_context": None if mean_ctx is None else round(mean_ctx, 1), "prefill_tokens": PREFILL_TOKENS,
            "p128": "128-token prompts, 128 outputs, temperature 0.6",
            "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.1f} GB of weights per step)", "peaks": pk["source"]}


def precheck(model, cfg, sizes, device) -> dict:
    """The logits of the very model that is timed, by the bfloat16 kernels, against the float32 path
    of the same weights, on one request of 2,200 tokens and three short ones cut in four ways (whole;
    the last 32 tokens one by one, which are replayed CUDA graphs; portions of 2 to 700 tokens; mixed
    on a pool that just holds the four).  If the float32 twin of all layers does not fit beside the
    model, both are cut to the layers that do.

    Limits, as fractions of the standard deviation of a row of logits (0.9 to 1.6 at these sizes):
    a row's root-mean-square difference 0.12 and its largest difference among 151,936 entries 0.6,
    a little over twice what 36 layers of Qwen3-8B sizes show on a B200 (0.052 and 0.26; the
    difference grows with the square root of the depth: 4 layers show 0.026 and 0.13); the bfloat16
    argmax must be the float32 argmax or within 0.5 of it; the float32 ways of cutting must agree to
    1e-4 of a row's largest logit.  A kernel that loses a tile of keys, a slice of K or a page moves
    a row by its whole spread."""
    import torch

    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.config import Qwen3Config
    from tiny_llm_infer_b200.engine import ModelRunner, random_model, selfcheck

    layers = sizes["num_hidden_layers"]
    free, _ = torch.cuda.mem_get_info()
    per_layer, ends = 4 * _layer_params(sizes), 4 * 2 * sizes["vocab_size"] * sizes["hidden_size"]
    fit = int((free * 0.8 - ends - (8 << 30)) // (per_layer * 1.5))        # the twin, and the cut bfloat16 model if one is needed
    check_layers = layers if layers * per_layer + ends + (8 << 30) < free * 0.8 else max(1, min(layers, fit))
    gen = torch.Generator().manual_seed(7)
    requests = {str(i): torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()
                for i, n in enumerate((2200, 300, 150, 90))}
    wanted = {k: selfcheck.wanted_positions(len(v)) for k, v in requests.items()}

    def ways(m, dtype):
        cache = CacheManager(m.cache_needs(), PAGE, selfcheck.pages_for(requests, PAGE), max_slots=4,
                             max_seq_len=2240, dtype=dtype, device=device)
        runner = ModelRunner(m, cache, max_batch_tokens=2240)
        rows = selfcheck.CutRunner(runner, requests, wanted).all_ways(seed=3)
        runner.check_kernels()
        cache.audit()
        return rows

    cut_cfg = Qwen3Config(layer_types=("full_attention",) * check_layers, **dict(sizes, num_hidden_layers=check_layers))
    exact_model = random_model(cut_cfg, seed=0, dtype=torch.float32, device=device, std=0.02)
    exact = ways(exact_model, torch.float32)
    del exact_model
    torch.cuda.empty_cache()
    fast_model = model if check_layers == layers else random_model(cut_cfg, seed=0, dtype=torch.bfloat16, device=device, std=0.02)
    fast = ways(fast_model, torch.bfloat16)
    del fast_model
    result = selfcheck.compare(fast, exact, near_tie=0.5)
    spread32 = max(selfcheck.spread_between_ways(exact).values())
    del exact, fast
    torch.cuda.empty_cache()
    names = ("whole", "tail", "portions", "mixed")
    out = {"layers": check_layers, "rows": len(wanted["0"]) + sum(len(wanted[k]) for k in "123"),
           "max_of_row_std": round(max(result[w + ":relative"] for w in names), 4),
           "rms_of_row_std": round(max(result[w + ":rms"] for w in names), 4),
           "argmax_misses": int(sum(result[w + ":argmax_misses"] for w in names)),
           "float32_ways_relative": float(f"{spread32:.2e}")}
    out["ok"] = bool(out["max_of_row_std"] <= 0.6 and out["rms_of_row_std"] <= 0.12 and out["argmax_misses"] == 0
                     and spread32 <= 1e-4)
    return out



# ---------------------------------------------------------------------- a design beside its closest relative
DESIGN_SIZES = {
    # width, heads, kv heads, head width, dense ff; experts, top, expert ff, shared ff (top * expert + shared = dense ff,
    # so that a token costs the same in a mixture layer as in a dense one); chunk of the attention mask
    "1b": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=6144, experts=32, top=4, expert_ff=1024, shared_ff=2048,
               chunk=2048, layers=8, vocab=32768),
    "8b": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, experts=64, top=4, expert_ff=2048, shared_ff=4096,
               chunk=4096, layers=4, vocab=32768),
}


class _DesignHarness:
    """What the ``--design`` benches share: the timing of one call (three warm-up calls, then the median of
    ``reps`` calls with L2 flushed before each, CUDA events on the launching stream) and a model's prefill and
    decode through the engine's step function."""

    def __init__(self, args):
        import torch
        from tiny_llm_infer_b200 import ops
        assert torch.cuda.is_available(), "bench.py needs a CUDA device"
        self.device = "cuda:0"
        self.pk = peaks()
        ops.lib()
        self.gen = torch.Generator().manual_seed(0)
        self.clocks = ClockSampler()
        self.clocks.start()
        self.windows = []
        self.tokens_pf, self.batch, self.context = 2048, args.batch, 2048
        self.steps, self.warmup = max(4, min(args.steps, 32)), max(args.warmup, 3)
        self.flush = torch.empty(160 << 20, dtype=torch.uint8, device=self.device)      # larger than L2

    def timed(self, fn, reps=5):
        import torch
        for _ in range(3):
            fn()
        out = []
        for _ in range(reps):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return statistics.median(out)

    def run_model(self, cfg, name, params, kv_bytes_per_token, state_bytes_per_request=0):
        """``params``: weights a prefill multiplies with per token (``active``) and weights a decode step reads
        (``read``); ``kv_bytes_per_token``: cache bytes a decode row reads per token of its context;
        ``state_bytes_per_request``: fixed-size state a decode row reads and writes."""
        import torch
        from tiny_llm_infer_b200 import ops
        from tiny_llm_infer_b200.cache import CacheManager
        from tiny_llm_infer_b200.engine import ModelRunner, StepEntry, random_model
        device, gen, batch, context, tokens_pf = self.device, self.gen, self.batch, self.context, self.tokens_pf
        steps, warmup, windows, timed = self.steps, self.warmup, self.windows, self.timed
        model = random_model(cfg, seed=0, dtype=torch.bfloat16, device=device, std=0.02)
        page = 16
        pages = (batch + 1) * (context // page) + 2 * (tokens_pf // page) + 64
        cache = CacheManager(model.cache_needs(), page, pages, max_slots=batch + 1, max_seq_len=context + 64,
                             dtype=torch.bfloat16, device=device)
        runner = ModelRunner(model, cache, max_batch_tokens=tokens_pf)
        vocab = cfg.vocab_size

        def toks(n):
            return torch.randint(0, vocab, (n,), generator=gen).tolist()

        def prefill_once():
            runner.step([StepEntry("pf", toks(tokens_pf), [tokens_pf - 1])])
            torch.cuda.synchronize()
            runner.release("pf")

        w0 = time.perf_counter()
        pf_ms = timed(prefill_once)
        windows.append((w0, time.perf_counter(), f"{name} prefill"))
        start_len = context - steps - warmup
        names = [f"d{i}" for i in range(batch)]
        for n in names:
            runner.step([StepEntry(n, toks(start_len), [])])
        w0 = time.perf_counter()
        times = []
        before = ops.launches
        for it in range(warmup + steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            nxt = toks(batch)
            a.record()
            logits = runner.step([StepEntry(n, [t], [0]) for n, t in zip(names, nxt)])
            b.record()
            torch.cuda.synchronize()
            if it == warmup - 1:
                before = ops.launches
            if it >= warmup:
                times.append(a.elapsed_time(b))
        launches = ops.launches - before
        windows.append((w0, time.perf_counter(), f"{name} decode"))
        assert bool(torch.isfinite(logits).all())
        dec_ms = statistics.median(times)
        for n in names:
            runner.release(n)
        runner.check_kernels()
        moved = 2.0 * params["read"] + batch * (context * kv_bytes_per_token + 2 * state_bytes_per_request)
        out = {"prefill_tokens_per_s": round(tokens_pf / pf_ms * 1e3, 1), "prefill_ms": round(pf_ms, 3),
               "prefill_tflops": round(2.0 * tokens_pf * params["active"] / pf_ms / 1e9, 1),
               "decode_tokens_per_s": round(batch / dec_ms * 1e3, 1), "decode_ms": round(dec_ms, 4),
               "decode_gbs": round(moved / dec_ms / 1e6, 1),
               "launches_per_decode_step": launches // max(steps, 1)}
        del runner, cache, model
        torch.cuda.empty_cache()
        return out


def design_bench(args) -> int:
    """``--design panolorn``: prefill and decode throughput of the Panolorn design at sizes that resemble a
    real model's layers (random weights, bfloat16; layers alternate dense and mixture feed-forwards), beside
    Qwen3 dense, the closest model the engine has, at equal sizes (same width, heads, head width, layers,
    vocabulary, and a feed-forward as wide as a token's share of the mixture), through the same step
    function; and the new kernels one by one beside their relatives, with their share of the measured
    peaks.  One JSON line."""
    import math
    import torch
    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.config import Qwen3Config
    from tiny_llm_infer_b200.config.panolorn import (AttentionMixerConfig, FeedForwardConfig, PanolornConfig,
                                                      PanolornLayerConfig)
    from tiny_llm_infer_b200.engine import ModelRunner, StepEntry, random_model

    hx = _DesignHarness(args)
    device, pk, gen, clocks, windows = hx.device, hx.pk, hx.gen, hx.clocks, hx.windows
    tokens_pf, batch, context, steps, warmup = hx.tokens_pf, hx.batch, hx.context, hx.steps, hx.warmup
    timed, run_model = hx.timed, hx.run_model

    record = {"sizes": {}}
    for size_name in ([args.model] if args.model in DESIGN_SIZES else sorted(DESIGN_SIZES)):
        z = DESIGN_SIZES[size_name]
        L, W, H, G, D = z["layers"], z["width"], z["heads"], z["kv_heads"], z["dim"]
        mixer = AttentionMixerConfig(H, G, D, D, 1.0 / math.sqrt(D), 50.0, z["chunk"])
        dense = FeedForwardConfig("dense", z["ff"])
        moe = FeedForwardConfig("moe", z["expert_ff"], experts=z["experts"], top=z["top"], shared_ff=z["shared_ff"])
        pcfg = PanolornConfig(vocab=z["vocab"], width=W, embedding_scale=math.sqrt(W), norm_eps=1e-5, layers=tuple(
            PanolornLayerConfig("attention", mixer, dense if i % 2 == 0 else moe) for i in range(L)))
        qcfg = Qwen3Config(hidden_size=W, intermediate_size=z["ff"], num_hidden_layers=L, num_attention_heads=H,
                           num_key_value_heads=G, head_dim=D, vocab_size=z["vocab"], max_position_embeddings=8192,
                           tie_word_embeddings=True, layer_types=("full_attention",) * L)
        attn = W * (H + 2 * G) * D + H * D * W
        gate = W * H * D
        p_active = L * (attn + gate + 3 * W * z["ff"]) + (L // 2) * W * z["experts"] + z["vocab"] * W
        # weights a decode step of `batch` rows reads: at most batch * top experts of a mixture layer
        hit = min(z["experts"], batch * z["top"])
        p_read = L * (attn + gate) + (L - L // 2) * 3 * W * z["ff"] \
            + (L // 2) * (3 * W * (hit * z["expert_ff"] + z["shared_ff"]) + W * z["experts"]) + z["vocab"] * W
        q_params = L * (attn + 3 * W * z["ff"]) + z["vocab"] * W
        kv = 2 * G * D * 2 * L
        print(f"[bench] design sizes {size_name}: Panolorn", file=sys.stderr, flush=True)
        ours = run_model(pcfg, f"panolorn {size_name}", {"active": p_active, "read": p_read}, kv)
        print(f"[bench] {ours}\n[bench] design sizes {size_name}: Qwen3 dense", file=sys.stderr, flush=True)
        theirs = run_model(qcfg, f"qwen3 {size_name}", {"active": q_params, "read": q_params}, kv)
        print(f"[bench] {theirs}", file=sys.stderr, flush=True)
        for r in (ours, theirs):
            r["prefill_frac_of_measured"] = round(r["prefill_tflops"] / pk["bf16_tflops"], 4)
            r["decode_hbm_frac_of_measured"] = round(r["decode_gbs"] / pk["hbm_gbs"], 4)
        record["sizes"][size_name] = {"panolorn": ours, "qwen3_dense": theirs, "config": z}

    # ---- kernels one by one at the larger sizes (inputs larger than L2 or L2 flushed between runs)
    z = DESIGN_SIZES["8b"]
    W, H, G, D = z["width"], z["heads"], z["kv_heads"], z["dim"]
    bf = torch.bfloat16
    kern = {}
    T = tokens_pf
    # norm of the sub-layer's output + sum + next norm, beside the sum + norm of the other block
    h = torch.randn(T * 4, W, device=device)
    delta = torch.randn(T * 4, W, device=device).to(bf)
    gain = torch.ones(W, device=device, dtype=bf)
    out = torch.empty_like(delta)
    nbytes = h.numel() * 8 + delta.numel() * 4
    for key, kw in (("add_rmsnorm", {}), ("postnorm_add_rmsnorm", dict(post_gain=gain, post_eps=1e-5))):
        ms = timed(lambda: ops.add_rmsnorm(h, delta, gain, 1e-5, out, **kw))
        kern[key] = {"us": round(ms * 1e3, 1), "gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3)}
    del h, delta, out
    # attention over a paged cache: prompt of 2048 tokens, and 64 one-token rows at context 2048
    page, ctx_len, rows = 16, 2048, 64
    n_pages = rows * ctx_len // page
    flat = (torch.randn(n_pages, page * 2 * G * D, device=device) * 0.5).to(bf)
    kv_u = flat.view(n_pages, 2, G, page, D)
    k_plane = flat[:, :G * page * D].unflatten(1, (G, page, D))
    v_plane = flat[:, G * page * D:].unflatten(1, (G, page, D))
    table = torch.arange(n_pages, dtype=torch.int32, device=device).view(rows, ctx_len // page).contiguous()
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / H) for i in range(H)], dtype=torch.float32, device=device)
    from tiny_llm_infer_b200.engine.batch import StepContext

    def context_for(segs):
        seg, tiles, dec, row = [], [], [], 0
        for s, (slot, p0, n) in enumerate(segs):
            seg.append([slot, row, n, p0])
            if n == 1:
                dec.append(row)
            else:
                tiles += [(s, off) for off in range(0, n, 64)]
            row += n
        tiles.sort(key=lambda t: (t[1] % 256 != 0, t[1] % 128 != 0))
        pos = torch.tensor([p0 + i for _, p0, n in segs for i in range(n)], dtype=torch.int32, device=device)
        slot = torch.tensor([sl for sl, _, n in segs for _ in range(n)], dtype=torch.int32, device=device)
        return StepContext(tokens=row, token_ids=None, positions=pos, token_slot=slot, want_rows=None, segments=[],
                           seg_info=torch.tensor(seg, dtype=torch.int32, device=device),
                           dec_rows=None if len(dec) == row else torch.tensor(dec, dtype=torch.int32, device=device),
                           n_dec=len(dec), pf_tiles=torch.tensor(tiles, dtype=torch.int32, device=device).view(-1, 2),
                           n_tiles=len(tiles), n_tiles128=sum(1 for t in tiles if t[1] % 128 == 0),
                           n_tiles256=sum(1 for t in tiles if t[1] % 256 == 0), max_context=ctx_len, max_segment=max(n for _, _, n in segs))

    for what, segs in (("prefill_2048", [(0, 0, T)]), ("decode_64_rows_ctx_2048", [(i, ctx_len - 1, 1) for i in range(rows)])):
        ctx = context_for(segs)
        n = ctx.tokens
        q = (torch.randn(n, H * D, device=device)).to(bf)
        gate_t = torch.randn(n, H * D, device=device).to(bf)
        o = torch.empty_like(q)
        if n > 1 and what.startswith("prefill"):
            flops = 4.0 * H * D * T * (T + 1) / 2
            unit = lambda ms: {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1), "frac_tensor": round(flops / ms / 1e9 / pk["bf16_tflops"], 3)}
        else:
            nbytes = rows * ctx_len * 2 * G * D * 2
            unit = lambda ms: {"us": round(ms * 1e3, 1), "gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3)}
        ms = timed(lambda: ops.attention_biased(q, k_plane, v_plane, ctx.positions, ctx.token_slot, table, page, H, G, D, D,
                                                1.0 / math.sqrt(D), o, softcap=50.0, chunk=z["chunk"], sink=True, slopes=slopes,
                                                gate=gate_t, ctx=ctx))
        kern[f"attention_biased_{what}"] = unit(ms)
        ms = timed(lambda: ops.paged_attention(q, kv_u, ctx.positions, ctx.token_slot, table, page, H, G, D, None,
                                               1.0 / math.sqrt(D), o, ctx=ctx))
        kern[f"paged_attention_{what}"] = unit(ms)
    ops.check_error_word(device)
    del flat, kv_u, k_plane, v_plane
    # the experts' products beside the dense products of the same work
    E, top, I = z["experts"], z["top"], z["expert_ff"]
    x = torch.randn(T, W, device=device).to(bf)
    w_gu = (torch.randn(E, 2 * I, W, device=device) * 0.02).to(bf)
    w_d = (torch.randn(E, W, I, device=device) * 0.02).to(bf)
    zr = torch.randn(T, E, device=device)
    ids, wts = ops.moe_route(zr, top)
    on_tensor_memory = ops.moe_tcgen05_pays(T * top, E, I, W, bf)
    plan = ops.MoePlan(ids, E, ops.MOE_TCGEN05_TILE if on_tensor_memory else None)
    flops = 2.0 * T * top * 3 * W * I

    def experts():
        a = ops.moe_grouped(x, w_gu, plan, top, gated=True, gather=True, weights=wts, interleaved=True)
        return ops.moe_grouped(a, w_d, plan, top, gated=False, gather=False)
    ms = timed(experts)
    kern["moe_grouped_products_2048_tokens"] = {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1),
                                                "frac_tensor": round(flops / ms / 1e9 / pk["bf16_tflops"], 3)}
    # four times the rows: an expert's 128-row tiles are then mostly full (at 2048 tokens an expert gets 128 rows
    # on average, so nearly every expert has a second, almost empty tile)
    T4 = 4 * T
    x4 = torch.randn(T4, W, device=device).to(bf)
    ids4, wts4 = ops.moe_route(torch.randn(T4, E, device=device), top)
    plan4 = ops.MoePlan(ids4, E, ops.MOE_TCGEN05_TILE if ops.moe_tcgen05_pays(T4 * top, E, I, W, bf) else None)

    def experts4():
        a = ops.moe_grouped(x4, w_gu, plan4, top, gated=True, gather=True, weights=wts4, interleaved=True)
        return ops.moe_grouped(a, w_d, plan4, top, gated=False, gather=False)
    ms = timed(experts4)
    kern["moe_grouped_products_8192_tokens"] = {"us": round(ms * 1e3, 1), "tflops": round(4 * flops / ms / 1e9, 1),
                                                "frac_tensor": round(4 * flops / ms / 1e9 / pk["bf16_tflops"], 3)}
    del x4, ids4, wts4, plan4
    wd_gu = ops.interleave_gate_up(*(torch.randn(2, top * I, W, device=device) * 0.02).to(bf)).contiguous()
    wd_d = (torch.randn(W, top * I, device=device) * 0.02).to(bf)
    ms = timed(lambda: ops.linear(ops.linear_swiglu(x, wd_gu, bf, interleaved=True), wd_d, out_dtype=bf))
    kern["dense_products_same_work_2048_tokens"] = {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1),
                                                    "frac_tensor": round(flops / ms / 1e9 / pk["bf16_tflops"], 3)}
    x8 = x[:8].contiguous()
    ids8, wts8 = ops.moe_route(zr[:8].contiguous(), top)
    plan8 = ops.MoePlan(ids8, E)
    nbytes = 8 * top * 3 * W * I * 2           # 32 different experts at most

    def experts8():
        a = ops.moe_grouped(x8, w_gu, plan8, top, gated=True, gather=True, weights=wts8, interleaved=True)
        return ops.moe_grouped(a, w_d, plan8, top, gated=False, gather=False)
    ms = timed(experts8)
    kern["moe_grouped_products_8_rows"] = {"us": round(ms * 1e3, 1), "gbs_at_most": round(nbytes / ms / 1e6, 1)}
    ms = timed(lambda: ops.linear(ops.linear_swiglu(x8, wd_gu, bf, interleaved=True), wd_d, out_dtype=bf))
    kern["dense_products_8_rows_of_one_expert_set"] = {"us": round(ms * 1e3, 1), "gbs": round(top * 3 * W * I * 2 / ms / 1e6, 1)}
    ops.check_error_word(device)
    record["kernels"] = kern
    clock_record = clocks.stop(windows)
    first = record["sizes"][sorted(record["sizes"])[0]]["panolorn"]
    print(json.dumps({"metric": f"decode tok/s @ batch {batch} (Panolorn design sizes, context {context}, 1 B200)",
                      "value": first["decode_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
                      "ms_per_step": first["decode_ms"], "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                      "design": "panolorn", "clocks": clock_record, "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"]},
                      **record}))
    return 0


KAKETAR_SIZES = {
    # width, layers (every fourth one latent attention, the others the delta rule), feed-forward on every layer;
    # delta rule: heads, key and value width, taps, low ranks; latent attention: heads, unrotated / rotated / value
    # width, the two latents (cached vector = kv_rank + rot = 128, the widest the tensor-core tiles take), window
    "1b": dict(width=2048, layers=8, ff=6144, vocab=32768, side=64, d_heads=16, d_dim=128, d_vdim=128, taps=4, rank=64,
               a_heads=16, a_dim=64, a_rot=32, a_vdim=128, q_rank=512, kv_rank=96, window=1024),
    "8b": dict(width=4096, layers=4, ff=12288, vocab=32768, side=64, d_heads=32, d_dim=128, d_vdim=128, taps=4, rank=128,
               a_heads=32, a_dim=64, a_rot=32, a_vdim=128, q_rank=1024, kv_rank=96, window=1024),
}


def kaketar_bench(args) -> int:
    """``--design kaketar``: prefill and decode throughput of the Kaketar design at sizes that resemble a real
    model's layers (random weights, bfloat16; three delta-rule layers to one of latent attention, a feed-forward
    and the token side input on every layer), beside Qwen3 dense, the closest model the engine has, at equal
    sizes (same width, layers, head count and width of the delta rule's heads, feed-forward, vocabulary),
    through the same step function; and the new kernels one by one beside their relatives, with their share of
    the measured peaks.  One JSON line."""
    import math
    import torch
    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.config import Qwen3Config
    from tiny_llm_infer_b200.config.kaketar import (ChannelDeltaConfig, DenseConfig, KaketarConfig, KaketarLayerConfig,
                                                     LatentAttentionConfig, RotationScaling)
    from tiny_llm_infer_b200.engine.batch import StepContext
    from tiny_llm_infer_b200.parts.delta_rule import state_floats

    hx = _DesignHarness(args)
    device, pk, clocks, windows = hx.device, hx.pk, hx.clocks, hx.windows
    tokens_pf, batch, context, steps, warmup = hx.tokens_pf, hx.batch, hx.context, hx.steps, hx.warmup
    timed, run_model = hx.timed, hx.run_model
    record = {"sizes": {}}
    for size_name in ([args.model] if args.model in KAKETAR_SIZES else sorted(KAKETAR_SIZES)):
        z = KAKETAR_SIZES[size_name]
        L, W = z["layers"], z["width"]
        dmix = ChannelDeltaConfig(z["d_heads"], z["d_heads"], z["d_dim"], z["d_vdim"], z["taps"], z["rank"], z["rank"])
        amix = LatentAttentionConfig(z["a_heads"], z["a_dim"], z["a_rot"], z["a_vdim"], z["q_rank"], z["kv_rank"],
                                     1.0 / math.sqrt(z["a_dim"] + z["a_rot"]), 10000.0, z["a_rot"], z["window"],
                                     RotationScaling(4.0, 1024.0, 32.0, 1.0))
        kcfg = KaketarConfig(vocab=z["vocab"], width=W, max_positions=4096, embedding_scale=1.0, norm_eps=1e-6, layers=tuple(
            KaketarLayerConfig("latent_attention", amix, DenseConfig(z["ff"])) if i % 4 == 3 else
            KaketarLayerConfig("channel_delta", dmix, DenseConfig(z["ff"])) for i in range(L)),
            logit_softcap=30.0, side_dim=z["side"])
        H, D = z["d_heads"], z["d_dim"]
        qcfg = Qwen3Config(hidden_size=W, intermediate_size=z["ff"], num_hidden_layers=L, num_attention_heads=H,
                           num_key_value_heads=max(H // 4, 1), head_dim=D, vocab_size=z["vocab"], max_position_embeddings=8192,
                           tie_word_embeddings=True, layer_types=("full_attention",) * L)
        n_lat = L // 4
        n_delta = L - n_lat
        hd, hv = z["d_heads"] * z["d_dim"], z["d_heads"] * z["d_vdim"]
        delta_w = W * (2 * hd + hv + z["d_heads"]) + 2 * W * z["rank"] + z["rank"] * (hd + hv) + hv * W
        ah = z["a_heads"]
        latent_w = W * (z["q_rank"] + z["kv_rank"] + z["a_rot"] + ah * z["a_vdim"]) + z["q_rank"] * ah * (z["a_dim"] + z["a_rot"]) \
            + ah * z["kv_rank"] * (z["a_dim"] + z["a_vdim"]) + ah * z["a_vdim"] * W
        side_w = 2 * W * z["side"]
        k_params = n_delta * delta_w + n_lat * latent_w + L * (2 * W * z["ff"] + side_w) + z["vocab"] * W
        G = max(H // 4, 1)
        q_params = L * (W * (H + 2 * G) * D + H * D * W + 3 * W * z["ff"]) + z["vocab"] * W
        state = 4 * n_delta * state_floats(z["d_heads"], z["d_heads"], z["d_dim"], z["d_vdim"], z["taps"])
        k_kv = 2 * n_lat * (z["kv_rank"] + z["a_rot"]) * min(z["window"], context) / context
        print(f"[bench] design sizes {size_name}: Kaketar", file=sys.stderr, flush=True)
        ours = run_model(kcfg, f"kaketar {size_name}", {"active": k_params, "read": k_params}, k_kv, state)
        print(f"[bench] {ours}\n[bench] design sizes {size_name}: Qwen3 dense", file=sys.stderr, flush=True)
        theirs = run_model(qcfg, f"qwen3 {size_name}", {"active": q_params, "read": q_params}, 2 * G * D * 2 * L)
        print(f"[bench] {theirs}", file=sys.stderr, flush=True)
        for r in (ours, theirs):
            r["prefill_frac_of_measured"] = round(r["prefill_tflops"] / pk["bf16_tflops"], 4)
            r["decode_hbm_frac_of_measured"] = round(r["decode_gbs"] / pk["hbm_gbs"], 4)
        record["sizes"][size_name] = {"kaketar": ours, "qwen3_dense": theirs, "config": z,
                                      "params": {"kaketar": k_params, "qwen3_dense": q_params}}

    # ---- kernels one by one at the larger sizes (L2 flushed between runs)
    z = KAKETAR_SIZES["8b"]
    W, bf, T = z["width"], torch.bfloat16, tokens_pf
    kern = {}

    def hbm(nbytes, ms):
        return {"us": round(ms * 1e3, 1), "gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3)}

    def tensor(flops, ms):
        return {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1), "frac_tensor": round(flops / ms / 1e9 / pk["bf16_tflops"], 3)}

    # the sum of a normed output that hands the stream on without a norm, beside the sum + norm of the other blocks
    h = torch.randn(T * 4, W, device=device)
    delta = torch.randn(T * 4, W, device=device).to(bf)
    gain32, gain16 = torch.ones(W, device=device), torch.ones(W, device=device, dtype=bf)
    out = torch.empty_like(delta)
    nbytes = h.numel() * 8 + delta.numel() * 4
    kern["stream_add_normed_delta"] = hbm(nbytes, timed(lambda: ops.stream_add(h, delta, out, post_gain=gain32, post_eps=1e-6)))
    kern["postnorm_add_rmsnorm"] = hbm(nbytes, timed(lambda: ops.add_rmsnorm(h, delta, gain16, 1e-6, out, post_gain=gain16, post_eps=1e-6)))
    kern["add_rmsnorm"] = hbm(nbytes, timed(lambda: ops.add_rmsnorm(h, delta, gain16, 1e-6, out)))
    del h, delta, out
    # embedding + position + norm beside the plain look-up
    table = torch.randn(z["vocab"], W, device=device).to(bf)
    pos_table = torch.randn(4096, W, device=device).to(bf)
    ids = torch.randint(0, z["vocab"], (T * 4,), device=device, dtype=torch.int32)
    positions = (torch.arange(T * 4, device=device, dtype=torch.int32) % 4096).contiguous()
    out32 = torch.empty(T * 4, W, device=device)
    kern["embedding_position_norm"] = hbm(T * 4 * W * (2 + 2 + 4), timed(lambda: ops.embedding_norm(ids, table, out32, 2.0, positions, pos_table, gain32, 1e-6)))
    kern["embedding"] = hbm(T * 4 * W * (2 + 4), timed(lambda: ops.embedding(ids, table, out32)))
    del table, pos_table, out32
    # activation of the plain feed-forward beside the gated one's
    x = torch.randn(T, z["ff"], device=device).to(bf)
    x2 = torch.randn(T, 2 * z["ff"], device=device).to(bf)
    o = torch.empty_like(x)
    kern["activation_gelu_erf"] = hbm(x.numel() * 4, timed(lambda: ops.activation(x, "gelu_erf")))
    kern["swiglu"] = hbm(x.numel() * 6, timed(lambda: ops.swiglu(x2, o)))
    del x, x2, o

    # the delta rule: 2048 tokens of one request, and 64 one-token rows (state read and written once per row)
    Hd, dk, dv, taps = z["d_heads"], z["d_dim"], z["d_vdim"], z["taps"]
    channels = 2 * Hd * dk + Hd * dv
    floats = state_floats(Hd, Hd, dk, dv, taps)
    rows = 64
    state = torch.zeros(rows, floats, device=device)
    conv_w = (torch.randn(channels, taps, device=device) * 0.5).to(bf)
    conv_t = conv_w.t().contiguous()
    dt_bias = torch.randn(Hd * dk, device=device) - 4.0
    rate = torch.ones(Hd, device=device)
    weight = torch.ones(dv, device=device)
    for what, n, seg in (("prefill_2048", T, [[0, 0, T, 0]]), ("decode_64_rows", rows, None)):
        proj = torch.randn(n, (channels + Hd + 7) // 8 * 8, device=device).to(bf)
        a = torch.randn(n, Hd * dk, device=device)
        gate = torch.randn(n, Hd * dv, device=device)
        slots = torch.zeros(n, dtype=torch.int32, device=device) if seg else torch.arange(n, dtype=torch.int32, device=device)
        seg_info = torch.tensor(seg, dtype=torch.int32, device=device) if seg else None
        ms = timed(lambda: ops.delta_rule(proj, conv_w, taps, a, dt_bias, rate, gate, weight, 1e-6, slots, seg_info, state,
                                          Hd, Hd, dk, dv, dk ** -0.5, 1e-6, bf, conv_t=conv_t))
        flops = 6.0 * n * Hd * dk * dv                      # decay and two rank-one steps per element of S, a read-out
        io = n * ((channels + Hd) * 2 + (Hd * dk + Hd * dv) * 4 + Hd * dv * 2) + (0 if seg else 2 * rows * Hd * dk * dv * 4)
        work = n * (2 * Hd * dk + 2 * Hd * dv + Hd * dk + Hd) * 4 * 2      # the float32 hand-over between the three kernels
        kern[f"delta_rule_{what}"] = {"us": round(ms * 1e3, 1), "tokens_per_s": round(n / ms * 1e3, 1),
                                      "gflops_fp32": round(flops / ms / 1e6, 1), "gbs": round((io + work) / ms / 1e6, 1),
                                      "frac_hbm": round((io + work) / ms / 1e6 / pk["hbm_gbs"], 3)}
    del state

    # attention: cached latents (multi-query, values inside the keys) beside Qwen3's paged attention at the same
    # head count; a prompt of 2048 tokens, and 64 one-token rows at context 2048 (the latents' window is 1024)
    page, ctx_len = 16, context
    n_pages = rows * ctx_len // page
    table = torch.arange(n_pages, dtype=torch.int32, device=device).view(rows, ctx_len // page).contiguous()

    def context_for(segs):
        seg, tiles, dec, row = [], [], [], 0
        for s, (slot, p0, n) in enumerate(segs):
            seg.append([slot, row, n, p0])
            if n == 1:
                dec.append(row)
            else:
                tiles += [(s, off) for off in range(0, n, 64)]
            row += n
        tiles.sort(key=lambda t: (t[1] % 256 != 0, t[1] % 128 != 0))
        pos = torch.tensor([p0 + i for _, p0, n in segs for i in range(n)], dtype=torch.int32, device=device)
        slot = torch.tensor([sl for sl, _, n in segs for _ in range(n)], dtype=torch.int32, device=device)
        return StepContext(tokens=row, token_ids=None, positions=pos, token_slot=slot, want_rows=None, segments=[],
                           seg_info=torch.tensor(seg, dtype=torch.int32, device=device),
                           dec_rows=None if len(dec) == row else torch.tensor(dec, dtype=torch.int32, device=device),
                           n_dec=len(dec), pf_tiles=torch.tensor(tiles, dtype=torch.int32, device=device).view(-1, 2),
                           n_tiles=len(tiles), n_tiles128=sum(1 for t in tiles if t[1] % 128 == 0),
                           n_tiles256=sum(1 for t in tiles if t[1] % 256 == 0), max_context=ctx_len, max_segment=max(n for _, _, n in segs))

    Ha, rank, rot, window = z["a_heads"], z["kv_rank"], z["a_rot"], z["window"]
    wide = rank + rot
    plane = (torch.randn(n_pages, 1, page, wide, device=device) * 0.5).to(bf)
    sink = torch.zeros(Ha, device=device)
    G, D = max(Ha // 4, 1), 128
    kv_u = (torch.randn(n_pages, 2, G, page, D, device=device) * 0.5).to(bf)
    for what, segs in (("prefill_2048", [(0, 0, T)]), ("decode_64_rows_ctx_2048", [(i, ctx_len - 1, 1) for i in range(rows)])):
        ctx = context_for(segs)
        n = ctx.tokens
        q = torch.randn(n, Ha * wide, device=device).to(bf)
        mix = torch.empty(n, Ha * rank, dtype=bf, device=device)
        ms = timed(lambda: ops.attention_biased(q, plane, plane, ctx.positions, ctx.token_slot, table, page, Ha, 1, wide, rank,
                                                0.1, mix, window=window, sink=True, sink_logits=sink, ctx=ctx, values_in_keys=True))
        if what.startswith("prefill"):
            keys = sum(min(i + 1, window) for i in range(T))
            kern[f"latent_attention_{what}"] = tensor(2.0 * Ha * (wide + rank) * keys, ms)
        else:
            kern[f"latent_attention_{what}"] = hbm(rows * min(window, ctx_len) * wide * 2, ms)
        q2 = torch.randn(n, Ha * D, device=device).to(bf)
        o2 = torch.empty_like(q2)
        ms = timed(lambda: ops.paged_attention(q2, kv_u, ctx.positions, ctx.token_slot, table, page, Ha, G, D, None,
                                               1.0 / math.sqrt(D), o2, ctx=ctx))
        if what.startswith("prefill"):
            kern[f"paged_attention_{what}"] = tensor(4.0 * Ha * D * T * (T + 1) / 2, ms)
        else:
            kern[f"paged_attention_{what}"] = hbm(rows * ctx_len * 2 * G * D * 2, ms)
    ops.check_error_word(device)
    record["kernels"] = kern
    clock_record = clocks.stop(windows)
    first = record["sizes"][sorted(record["sizes"])[0]]["kaketar"]
    print(json.dumps({"metric": f"decode tok/s @ batch {batch} (Kaketar design sizes, context {context}, 1 B200)",
                      "value": first["decode_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
                      "ms_per_step": first["decode_ms"], "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                      "design": "kaketar", "clocks": clock_record, "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"]},
                      **record}))
    return 0


TETODRA_SIZES = {
    # width, layers in the order parallel, parallel_2, delta, parallel_2 (repeated), feed-forward on every layer;
    # both attentions: heads, key/value heads, head width (keys and values); both side memories: heads, key and value
    # width; delta rule: heads, heads of queries and keys, widths, taps
    "1b": dict(width=2048, layers=8, ff=6144, vocab=32768, a_heads=16, a_kv=4, a_dim=128, m_heads=8, m_dim=128, m_vdim=128,
               d_heads=16, d_kv=8, d_dim=128, d_vdim=128, taps=4),
    "8b": dict(width=4096, layers=4, ff=12288, vocab=32768, a_heads=32, a_kv=8, a_dim=128, m_heads=16, m_dim=128, m_vdim=128,
               d_heads=32, d_kv=16, d_dim=128, d_vdim=128, taps=4),
}


def _model_costs(cfg, context):
    """(weights a token multiplies with, cache bytes a decode row reads per token of its context, bytes of a
    request's fixed-size state), from the model's own description: every matrix once (the tied head counts as the
    embedding; other look-up tables do not), the planes of every cache within its reach, every state."""
    import torch
    from tiny_llm_infer_b200.config import describe_model
    from tiny_llm_infer_b200.models.model import Model, expected_tensors
    desc = describe_model(cfg)
    names, _ = expected_tensors(desc)
    params = sum(math.prod(spec.shape) for name, spec in names.items()
                 if len(spec.shape) == 2 and not (name.endswith("embed") and name != desc.embedding.prefix + desc.embedding.params.get("name", "")))
    kv = state = 0.0
    for cache, st in Model(desc, torch.bfloat16, None).cache_needs().values():
        if cache is not None:
            reach = min(cache.window or context, context)
            kv += 2.0 * sum(h * w for h, w in cache.planes) * reach / context
        if st is not None:
            state += 4.0 * math.prod(st.shape)
    return params, kv, state


def _kaketar_at(z):
    from tiny_llm_infer_b200.config.kaketar import (ChannelDeltaConfig, DenseConfig, KaketarConfig, KaketarLayerConfig,
                                                     LatentAttentionConfig, RotationScaling)
    dmix = ChannelDeltaConfig(z["d_heads"], z["d_heads"], z["d_dim"], z["d_vdim"], z["taps"], z["rank"], z["rank"])
    amix = LatentAttentionConfig(z["a_heads"], z["a_dim"], z["a_rot"], z["a_vdim"], z["q_rank"], z["kv_rank"],
                                 1.0 / math.sqrt(z["a_dim"] + z["a_rot"]), 10000.0, z["a_rot"], z["window"],
                                 RotationScaling(4.0, 1024.0, 32.0, 1.0))
    return KaketarConfig(vocab=z["vocab"], width=z["width"], max_positions=4096, embedding_scale=1.0, norm_eps=1e-6, layers=tuple(
        KaketarLayerConfig("latent_attention", amix, DenseConfig(z["ff"])) if i % 4 == 3 else
        KaketarLayerConfig("channel_delta", dmix, DenseConfig(z["ff"])) for i in range(z["layers"])),
        logit_softcap=30.0, side_dim=z["side"])


def tetodra_bench(args) -> int:
    """``--design tetodra``: prefill and decode throughput of the Tetodra design at sizes that resemble a real
    model's layers (random weights, bfloat16; layers in the order attention with keys as values beside a matrix
    memory, attention with a rotation beside gated linear attention, delta rule with a decay per head, the second
    kind again; a feed-forward on every layer), beside the two closest models the engine has at equal width,
    layers, feed-forward and vocabulary, through the same step function: Kaketar (delta rule and attention, its
    own bench's sizes) and Qwen3 dense.  Then the design's kernels one by one beside their relatives, with their
    share of the measured peaks.  One JSON line."""
    import torch
    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.config import Qwen3Config
    from tiny_llm_infer_b200.config.tetodra import (DenseConfig, GatedDeltaConfig, GatedLinearConfig, KeyValueAttentionConfig,
                                                     MatrixMemoryConfig, PairConfig, RotaryAttentionConfig, TetodraConfig,
                                                     TetodraLayerConfig)
    from tiny_llm_infer_b200.engine.batch import StepContext
    from tiny_llm_infer_b200.parts.attention_biased import distance_buckets
    from tiny_llm_infer_b200.parts.delta_rule import state_floats

    hx = _DesignHarness(args)
    device, pk, clocks, windows = hx.device, hx.pk, hx.clocks, hx.windows
    tokens_pf, batch, context, steps, warmup = hx.tokens_pf, hx.batch, hx.context, hx.steps, hx.warmup
    timed, run_model = hx.timed, hx.run_model
    record = {"sizes": {}}
    for size_name in ([args.model] if args.model in TETODRA_SIZES else sorted(TETODRA_SIZES)):
        z = TETODRA_SIZES[size_name]
        L, W, D = z["layers"], z["width"], z["a_dim"]
        ff = DenseConfig(z["ff"])
        keyed = PairConfig(KeyValueAttentionConfig(z["a_heads"], z["a_kv"], D, D, D ** -0.5, 128.0, 0.25, 512, 32),
                           MatrixMemoryConfig(z["m_heads"], z["m_dim"], z["m_vdim"], 12.0), 0.5, 1.0)
        rotary = PairConfig(RotaryAttentionConfig(z["a_heads"], z["a_kv"], D, D, D ** -0.5, 1000000.0, D),
                            GatedLinearConfig(z["m_heads"], z["m_dim"], z["m_vdim"], 8.0, W // 64), 0.75, 0.75)
        delta = GatedDeltaConfig(z["d_heads"], z["d_kv"], z["d_dim"], z["d_vdim"], z["taps"])
        kinds = [("parallel", keyed), ("parallel_2", rotary), ("delta", delta), ("parallel_2", rotary)]
        tcfg = TetodraConfig(vocab=z["vocab"], width=W, embedding_scale=1.0, norm_eps=1e-5, residual_mult=0.8,
                             layers=tuple(TetodraLayerConfig(*kinds[i % 4], ff) for i in range(L)))
        H, G = z["a_heads"], z["a_kv"]
        qcfg = Qwen3Config(hidden_size=W, intermediate_size=z["ff"], num_hidden_layers=L, num_attention_heads=H,
                           num_key_value_heads=G, head_dim=D, vocab_size=z["vocab"], max_position_embeddings=8192,
                           tie_word_embeddings=True, layer_types=("full_attention",) * L)
        kcfg = _kaketar_at(KAKETAR_SIZES[size_name])
        q_params = L * (W * (H + 2 * G) * D + H * D * W + 3 * W * z["ff"]) + z["vocab"] * W
        entry = {"config": z, "params": {}}
        for label, cfg, costs in (("tetodra", tcfg, _model_costs(tcfg, context)), ("kaketar", kcfg, _model_costs(kcfg, context)),
                                  ("qwen3_dense", qcfg, (q_params, 2.0 * G * D * 2 * L, 0.0))):
            print(f"[bench] design sizes {size_name}: {label}", file=sys.stderr, flush=True)
            params, kv, state = costs
            r = run_model(cfg, f"{label} {size_name}", {"active": params, "read": params}, kv, state)
            r["prefill_frac_of_measured"] = round(r["prefill_tflops"] / pk["bf16_tflops"], 4)
            r["decode_hbm_frac_of_measured"] = round(r["decode_gbs"] / pk["hbm_gbs"], 4)
            print(f"[bench] {r}", file=sys.stderr, flush=True)
            entry[label] = r
            entry["params"][label] = params
        record["sizes"][size_name] = entry

    # ---- kernels one by one at the larger sizes (L2 flushed between runs)
    z = TETODRA_SIZES["8b"]
    W, bf, T = z["width"], torch.bfloat16, tokens_pf
    kern = {}

    def hbm(nbytes, ms):
        return {"us": round(ms * 1e3, 1), "gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3)}

    def tensor(flops, ms):
        return {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1), "frac_tensor": round(flops / ms / 1e9 / pk["bf16_tflops"], 3)}

    # the scaled sum of three outputs with the layer norm, beside the sum of one output with the RMS norm
    h = torch.randn(T * 4, W, device=device)
    deltas = [torch.randn(T * 4, W, device=device).to(bf) for _ in range(3)]
    scales = [torch.rand(W, device=device) for _ in range(3)]
    gain16 = torch.ones(W, device=device, dtype=bf)
    out = torch.empty_like(deltas[0])
    per = h.numel()
    kern["scaled_add_layernorm_3_outputs"] = hbm(per * (8 + 3 * 2 + 2), timed(lambda: ops.scaled_add_layernorm(h, deltas, scales, gain16, 1e-5, out)))
    kern["scaled_add_layernorm_1_output"] = hbm(per * (8 + 2 + 2), timed(lambda: ops.scaled_add_layernorm(h, deltas[:1], scales[:1], gain16, 1e-5, out)))
    kern["add_rmsnorm"] = hbm(per * (8 + 2 + 2), timed(lambda: ops.add_rmsnorm(h, deltas[0], gain16, 1e-5, out)))
    del h, deltas, out

    rows, page, ctx_len = 64, 16, context

    def context_for(segs):
        seg, tiles, dec, row = [], [], [], 0
        for s, (slot, p0, n) in enumerate(segs):
            seg.append([slot, row, n, p0])
            if n == 1:
                dec.append(row)
            else:
                tiles += [(s, off) for off in range(0, n, 64)]
            row += n
        tiles.sort(key=lambda t: (t[1] % 256 != 0, t[1] % 128 != 0))
        pos = torch.tensor([p0 + i for _, p0, n in segs for i in range(n)], dtype=torch.int32, device=device)
        slot = torch.tensor([sl for sl, _, n in segs for _ in range(n)], dtype=torch.int32, device=device)
        return StepContext(tokens=row, token_ids=None, positions=pos, token_slot=slot, want_rows=None, segments=[],
                           seg_info=torch.tensor(seg, dtype=torch.int32, device=device),
                           dec_rows=None if len(dec) == row else torch.tensor(dec, dtype=torch.int32, device=device),
                           n_dec=len(dec), pf_tiles=torch.tensor(tiles, dtype=torch.int32, device=device).view(-1, 2),
                           n_tiles=len(tiles), n_tiles128=sum(1 for t in tiles if t[1] % 128 == 0),
                           n_tiles256=sum(1 for t in tiles if t[1] % 256 == 0), max_context=ctx_len, max_segment=max(n for _, _, n in segs))

    # attention: scores with a table of distance biases and a learned sink, and plain scores after a rotation, over
    # two planes of the paged cache, beside Qwen3's paged attention at the same heads; a prompt of 2048 tokens, and
    # 64 one-token rows at context 2048.  Before each, the kernel that norms, scales or turns queries and keys and
    # writes the cache, beside Qwen3's
    H, G, D = z["a_heads"], z["a_kv"], z["a_dim"]
    n_pages = rows * ctx_len // page
    table = torch.arange(n_pages, dtype=torch.int32, device=device).view(rows, ctx_len // page).contiguous()
    pool = (torch.randn(n_pages, 2 * G * page * D, device=device) * 0.5).to(bf)
    k_plane = pool[:, :G * page * D].unflatten(1, (G, page, D))
    v_plane = pool[:, G * page * D:].unflatten(1, (G, page, D))
    kv_u = pool.view(n_pages, 2, G, page, D)
    bias = torch.randn(H, 129, device=device)
    sink = torch.randn(H, device=device)
    gain = torch.ones(D, device=device, dtype=bf)
    inv_freq = (1000000.0 ** (-torch.arange(D // 2, dtype=torch.float64) * 2 / D)).float().to(device)
    for what, segs in (("prefill_2048", [(0, 0, T)]), ("decode_64_rows_ctx_2048", [(i, ctx_len - 1, 1) for i in range(rows)])):
        ctx = context_for(segs)
        n = ctx.tokens
        q = torch.randn(n, H * D, device=device).to(bf)
        o = torch.empty_like(q)
        keyed_proj = torch.randn(n, (H + G) * D, device=device).to(bf)
        full_proj = torch.randn(n, (H + 2 * G) * D, device=device).to(bf)
        moved = n * ((H + 2 * G) * D * 2 + (H + 2 * G) * D * 2)
        kern[f"qkv_store_keys_as_values_{what}"] = hbm(n * ((H + G) * D * 2 + (H + 2 * G) * D * 2), timed(lambda: ops.qkv_unit_store(
            keyed_proj, q, ctx.positions, ctx.token_slot, table, k_plane, v_plane, page, H, G, D, D, 1e-5, q_gain=gain, k_gain=gain,
            q_temperature=(0.25, 512), values_are_keys=True)))
        kern[f"qkv_store_rotation_{what}"] = hbm(moved, timed(lambda: ops.qkv_unit_store(
            full_proj, q, ctx.positions, ctx.token_slot, table, k_plane, v_plane, page, H, G, D, D, None, inv_freq=inv_freq, rot_dims=D)))
        kern[f"qwen3_qk_norm_rope_store_{what}"] = hbm(moved, timed(lambda: ops.qk_norm_rope_store(
            full_proj, gain, gain, 1e-6, inv_freq, D, ctx.positions, ctx.token_slot, table, kv_u, page, q, H, G, D,
            ops.QK_NORM | ops.QK_ROPE | ops.QK_STORE | ops.QK_QOUT)))
        runs = {"attention_table_sink": lambda: ops.attention_biased(q, k_plane, v_plane, ctx.positions, ctx.token_slot, table, page, H, G, D, D,
                                                                     D ** -0.5, o, sink=True, sink_logits=sink, distance_bias=bias, ctx=ctx),
                "attention_two_planes": lambda: ops.attention_biased(q, k_plane, v_plane, ctx.positions, ctx.token_slot, table, page, H, G, D, D,
                                                                     D ** -0.5, o, ctx=ctx),
                "paged_attention": lambda: ops.paged_attention(q, kv_u, ctx.positions, ctx.token_slot, table, page, H, G, D, None,
                                                               D ** -0.5, o, ctx=ctx)}
        for name, fn in runs.items():
            ms = timed(fn)
            kern[f"{name}_{what}"] = tensor(4.0 * H * D * T * (T + 1) / 2, ms) if what.startswith("prefill") else \
                hbm(rows * ctx_len * 2 * G * D * 2, ms)
    del pool, k_plane, v_plane, kv_u

    # the recurrences on the scan kernel: 2048 tokens of one request, and 64 one-token rows (state read and written
    # once per row): the matrix memory, the gated linear attention, the delta rule with a decay per head, and
    # Kaketar's delta rule with a decay per channel
    Hm, mk, mv = z["m_heads"], z["m_dim"], z["m_vdim"]
    Hd, Gd, dk, dv, taps = z["d_heads"], z["d_kv"], z["d_dim"], z["d_vdim"], z["taps"]

    def scan_record(n, ms, heads, k, v, io, work, state_words):
        total = io + work + (0 if n == T else 2 * rows * state_words * 4)
        return {"us": round(ms * 1e3, 1), "tokens_per_s": round(n / ms * 1e3, 1),
                "gflops_fp32": round(6.0 * n * heads * k * v / ms / 1e6, 1), "gbs": round(total / ms / 1e6, 1),
                "frac_hbm": round(total / ms / 1e6 / pk["hbm_gbs"], 3)}

    for what, n, seg in (("prefill_2048", T, [[0, 0, T, 0]]), ("decode_64_rows", rows, None)):
        slots = torch.zeros(n, dtype=torch.int32, device=device) if seg else torch.arange(n, dtype=torch.int32, device=device)
        seg_info = torch.tensor(seg, dtype=torch.int32, device=device) if seg else None
        # matrix memory and gated linear attention
        proj = torch.randn(n, Hm * (2 * mk + 2 * mv), device=device).to(bf)
        gate = proj[:, Hm * (2 * mk + mv):]
        for kind, zc, p0, per_head, act in (("log_gates", 2 * Hm, 12.0, True, "sigmoid"), ("channel_decay", Hm * mk, 1.0 / 8, False, "silu")):
            words = ops.linear_recurrence_state_floats(kind, Hm, mk, mv)
            state = torch.zeros(rows, words, device=device)
            zz = torch.randn(n, zc, device=device)
            zb = torch.randn(zc, device=device) + 3.0
            weight = torch.ones(Hm * mv if per_head else mv, device=device)
            ms = timed(lambda: ops.linear_recurrence(proj, kind, zz, zb, p0, gate, act, weight, per_head, 1e-5, slots, seg_info, state,
                                                     Hm, mk, mv, mk ** -0.5, bf))
            io = n * (Hm * (2 * mk + 2 * mv) * 2 + zc * 4 + Hm * mv * 2)
            work = n * (3 * Hm * mk + 2 * Hm * (mv + 1)) * 4 * 2
            name = "matrix_memory" if kind == "log_gates" else "gated_linear_attention"
            kern[f"{name}_{what}"] = scan_record(n, ms, Hm, mk, mv, io, work, words)
            del state
        # the two delta rules
        for name, G2, per_head in (("delta_rule_decay_per_head", Gd, True), ("kaketar_delta_rule_decay_per_channel", Hd, False)):
            channels = 2 * G2 * dk + Hd * dv
            words = ops.delta_rule_state_floats(Hd, G2, dk, dv, taps)
            state = torch.zeros(rows, words, device=device)
            conv_w = (torch.randn(channels, taps, device=device) * 0.5).to(bf)
            conv_t = conv_w.t().contiguous()
            proj = torch.randn(n, (channels + Hd + 7) // 8 * 8, device=device).to(bf)
            a = torch.randn(n, Hd if per_head else Hd * dk, device=device)
            dt_bias = torch.randn(Hd if per_head else Hd * dk, device=device) - 4.0
            rate = torch.ones(Hd, device=device)
            gate = torch.randn(n, Hd * dv, device=device).to(bf)
            weight = torch.ones(dv, device=device)
            ms = timed(lambda: ops.delta_rule(proj, conv_w, taps, a, dt_bias, rate, gate, weight, 1e-5, slots, seg_info, state,
                                              Hd, G2, dk, dv, dk ** -0.5, 1e-6, bf, conv_t=conv_t, decay_per_head=per_head,
                                              gate_act="silu" if per_head else "sigmoid"))
            io = n * ((channels + Hd) * 2 + a.shape[1] * 4 + Hd * dv * 2 + Hd * dv * 2)
            work = n * (2 * G2 * dk + 2 * Hd * dv + Hd * dk + Hd) * 4 * 2
            kern[f"{name}_{what}"] = scan_record(n, ms, Hd, dk, dv, io, work, words)
            del state
    ops.check_error_word(device)
    record["kernels"] = kern
    clock_record = clocks.stop(windows)
    first = record["sizes"][sorted(record["sizes"])[0]]["tetodra"]
    print(json.dumps({"metric": f"decode tok/s @ batch {batch} (Tetodra design sizes, context {context}, 1 B200)",
                      "value": first["decode_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
                      "ms_per_step": first["decode_ms"], "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                      "design": "tetodra", "clocks": clock_record, "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"]},
                      **record}))
    return 0


PEVOLORN_SIZES = {
    # width; layers in the order latent attention, pair, pair, latent attention that borrows the first one's cache
    # (repeated); latent attention: heads, unrotated and rotated query/key widths, value width, latent width (latent +
    # rotated = 128, which the tensor-core attention kernels take); the pair's attention: heads, key/value heads, widths;
    # the pair's state space: heads, head width, state, groups; the mixture: experts (the last two of the router's
    # outputs are identity experts), top, expert and shared widths (top * expert + shared = the dense width of the others)
    "1b": dict(width=2048, layers=8, vocab=32768, l_heads=16, l_dim=64, l_rot=32, l_vdim=64, l_rank=96, a_heads=16, a_kv=4,
               a_dim=128, s_heads=32, s_dim=64, s_state=128, s_groups=4, taps=4, experts=30, identity=2, groups=8, keep=4,
               top=4, expert_ff=1024, shared_ff=2048, ff=6144),
    "8b": dict(width=4096, layers=4, vocab=32768, l_heads=32, l_dim=64, l_rot=32, l_vdim=64, l_rank=96, a_heads=32, a_kv=8,
               a_dim=128, s_heads=64, s_dim=64, s_state=128, s_groups=8, taps=4, experts=62, identity=2, groups=8, keep=4,
               top=4, expert_ff=2048, shared_ff=4096, ff=12288),
}


def _pevolorn_at(z):
    from tiny_llm_infer_b200.config.pevolorn import (GroupedAttentionConfig, LatentConfig, MixtureConfig, PairConfig,
                                                      PevolornConfig, PevolornLayerConfig, StateSpaceConfig)
    moe = MixtureConfig(z["expert_ff"], z["experts"], z["top"], z["identity"], z["groups"], z["keep"], z["shared_ff"])

    def latent(kv_from):
        return PevolornLayerConfig("latent_attention", LatentConfig(
            z["l_heads"], z["l_dim"], z["l_rot"], z["l_vdim"], z["l_rank"], (z["l_dim"] + z["l_rot"]) ** -0.5, 10000.0,
            z["l_rot"], kv_from), moe)
    pair = PevolornLayerConfig("parallel", PairConfig(
        GroupedAttentionConfig(z["a_heads"], z["a_kv"], z["a_dim"], z["a_dim"], 8.0 / z["a_dim"], 30.0, 1000000.0, z["a_dim"] // 2),
        StateSpaceConfig(z["s_heads"], z["s_dim"], z["s_state"], z["s_groups"], z["taps"], z["s_groups"]), 1.2, 1.1), moe)
    layers = []
    for i in range(z["layers"]):
        layers.append([latent(None), pair, pair, latent(i - 3)][i % 4])
    return PevolornConfig(vocab=z["vocab"], width=z["width"], norm_eps=1e-6, postln_alpha=3.0, layers=tuple(layers))


def pevolorn_bench(args) -> int:
    """``--design pevolorn``: prefill and decode throughput of the Pevolorn design at sizes that resemble a real
    model's layers (random weights, bfloat16; layers in the order latent attention, attention beside a state space
    twice, latent attention on the first one's cache; a mixture of experts on every layer), beside the closest
    models the engine has at equal width, layers, feed-forward share and vocabulary, through the same step
    function: Panolorn (capped attention, mixtures on every second layer) and Qwen3 dense.  Then the design's
    kernels one by one beside their relatives, with their share of the measured peaks.  One JSON line."""
    import torch
    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.config import Qwen3Config
    from tiny_llm_infer_b200.config.panolorn import (AttentionMixerConfig, FeedForwardConfig, PanolornConfig,
                                                      PanolornLayerConfig)
    from tiny_llm_infer_b200.engine.batch import StepContext
    from tiny_llm_infer_b200.parts.registry import lookup
    from tiny_llm_infer_b200.parts.spec import PartSpec

    hx = _DesignHarness(args)
    device, pk, clocks, windows = hx.device, hx.pk, hx.clocks, hx.windows
    tokens_pf, batch, context, steps, warmup = hx.tokens_pf, hx.batch, hx.context, hx.steps, hx.warmup
    timed, run_model = hx.timed, hx.run_model
    record = {"sizes": {}}
    for size_name in ([args.model] if args.model in PEVOLORN_SIZES else sorted(PEVOLORN_SIZES)):
        z = PEVOLORN_SIZES[size_name]
        L, W, H, G, D = z["layers"], z["width"], z["a_heads"], z["a_kv"], z["a_dim"]
        vcfg = _pevolorn_at(z)
        pz = DESIGN_SIZES[size_name]
        pcfg = PanolornConfig(vocab=z["vocab"], width=W, embedding_scale=math.sqrt(W), norm_eps=1e-5, layers=tuple(
            PanolornLayerConfig("attention", AttentionMixerConfig(H, G, D, D, 1.0 / math.sqrt(D), 50.0, pz["chunk"]),
                                FeedForwardConfig("dense", z["ff"]) if i % 2 == 0 else
                                FeedForwardConfig("moe", pz["expert_ff"], experts=pz["experts"], top=pz["top"], shared_ff=pz["shared_ff"]))
            for i in range(L)))
        qcfg = Qwen3Config(hidden_size=W, intermediate_size=z["ff"], num_hidden_layers=L, num_attention_heads=H,
                           num_key_value_heads=G, head_dim=D, vocab_size=z["vocab"], max_position_embeddings=8192,
                           tie_word_embeddings=True, layer_types=("full_attention",) * L)
        # weights per layer kind: what a token multiplies with, and what a decode step of `batch` rows reads
        lat_own = W * (z["l_heads"] * (z["l_dim"] + z["l_rot"]) + z["l_rank"] + z["l_rot"] + z["l_heads"]) \
            + z["l_rank"] * z["l_heads"] * (z["l_dim"] + z["l_vdim"]) + z["l_heads"] * z["l_vdim"] * W
        lat_borrowed = lat_own - W * (z["l_rank"] + z["l_rot"])
        inner = z["s_heads"] * z["s_dim"]
        pair_w = W * ((H + 2 * G) * D + H) + H * D * W + W * (2 * inner + 2 * z["s_groups"] * z["s_state"] + z["s_heads"]) + inner * W
        total = z["experts"] + z["identity"]
        moe_active = W * total + 2 * W * (z["top"] * z["expert_ff"] + z["shared_ff"])
        moe_read = W * total + 2 * W * (min(z["experts"], batch * z["top"]) * z["expert_ff"] + z["shared_ff"])
        kinds = [lat_own, pair_w, pair_w, lat_borrowed]
        mix = sum(kinds[i % 4] for i in range(L))
        v_params = {"active": mix + L * moe_active + z["vocab"] * W, "read": mix + L * moe_read + z["vocab"] * W}
        _, v_kv, v_state = _model_costs(vcfg, context)
        attn = W * (H + 2 * G) * D + H * D * W
        gate = W * H * D
        hit = min(pz["experts"], batch * pz["top"])
        p_params = {"active": L * (attn + gate + 3 * W * z["ff"]) + (L // 2) * W * pz["experts"] + z["vocab"] * W,
                    "read": L * (attn + gate) + (L - L // 2) * 3 * W * z["ff"]
                    + (L // 2) * (3 * W * (hit * pz["expert_ff"] + pz["shared_ff"]) + W * pz["experts"]) + z["vocab"] * W}
        q_params = L * (attn + 3 * W * z["ff"]) + z["vocab"] * W
        kv = 2 * G * D * 2 * L
        entry = {"config": z, "params": {}}
        for label, cfg, params, kvb, st in (("pevolorn", vcfg, v_params, v_kv, v_state), ("panolorn", pcfg, p_params, kv, 0.0),
                                            ("qwen3_dense", qcfg, {"active": q_params, "read": q_params}, kv, 0.0)):
            print(f"[bench] design sizes {size_name}: {label}", file=sys.stderr, flush=True)
            r = run_model(cfg, f"{label} {size_name}", params, kvb, st)
            r["prefill_frac_of_measured"] = round(r["prefill_tflops"] / pk["bf16_tflops"], 4)
            r["decode_hbm_frac_of_measured"] = round(r["decode_gbs"] / pk["hbm_gbs"], 4)
            print(f"[bench] {r}", file=sys.stderr, flush=True)
            entry[label] = r
            entry["params"][label] = params
        record["sizes"][size_name] = entry

    # ---- kernels one by one at the larger sizes (L2 flushed between runs)
    z = PEVOLORN_SIZES["8b"]
    W, bf, T = z["width"], torch.bfloat16, tokens_pf
    kern = {}

    def hbm(nbytes, ms):
        return {"us": round(ms * 1e3, 1), "gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3)}

    def tensor(flops, ms):
        return {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1), "frac_tensor": round(flops / ms / 1e9 / pk["bf16_tflops"], 3)}

    # the norm of a weighted sum that becomes the stream, beside the sums with a norm of the other designs
    h = torch.randn(T * 4, W, device=device)
    deltas = [torch.randn(T * 4, W, device=device).to(bf) for _ in range(2)]
    gain32, gain16 = torch.ones(W, device=device), torch.ones(W, device=device, dtype=bf)
    bias = torch.randn(W, device=device)
    out = torch.empty_like(deltas[0])
    per = h.numel()
    kern["sum_rmsnorm_2_outputs_bias"] = hbm(per * (8 + 2 * 2 + 2), timed(lambda: ops.sum_rmsnorm(h, deltas, [1.2, 1.1], 3.0, gain32, 1e-6, out, bias=bias)))
    kern["sum_rmsnorm_1_output"] = hbm(per * (8 + 2 + 2), timed(lambda: ops.sum_rmsnorm(h, deltas[:1], [1.0], 3.0, gain32, 1e-6, out)))
    kern["postnorm_add_rmsnorm"] = hbm(per * (8 + 2 + 2), timed(lambda: ops.add_rmsnorm(h, deltas[0], gain16, 1e-5, out, post_gain=gain16, post_eps=1e-5)))
    kern["add_rmsnorm"] = hbm(per * (8 + 2 + 2), timed(lambda: ops.add_rmsnorm(h, deltas[0], gain16, 1e-5, out)))
    del h, deltas, out

    rows, page, ctx_len = 64, 16, context

    def context_for(segs):
        seg, tiles, dec, row = [], [], [], 0
        for s, (slot, p0, n) in enumerate(segs):
            seg.append([slot, row, n, p0])
            if n == 1:
                dec.append(row)
            else:
                tiles += [(s, off) for off in range(0, n, 64)]
            row += n
        tiles.sort(key=lambda t: (t[1] % 256 != 0, t[1] % 128 != 0))
        pos = torch.tensor([p0 + i for _, p0, n in segs for i in range(n)], dtype=torch.int32, device=device)
        slot = torch.tensor([sl for sl, _, n in segs for _ in range(n)], dtype=torch.int32, device=device)
        return StepContext(tokens=row, token_ids=None, positions=pos, token_slot=slot, want_rows=None, segments=[],
                           seg_info=torch.tensor(seg, dtype=torch.int32, device=device),
                           dec_rows=None if len(dec) == row else torch.tensor(dec, dtype=torch.int32, device=device),
                           n_dec=len(dec), pf_tiles=torch.tensor(tiles, dtype=torch.int32, device=device).view(-1, 2),
                           n_tiles=len(tiles), n_tiles128=sum(1 for t in tiles if t[1] % 128 == 0),
                           n_tiles256=sum(1 for t in tiles if t[1] % 256 == 0), max_context=ctx_len, max_segment=max(n for _, _, n in segs))

    # the pair's attention (biases, rotation of half a head, unit queries and keys, cap, a gate per head) beside
    # Panolorn's (unit queries and keys, cap, slopes, chunk, a gate per element) on the same kernels, and the
    # latent attention (keys of 128 whose first 96 elements are the values, one key head for all query heads)
    H, G, D = z["a_heads"], z["a_kv"], z["a_dim"]
    n_pages = rows * ctx_len // page
    table = torch.arange(n_pages, dtype=torch.int32, device=device).view(rows, ctx_len // page).contiguous()
    pool = (torch.randn(n_pages, 2 * G * page * D, device=device) * 0.5).to(bf)
    k_plane = pool[:, :G * page * D].unflatten(1, (G, page, D))
    v_plane = pool[:, G * page * D:].unflatten(1, (G, page, D))
    lat_plane = pool[:, :page * D].unflatten(1, (1, page, D))
    inv_freq = (1000000.0 ** (-torch.arange(D // 4, dtype=torch.float64) * 4 / D)).float().to(device)
    in_bias = torch.randn((H + 2 * G) * D, device=device)
    slopes = torch.rand(H, device=device) * 0.01
    LH, rank = z["l_heads"], z["l_rank"]
    for what, segs in (("prefill_2048", [(0, 0, T)]), ("decode_64_rows_ctx_2048", [(i, ctx_len - 1, 1) for i in range(rows)])):
        ctx = context_for(segs)
        n = ctx.tokens
        q = torch.randn(n, H * D, device=device).to(bf)
        o = torch.empty_like(q)
        proj = torch.randn(n, (H + 2 * G) * D + 2 * H * D, device=device).to(bf)
        head_gate, full_gate = proj[:, (H + 2 * G) * D:(H + 2 * G) * D + H], proj[:, (H + 2 * G) * D:(H + 2 * G) * D + H * D]
        moved = n * ((H + 2 * G) * D * 2 + (H + 2 * G) * D * 2)
        kern[f"qkv_store_bias_rotation_unit_{what}"] = hbm(moved, timed(lambda: ops.qkv_unit_store(
            proj, q, ctx.positions, ctx.token_slot, table, k_plane, v_plane, page, H, G, D, D, 1e-6, inv_freq=inv_freq,
            rot_dims=D // 2, bias=in_bias)))
        kern[f"panolorn_qkv_store_unit_{what}"] = hbm(moved, timed(lambda: ops.qkv_unit_store(
            proj, q, ctx.positions, ctx.token_slot, table, k_plane, v_plane, page, H, G, D, D, 1e-6)))
        ql = torch.randn(n, LH * D, device=device).to(bf)
        ol = torch.empty(n, LH * rank, device=device, dtype=bf)
        runs = {"attention_cap_gate_per_head": (lambda: ops.attention_biased(
                    q, k_plane, v_plane, ctx.positions, ctx.token_slot, table, page, H, G, D, D, 8.0 / D, o, softcap=30.0,
                    gate=head_gate, gate_per_head=True, ctx=ctx), H, D, D, G * 2 * D),
                "panolorn_attention_cap_slopes_gate": (lambda: ops.attention_biased(
                    q, k_plane, v_plane, ctx.positions, ctx.token_slot, table, page, H, G, D, D, D ** -0.5, o, softcap=50.0,
                    chunk=4096, sink=True, slopes=slopes, gate=full_gate, ctx=ctx), H, D, D, G * 2 * D),
                "latent_attention_keys_are_values": (lambda: ops.attention_biased(
                    ql, lat_plane, lat_plane, ctx.positions, ctx.token_slot, table, page, LH, 1, D, rank, D ** -0.5, ol,
                    values_in_keys=True, ctx=ctx), LH, D, rank, D)}
        for name, (fn, heads, dk, dv, row_elems) in runs.items():
            ms = timed(fn)
            kern[f"{name}_{what}"] = tensor(2.0 * heads * (dk + dv) * T * (T + 1) / 2, ms) if what.startswith("prefill") else \
                hbm(rows * ctx_len * row_elems * 2, ms)
    del pool, k_plane, v_plane, lat_plane

    # the state space on the scan kernel beside Tetodra's gated linear attention at equal state: 2048 tokens of one
    # request, and 64 one-token rows (state read and written once per row)
    Hs, P, N, Gs, taps = z["s_heads"], z["s_dim"], z["s_state"], z["s_groups"], z["taps"]
    inner, channels = Hs * P, Hs * P + 2 * Gs * N

    def scan_record(n, ms, io, work, state_words):
        total = io + work + (0 if n == T else 2 * rows * state_words * 4)
        return {"us": round(ms * 1e3, 1), "tokens_per_s": round(n / ms * 1e3, 1),
                "gflops_fp32": round(6.0 * n * Hs * N * P / ms / 1e6, 1), "gbs": round(total / ms / 1e6, 1),
                "frac_hbm": round(total / ms / 1e6 / pk["hbm_gbs"], 3)}

    for what, n, seg in (("prefill_2048", T, [[0, 0, T, 0]]), ("decode_64_rows", rows, None)):
        slots = torch.zeros(n, dtype=torch.int32, device=device) if seg else torch.arange(n, dtype=torch.int32, device=device)
        seg_info = torch.tensor(seg, dtype=torch.int32, device=device) if seg else None
        words = ops.state_space_state_floats(Hs, Gs, N, P, taps)
        state = torch.zeros(rows, words, device=device)
        proj = torch.randn(n, (inner + channels + Hs + 7) // 8 * 8, device=device).to(bf)
        conv_w = (torch.randn(channels, taps, device=device) * 0.5).to(bf)
        conv_b = torch.randn(channels, device=device) * 0.1
        dt_bias, rate, skip = torch.randn(Hs, device=device) - 2.0, torch.ones(Hs, device=device), torch.ones(Hs, device=device)
        weight = torch.ones(inner, device=device)
        conv_t = conv_w.t().contiguous()
        ms = timed(lambda: ops.state_space(proj, conv_w, conv_b, taps, dt_bias, rate, skip, weight, 1e-6, Gs, slots, seg_info,
                                           state, Hs, Gs, N, P, bf, conv_t=conv_t))
        io = n * ((inner + channels + Hs) * 2 + inner * 2)
        work = n * (2 * Gs * N + 2 * inner + 2 * Hs) * 4 * 2
        kern[f"state_space_{what}"] = scan_record(n, ms, io, work, words)
        del state
        words = ops.linear_recurrence_state_floats("channel_decay", Hs, N, P)
        state = torch.zeros(rows, words, device=device)
        proj = torch.randn(n, Hs * (2 * N + 2 * P), device=device).to(bf)
        gate = proj[:, Hs * (2 * N + P):]
        zz, zb, w2 = torch.randn(n, Hs * N, device=device), torch.randn(Hs * N, device=device) + 3.0, torch.ones(P, device=device)
        ms = timed(lambda: ops.linear_recurrence(proj, "channel_decay", zz, zb, 1.0 / 8, gate, "silu", w2, False, 1e-5, slots, seg_info,
                                                 state, Hs, N, P, N ** -0.5, bf))
        io = n * (Hs * (2 * N + 2 * P) * 2 + Hs * N * 4 + inner * 2)
        work = n * (3 * Hs * N + 2 * inner) * 4 * 2
        kern[f"tetodra_gated_linear_attention_{what}"] = scan_record(n, ms, io, work, words)
        del state

    # the mixture: the router over all experts beside the router by largest logits, and the whole part (plain experts
    # with the squared ReLU, identity experts) beside Panolorn's (gated experts) at equal widths, 8 rows and 8192
    E, I, top, eff, sff = z["experts"], z["identity"], z["top"], z["expert_ff"], z["shared_ff"]
    zl = torch.randn(8192, E + I, device=device)
    corr = torch.randn(E + I, device=device) * 0.01
    kern["moe_route_grouped_8192_rows"] = {"us": round(timed(lambda: ops.moe_route_grouped(zl, top, "softmax", corr, z["groups"], z["keep"])) * 1e3, 1)}
    kern["moe_route_8192_rows"] = {"us": round(timed(lambda: ops.moe_route(zl, top)) * 1e3, 1)}
    cls = lookup("feed_forward", "moe")
    ours = cls(dtype=bf, device=device, hidden_size=W, experts=E, top=top, expert_size=eff, activation="relu2",
               router_scores="softmax_all", weight_on="output", gated=False, names=("up", "down"), correction=True,
               groups=(z["groups"], z["keep"]), identity=I,
               shared=PartSpec("mlp", dict(hidden_size=W, intermediate_size=sff, activation="relu2", names=("up", "down")), "shared."))
    theirs = cls(dtype=bf, device=device, hidden_size=W, experts=E + I, top=top, expert_size=eff, activation="silu",
                 shared=PartSpec("swiglu", dict(hidden_size=W, intermediate_size=sff, names=("gate", "up", "down")), "shared."))
    for part in (ours, theirs):
        specs = type(part).param_specs(**{k: v for k, v in dict(
            hidden_size=W, experts=part.experts, top=top, expert_size=eff, shared=part.shared_spec, gated=part.gated,
            names=part.names, correction=part.correction, identity=part.identity).items()})
        part.load({name: (torch.randn(spec.shape, device=device) * (0.02 if len(spec.shape) == 2 else 0.01)).to(bf)
                   for name, spec in specs.items()})
    for n in (8, 8192):
        x = torch.randn(n, W, device=device).to(bf)
        for name, part, mats in (("mixture_plain_experts_identity", ours, 2), ("panolorn_mixture_gated_experts", theirs, 3)):
            ms = timed(lambda: part.forward(x, None))
            if n == 8:
                hit = min(part.experts, n * top)
                kern[f"{name}_{n}_rows"] = hbm(mats * W * (hit * eff + sff) * 2, ms)
            else:
                kern[f"{name}_{n}_rows"] = tensor(2.0 * n * mats * W * (top * eff + sff), ms)
    ops.check_error_word(device)
    record["kernels"] = kern
    clock_record = clocks.stop(windows)
    first = record["sizes"][sorted(record["sizes"])[0]]["pevolorn"]
    print(json.dumps({"metric": f"decode tok/s @ batch {batch} (Pevolorn design sizes, context {context}, 1 B200)",
                      "value": first["decode_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
                      "ms_per_step": first["decode_ms"], "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                      "design": "pevolorn", "clocks": clock_record, "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"]},
                      **record}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="8b", choices=sorted(set(MODELS) | set(DESIGN_SIZES) | set(TETODRA_SIZES) | set(PEVOLORN_SIZES)),
                    help="the sizes: 8b is the benchmark configuration, 0.6b and 32b the other two the reference is quoted on")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the model has (named in the record) if memory or time needs it")
    ap.add_argument("--mixed", action="store_true",
                    help="the mixed run (64 requests, prompts of 16 to 1024 tokens, 256 outputs each at temperature "
                         "0.6, budget 2048, through LLM.generate) with the sizes of --model; at the default sizes it "
                         "runs anyway, with the Qwen3-0.6B sizes it belongs to")
    ap.add_argument("--skip-points", action="store_true",
                    help="leave out the batch 1 and 64 points, the 128-token workload and the 0.6B mixed run")
    ap.add_argument("--skip-check", action="store_true", help="leave out the logits check before the timed phases")
    ap.add_argument("--ref-all", action="store_true",
                    help="reference arm: its model_main --bench at batch 1, 8 and 64 instead of --batch alone")
    ap.add_argument("--design", default=None, choices=["panolorn", "kaketar", "tetodra", "pevolorn"],
                    help="instead of the default workload: this design's prefill and decode throughput at sizes that "
                         "resemble a real model's layers beside Qwen3 dense at equal sizes, and its kernels one by one")
    ap.add_argument("--only", default="all", choices=["all", "prefill", "decode", "e2e", "mixed", "p128"],
                    help="run one phase only (for profiling a small case); the record then lacks the others")
    args = ap.parse_args()
    if args.design is not None:
        if args.gpus != 1 or args.impl != "ours":
            print("bench.py: --design runs this engine on one GPU")
            return 2
        return {"kaketar": kaketar_bench, "tetodra": tetodra_bench, "pevolorn": pevolorn_bench}.get(args.design, design_bench)(args)
    if args.model not in MODELS:
        ap.error(f"--model {args.model} goes with --design")
    model_name, model_sizes = MODELS[args.model]
    if args.layers is None:
        args.layers = model_sizes["num_hidden_layers"]
    if args.only == "mixed":
        args.mixed = True

    if args.impl == "reference":
        return reference_arm(args, model_name, model_sizes)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} has nothing to measure")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch

    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.config import Qwen3Config
    from tiny_llm_infer_b200.engine import LLM, StepEntry, random_model
    from tiny_llm_infer_b200.sampling import SamplingParams

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    device = "cuda:0"
    pk = peaks()
    sizes = dict(model_sizes, num_hidden_layers=args.layers)
    cfg = Qwen3Config(layer_types=("full_attention",) * args.layers, **sizes)
    ops.lib()
    t0 = time.perf_counter()
    model = random_model(cfg, seed=0, dtype=torch.bfloat16, device=device, std=0.02)
    torch.cuda.synchronize()
    print(f"[bench] model built in {time.perf_counter() - t0:.1f} s", file=sys.stderr, flush=True)

    max_batch = 64 if (not args.skip_points or args.mixed) else max(args.batch, 1)
    pages = max_batch * (CONTEXT // PAGE) + 2 * (PREFILL_TOKENS // PAGE) + 64
    llm = LLM(None, dtype="bfloat16", max_model_len=CONTEXT, num_kv_blocks=pages, block_size=PAGE,
              max_num_batched_tokens=PREFILL_TOKENS, max_num_seqs=max_batch, device=device, loaded=(model, cfg))
    runner, engine = llm.runner, llm.engine
    gen = torch.Generator().manual_seed(0)
    vocab = cfg.vocab_size

    def tokens(n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    # byte and flop counts
    layer_params = _layer_params(sizes)
    weight_bytes = 2 * (args.layers * layer_params + vocab * cfg.hidden_size)
    kv_bytes_per_token = 2 * cfg.kv_dim * 2 * args.layers
    windows = []
    clocks = ClockSampler()
    clocks.start()

    # ---------------------------------------------------------------- prefill of 2048 tokens
    def prefill_once():
        toks = tokens(PREFILL_TOKENS)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry("prefill", toks, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.release("prefill")
        return start.elapsed_time(end)

    prefill = None
    if args.only in ("all", "prefill"):
        for _ in range(3):
            prefill_once()
        w0 = time.perf_counter()
        prefill_ms = statistics.median(prefill_once() for _ in range(5))
        windows.append((w0, time.perf_counter(), "prefill"))
        prefill_flops = 2.0 * PREFILL_TOKENS * args.layers * layer_params \
            + args.layers * 2.0 * PREFILL_TOKENS ** 2 * cfg.q_dim + 2.0 * vocab * cfg.hidden_size
        prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                   "ms": round(prefill_ms, 3),
                   "frac": round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        if pk.get("bf16_tflops_sustained"):
            prefill["frac_sustained"] = round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
        print(f"[bench] prefill {prefill}", file=sys.stderr, flush=True)

    # ---------------------------------------------------------------- decode, timed on the device
    def decode_device(batch, steps, warmup, end_context=CONTEXT, what="decode"):
        """Tokens per second of `steps` decode steps of `batch` requests that end at `end_context`."""
        start_len = end_context - (steps + warmup)
        names = [f"d{batch}_{i}" for i in range(batch)]
        for name in names:                                   # real prefill, in portions of 2048
            toks = tokens(start_len)
            for i in range(0, start_len, PREFILL_TOKENS):
                runner.step([StepEntry(name, toks[i:i + PREFILL_TOKENS], [])])
        params = torch.tensor([[0.6, 1.0]] * batch, device=device)
        seeds = torch.arange(batch, dtype=torch.int64, device=device)
        out = torch.empty(batch, dtype=torch.int32, device=device)
        nxt = [[int(t)] for t in torch.randint(0, vocab, (batch,), generator=gen)]
        times = []
        torch.cuda.synchronize()
        before = ops.launches
        w_start = None
        for it in range(warmup + steps):
            if it == warmup:
                torch.cuda.synchronize()
                before = ops.launches
                w_start = time.perf_counter()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            logits = runner.step([StepEntry(n, t, [0]) for n, t in zip(names, nxt)])
            ops.sample(logits, params, seeds, out, any_nucleus=False)
            end.record()
            nxt = [[t] for t in out.cpu().tolist()]          # the next step feeds what was sampled
            if it >= warmup:
                times.append((start, end))
        torch.cuda.synchronize()
        windows.append((w_start, time.perf_counter(), f"{what} b{batch}"))
        launches = ops.launches - before
        ms = sum(a.elapsed_time(b) for a, b in times) / steps
        for name in names:
            runner.release(name)
        mean_ctx = start_len + warmup + (steps - 1) / 2.0 + 1
        return batch / (ms / 1e3), ms, launches, mean_ctx

    def hbm_fraction(batch, ms, ctx):
        return (weight_bytes + batch * ctx * kv_bytes_per_token) / (ms / 1e3) / 1e9

    value = ms_per_step = launches = mean_ctx = roofline = None
    if args.only in ("all", "decode"):
        value, ms_per_step, launches, mean_ctx = decode_device(args.batch, args.steps, args.warmup)
        achieved = hbm_fraction(args.batch, ms_per_step, mean_ctx)
        roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / pk["hbm_gbs"], 4)}
        print(f"[bench] decode b{args.batch}: {value:.1f} tok/s, {ms_per_step:.3f} ms/step, {roofline}",
              file=sys.stderr, flush=True)

    # ---------------------------------------------------------------- the same through the entry point
    def decode_e2e(batch, steps, warmup):
        # requests whose prompts are done decode while the others' prompts are still computed:
        # leave them room for those steps too, so that all are still running when timing ends
        extra = batch * -(-CONTEXT // PREFILL_TOKENS) + 2
        sp = SamplingParams(max_tokens=steps + warmup + extra, temperature=0.6, ignore_eos=True)
        start_len = CONTEXT - sp.max_tokens - 1
        for i in range(batch):
            engine.add_request(tokens(start_len), SamplingParams(**{**sp.__dict__, "seed": i + 1}))
        while engine.scheduler.waiting:                      # prompts, outside the timed region
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        t_start = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t_start
        windows.append((t_start, t_start + elapsed, f"e2e b{batch}"))
        while not engine.is_finished():
            engine.step()
        bucket = 1
        while bucket < batch:
            bucket *= 2
        # rows' ids/positions/slots/wanted, where the tokens sampled by the step before go, sampling params, keys
        h2d = (4 * bucket + 2 * batch) * 4 + batch * 8 + batch * 8
        return batch * steps / elapsed, h2d, batch * 4

    e2e = None
    if args.only in ("all", "e2e"):
        e2e_value, h2d, d2h = decode_e2e(args.batch, args.steps, args.warmup)
        e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        print(f"[bench] e2e b{args.batch}: {e2e_value:.1f} tok/s", file=sys.stderr, flush=True)

    points = {}
    if not args.skip_points and args.only == "all":
        for b in (1, 64):
            v, ms_b, _, ctx_b = decode_device(b, min(args.steps, 32), args.warmup)
            points[f"decode_b{b}"] = round(v, 1)
            bw = hbm_fraction(b, ms_b, ctx_b)
            points[f"decode_b{b}_hbm_frac"] = round(bw / pk["hbm_gbs"], 4)
            print(f"[bench] decode b{b}: {v:.1f} tok/s, {ms_b:.3f} ms/step, {bw:.0f} GB/s", file=sys.stderr, flush=True)

    # ---------------------------------------------------------------- 128-token prompts, 128 outputs
    # The reference's own benchmark (benchmark/run_benchmark.sh:32-42, model/model_main.cpp:150-175,
    # 354-368): `batch` prompts of 128 uniform token ids, 128 outputs each at temperature 0.6 with
    # end-of-sequence ignored, output tokens / wall time from the first add_request to the last result,
    # prompts included; three warm-up runs, then the median of five.  Beside it the decode steps of the
    # same workload alone (contexts 128 to 256), timed on the device, with their share of the HBM peak.
    def p128_e2e(batch):
        rates = []
        for run in range(8):
            prompts = [tokens(128) for _ in range(batch)]
            params = [SamplingParams(max_tokens=128, temperature=0.6, ignore_eos=True, seed=1000 * run + i + 1)
                      for i in range(batch)]
            torch.cuda.synchronize()
            t_start = time.perf_counter()
            outs = llm.generate(prompts, params)
            elapsed = time.perf_counter() - t_start
            assert sum(len(o.token_ids) for o in outs) == 128 * batch
            if run >= 3:
                rates.append(128 * batch / elapsed)
                windows.append((t_start, t_start + elapsed, f"128/128 e2e b{batch}"))
        return statistics.median(rates)

    if (not args.skip_points and args.only == "all") or args.only == "p128":
        for b in (1, 8, 64):
            v, ms_b, _, ctx_b = decode_device(b, 120, 8, end_context=256, what="128/128 decode")
            points[f"p128_decode_b{b}"] = round(v, 1)
            points[f"p128_hbm_frac_b{b}"] = round(hbm_fraction(b, ms_b, ctx_b) / pk["hbm_gbs"], 4)
            points[f"p128_e2e_b{b}"] = round(p128_e2e(b), 1)
            print(f"[bench] 128/128 b{b}: decode steps {v:.1f} tok/s ({ms_b:.3f} ms/step, {points[f'p128_hbm_frac_b{b}']} of HBM), "
                  f"end to end {points[f'p128_e2e_b{b}']} output tok/s", file=sys.stderr, flush=True)

    # ---------------------------------------------------------------- the logits of the model that was timed
    # (after the timed phases: seconds of float32 products before them leave the GPU at lower clocks
    # under its power cap; a mismatch fails the run all the same, and no record is printed)
    check = None
    if not args.skip_check and args.only == "all":
        t0 = time.perf_counter()
        check = precheck(model, cfg, sizes, device)
        print(f"[bench] logits check in {time.perf_counter() - t0:.1f} s: {check}", file=sys.stderr, flush=True)
        if not check["ok"]:
            clocks.stop(windows)
            print(json.dumps({"error": "the bfloat16 kernels' logits do not match the float32 path", "check": check}))
            return 1

    # ---------------------------------------------------------------- the mixed run
    def mixed_run(the_llm, the_vocab):
        g2 = torch.Generator().manual_seed(1)

        def workload():
            lens = torch.randint(16, 1025, (64,), generator=g2).tolist()
            return ([torch.randint(0, the_vocab, (n,), generator=g2).tolist() for n in lens],
                    [SamplingParams(max_tokens=256, temperature=0.6, ignore_eos=True, seed=i + 1) for i in range(64)])
        the_llm.generate(*workload())                               # first run: graphs are captured
        prompts, params = workload()
        torch.cuda.synchronize()
        t_start = time.perf_counter()
        outs = the_llm.generate(prompts, params)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t_start
        windows.append((t_start, t_start + elapsed, "mixed run"))
        made = sum(len(o.token_ids) for o in outs)
        return {"value": round(made / elapsed, 1), "unit": "generated tokens/s", "requests": 64,
                "prompt_tokens": sum(map(len, prompts)), "generated_tokens": made, "seconds": round(elapsed, 3)}

    mixed = None
    if args.mixed:
        mixed = dict(mixed_run(llm, vocab), model=model_name)
    elif args.model == "8b" and not args.skip_points and args.only == "all":
        # the mixed continuous-batching run belongs to the Qwen3-0.6B sizes: a second, small model
        del llm, runner, engine, model
        torch.cuda.empty_cache()
        name06, sizes06 = MODELS["0.6b"]
        cfg06 = Qwen3Config(layer_types=("full_attention",) * sizes06["num_hidden_layers"], **sizes06)
        model06 = random_model(cfg06, seed=0, dtype=torch.bfloat16, device=device, std=0.02)
        llm06 = LLM(None, dtype="bfloat16", max_model_len=CONTEXT, num_kv_blocks=64 * (1280 // PAGE) + 64, block_size=PAGE,
                    max_num_batched_tokens=PREFILL_TOKENS, max_num_seqs=64, device=device, loaded=(model06, cfg06))
        mixed = dict(mixed_run(llm06, cfg06.vocab_size), model=name06)
    if mixed is not None:
        points["mixed_run_tokens_per_s"] = mixed["value"]
        print(f"[bench] mixed run: {mixed}", file=sys.stderr, flush=True)

    record = {
        "metric": f"decode tok/s @ batch {args.batch} ({model_name}, context 4096, 1 B200)",
        "value": None if value is None else round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": None if ms_per_step is None else round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids)",
        "config": _config(model_name, args.batch, args.layers, model_sizes, sizes, mean_ctx, weight_bytes, pk),
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill, "roofline": roofline, "points": points, "mixed": mixed, "check": check,
        "clocks": clocks.stop(windows),
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
