"""Varunex on the GPU against the plain float64 model (plain_varunex.py): each
mechanism alone; whole prompts; token-by-token decoding from the first token;
portions down to two tokens; batches of unequal requests; pages and slots used
again; keys far away, at page borders and at the edges of the window; the sink;
long decoding through graphs; greedy generation through the scheduler; the
trace program."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_varunex as P
from tiny import nmse, read_weights
from varunex_util import CONFIGS, diff_layer, latent_layer, memory_layer, model_folder, random_tokens, write_folder

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# float32: the engine against the float64 plain model.  bfloat16: against the plain model with
# the matrices rounded to bfloat16 (activations are not rounded there, so the bound is that of
# 16-bit activations through a few layers).
BOUND = {"float32": 1e-9, "bfloat16": 2e-3}


def rounded(w, dtype):
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()} if dtype == "bfloat16" else w


def weights_for(name, dtype):
    return rounded(read_weights(model_folder(name)), dtype)


_plain = {}


def plain_logits(name, dtype, tokens):
    key = (name, dtype, tuple(tokens))
    if key not in _plain:
        with torch.no_grad():
            _plain[key] = P.forward(CONFIGS[name], weights_for(name, dtype), list(tokens))
    return _plain[key]


def engine_for(name, dtype, **kw):
    from kipp_b200.engine import Engine
    opts = dict(dtype=dtype, page_size=16, cache_tokens=1024, max_requests=4, max_batch_tokens=1024)
    opts.update(kw)
    return Engine.from_folder(model_folder(name), **opts)


def close(got, want, dtype, what="", factor=1.0):
    e = nmse(got.cpu(), want)
    assert e <= BOUND[dtype] * factor, f"{what}: NMSE {e:.3e} > {BOUND[dtype] * factor:.1e}"


def layers_of(kind):
    return [(n, i) for n in sorted(CONFIGS) for i, l in enumerate(CONFIGS[n]["layers"]) if l["type"] == kind]


# ------------------------------------------------------------------ each mechanism alone
def run_mixer(name, layer, dtype, fn, portions):
    """The layer's mixer on random input, in portions: each reads the cache or
    the state the one before left."""
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    T = sum(portions)
    g = torch.Generator().manual_seed(100 + layer)
    h_dev = torch.randn(T, cfg["width"], generator=g, dtype=torch.float64).to("cuda", eng.dtype).contiguous()
    w = {k: v.double() for k, v in weights_for(name, dtype).items()}
    with torch.no_grad():
        want = fn(w, f"l{layer}.mix.", cfg["layers"][layer]["mixer"], h_dev.double().cpu(), cfg["norm"]["eps"])
    out = torch.zeros(T, cfg["width"], device="cuda")
    at = 0
    for n in portions:
        eng.run_part([StepEntry("m", [0] * n, [])], layer, "mixer", input=h_dev[at:at + n].contiguous(), residual=out[at:at + n])
        at += n
    close(out, want, dtype, f"{name} layer {layer}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", layers_of("latent_attention"))
def test_latent_attention_alone(name, layer, dtype):
    run_mixer(name, layer, dtype, P.latent_attention, (40, 1, 2, 35, 1))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", layers_of("attention"))
def test_differential_attention_alone(name, layer, dtype):
    run_mixer(name, layer, dtype, P.differential_attention, (33, 2, 1, 70, 1, 1))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", layers_of("mlstm"))
def test_gated_memory_alone(name, layer, dtype):
    run_mixer(name, layer, dtype, P.mlstm, (17, 1, 2, 40, 1))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [("A", 0), ("B", 1), ("C", 3)])
def test_layer_norm_and_feed_forward_alone(name, layer, dtype):
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    T = 33
    g = torch.Generator().manual_seed(300 + layer)
    x = (3.0 * torch.randn(T, cfg["width"], generator=g) + 0.7).to("cuda").contiguous()
    w = {k: v.double() for k, v in weights_for(name, dtype).items()}
    p = f"l{layer}."
    normed = torch.zeros(T, cfg["width"], device="cuda", dtype=eng.dtype)
    eng.run_part([StepEntry("n", [0] * T, [])], layer, "input_norm", residual=x, output=normed)
    close(normed.double(), P.layer_norm(x.double().cpu(), w[p + "norm1"], w[p + "norm1.b"], cfg["norm"]["eps"]), dtype, "layer norm",
          factor=0.02 if dtype == "bfloat16" else 1.0)
    out = torch.zeros(T, cfg["width"], device="cuda")
    eng.run_part([StepEntry("f", [0] * T, [])], layer, "feed_forward", input=normed, residual=out)
    close(out, P.dense_ff(w, p + "mlp.", normed.double().cpu()), dtype, "feed-forward")


# ------------------------------------------------------------------ whole models
LENGTH = {"A": 131, "B": 70, "C": 230, "D": 50, "E": 150, "F": 140}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_every_way_of_cutting_it(name, dtype):
    """Whole; token by token from the very first token; portions down to two
    tokens: every position against the plain model, and (32-bit) the ways of
    cutting against one another."""
    from kipp_b200.engine import StepEntry
    toks = random_tokens(CONFIGS[name]["vocab"], LENGTH[name], seed=1)
    want = plain_logits(name, dtype, toks)
    eng = engine_for(name, dtype)
    n = len(toks)
    whole = eng.step([StepEntry("w", toks, list(range(n)))], check=True).clone()
    eng.finish("w")
    close(whole, want, dtype, "whole")
    rows = [eng.step([StepEntry("t", [t], [0])]).clone() for t in toks]
    eng.synchronize()
    eng.finish("t")
    single = torch.cat(rows)
    close(single, want, dtype, "token by token")
    # the first tokens of a sequence, each position on its own
    for pos in range(min(4, n)):
        e = nmse(single[pos:pos + 1].cpu(), want[pos:pos + 1])
        assert e <= BOUND[dtype] * 5, f"position {pos}: NMSE {e:.3e}"
    cut, at, i = [], 0, 0
    sizes = [2, 7, 2, 19, 3, 33, 2, 16, 17, 5, 64]
    while at < n:
        k = min(sizes[i % len(sizes)], n - at)
        cut.append(eng.step([StepEntry("c", toks[at:at + k], list(range(k)))]).clone())
        at, i = at + k, i + 1
    eng.synchronize()
    eng.finish("c")
    cut = torch.cat(cut)
    close(cut, want, dtype, "portions")
    if dtype == "float32":
        assert nmse(single.cpu(), whole.cpu()) <= 1e-10 and nmse(cut.cpu(), whole.cpu()) <= 1e-10
    # in bfloat16 the attention over a latent runs on the tensor-core kernel where the key row is a
    # multiple of 16 wide and the latent a multiple of 8 (a layer of A, C, D), else on CUDA cores (B)
    used = eng.info()["counters"]["shared_key_launches"]
    assert (used > 0) == (dtype == "bfloat16" and name != "B"), used
    # and prompt steps of more than 64 tokens of the differential attention on the tensor-core
    # kernel of the mixed-head attention where the head sizes are multiples of 16 (C, F)
    used = eng.info()["counters"]["mix_mma_launches"]
    assert (used > 0) == (dtype == "bfloat16" and name in ("C", "F")), used


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(name, dtype):
    """Six requests through two slots and a cache that holds two of them: portions
    of one beside decoded tokens of another; every request's logits are those of
    the request alone."""
    from kipp_b200.engine import StepEntry
    vocab = CONFIGS[name]["vocab"]
    lengths = [37, 64, 5, 90, 18, 71]
    seqs = {f"r{i}": random_tokens(vocab, n, seed=20 + i) for i, n in enumerate(lengths)}
    eng = engine_for(name, dtype, cache_tokens=256, max_requests=2, max_batch_tokens=256)
    waiting, live, got = list(seqs), {}, {r: [] for r in seqs}
    tick = 0
    while waiting or live:
        while waiting and len(live) < 2:
            live[waiting.pop(0)] = 0
        entries = []
        for j, (rid, at) in enumerate(live.items()):
            toks = seqs[rid]
            head = max(len(toks) - 9, 1)
            k = 1 if at >= head else min([13, 2, 30, 5][(tick + j) % 4], head - at)
            entries.append(StepEntry(rid, toks[at:at + k], list(range(k))))
        logits = eng.step(entries, check=True)
        row = 0
        for e in entries:
            k = len(e.tokens)
            got[e.request].append(logits[row:row + k].clone())
            row += k
            live[e.request] += k
            if live[e.request] == len(seqs[e.request]):
                eng.finish(e.request)
                del live[e.request]
        eng.cache.check()
        tick += 1
    for rid, toks in seqs.items():
        close(torch.cat(got[rid]), plain_logits(name, dtype, toks), dtype, rid)
    info = eng.info()
    assert info["free_slots"] == 2 and all(g["free_pages"] == g["pages"] for g in info["cache_groups"])


# ------------------------------------------------------------------ edges, made to show
def needle_config(kind, window=0):
    """One layer whose attention is sharp (a large score scale), so that a key
    wrongly seen or wrongly dropped moves the logits far more than rounding."""
    layer = (diff_layer(3, 1, 16, 8, window, 8, None, diff=0.35, scale=4.0) if kind == "attention"
             else latent_layer(3, 8, 8, 8, 16, 12, None, scale=4.0))
    return {"architecture": "Varunex", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "layers": [layer]}


# In bfloat16 the sharp scores that make a wrong key show also magnify the rounding of q and k (and
# the difference of two maps magnifies it once more): four times the bound for a sequence, ten
# times for a single row.  What a wrong key does must still stand far above that.
SHARP = {"float32": 1.0, "bfloat16": 4.0}


def positions_alone(got, want, positions, dtype):
    bound = BOUND[dtype] * (10 if dtype == "bfloat16" else 1)
    for pos in sorted(set(positions) & set(range(len(want)))):
        e = nmse(got[pos:pos + 1].cpu(), want[pos:pos + 1])
        assert e <= bound, f"position {pos}: NMSE {e:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [16, 17, 32, 33, 5, 1, 30])
def test_keys_just_inside_and_outside_the_window(window, dtype, tmp_path):
    from kipp_b200.engine import Engine, StepEntry
    cfg = needle_config("attention", window)
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=window * 100, sigma=0.3, norm_jitter=0.1))
    w = rounded(read_weights(folder), dtype)
    toks = random_tokens(97, 120, seed=window)
    with torch.no_grad():
        want = P.forward(cfg, w, toks)
        # the oracle itself tells a window that is one token off from the right one
        off = needle_config("attention", window + 1)
        assert nmse(P.forward(off, w, toks)[window + 1:], want[window + 1:]) > 3 * SHARP[dtype] * BOUND[dtype]
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=256, max_requests=2, max_batch_tokens=256)
    whole = eng.step([StepEntry("w", toks, list(range(120)))], check=True).clone()
    close(whole, want, dtype, "prompt", SHARP[dtype])
    # the same positions decoded one by one after a prompt portion that ends inside the first page
    first = eng.step([StepEntry("d", toks[:11], list(range(11)))]).clone()
    rows = torch.cat([first] + [eng.step([StepEntry("d", [t], [0])]).clone() for t in toks[11:]])
    eng.synchronize()
    close(rows, want, dtype, "decoded", SHARP[dtype])
    edges = {window - 1, window, window + 1, 2 * window - 1, 2 * window, 15, 16, 17, 119}
    positions_alone(rows, want, edges, dtype)
    positions_alone(whole, want, edges, dtype)
    # a window group gives its pages back as the window passes them
    assert eng.info()["cache_groups"][0]["window"] == window


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_across_many_pages(dtype, tmp_path):
    """Sharp attention over a cached latent: a query's weight sits on a few keys
    anywhere in a long past, so a key lost at a page border or in a run of keys
    shows."""
    from kipp_b200.engine import Engine, StepEntry
    cfg = needle_config("latent_attention")
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=77, sigma=0.3, norm_jitter=0.1),
                          override=lambda name, t: 4.0 * t if name.endswith("mix.o") else None)
    w = rounded(read_weights(folder), dtype)
    n = 330
    toks = random_tokens(97, n, seed=5)
    with torch.no_grad():
        want = P.forward(cfg, w, toks)
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=1024, max_requests=2, max_batch_tokens=512)
    whole = eng.step([StepEntry("w", toks, list(range(n)))], check=True).clone()
    close(whole, want, dtype, "prompt", SHARP[dtype])
    head = eng.step([StepEntry("d", toks[:259], list(range(259)))]).clone()
    rows = torch.cat([head] + [eng.step([StepEntry("d", [t], [0])]).clone() for t in toks[259:]])
    eng.synchronize()
    close(rows, want, dtype, "decoded", SHARP[dtype])
    positions_alone(rows, want, {0, 1, 2, 255, 256, 257, 258, 259, 260, 271, 272, 273, 319, 320, 321, n - 1}, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_counts_once_in_prompts_and_in_decoding(dtype, tmp_path):
    """Scores of ordinary size beside one head's large sink, one far below every
    score and one in between: leaving the sinks out, or counting them once per
    run of keys, would move the logits far beyond rounding."""
    from kipp_b200.engine import Engine, StepEntry
    cfg = {"architecture": "Varunex", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
           "layers": [latent_layer(3, 8, 8, 8, 16, 12, None)]}

    def sinks(name, t):
        if name.endswith("mix.sink"):
            return torch.tensor([5.0, -30.0, 1.0])
        return 4.0 * t if name.endswith("mix.o") else None

    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=78, sigma=0.3, norm_jitter=0.1), override=sinks)
    w = rounded(read_weights(folder), dtype)
    n = 200
    toks = random_tokens(97, n, seed=6)
    with torch.no_grad():
        want = P.forward(cfg, w, toks)
        gone = {k: (v - 40.0 if k.endswith("mix.sink") else v) for k, v in w.items()}
        assert nmse(P.forward(cfg, gone, toks), want) > 10 * BOUND[dtype]
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=512, max_requests=2, max_batch_tokens=512)
    whole = eng.step([StepEntry("w", toks, list(range(n)))], check=True).clone()
    close(whole, want, dtype, "prompt")
    # few tokens at a time: their keys are walked in runs that are merged, the sink joins after
    head = eng.step([StepEntry("d", toks[:3], list(range(3)))]).clone()
    rows = torch.cat([head] + [eng.step([StepEntry("d", [t], [0])]).clone() for t in toks[3:]])
    eng.synchronize()
    close(rows, want, dtype, "decoded")
    positions_alone(rows, want, {0, 1, 2, 3, 63, 64, 65, 127, 128, 129, n - 1}, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_of_a_batch_through_graphs(dtype):
    """Two requests of unequal length decoded together for 150 steps (the steps are
    graph replays after the first); the state and the window move with every token."""
    from kipp_b200.engine import StepEntry
    name = "A"
    vocab = CONFIGS[name]["vocab"]
    a, b = random_tokens(vocab, 170, seed=41), random_tokens(vocab, 155, seed=42)
    eng = engine_for(name, dtype)
    eng.step([StepEntry("a", a[:20], []), StepEntry("b", b[:5], [])])
    got_a, got_b = [], []
    for i in range(150):
        logits = eng.step([StepEntry("a", [a[20 + i]], [0]), StepEntry("b", [b[5 + i]], [0])])
        got_a.append(logits[0:1].clone())
        got_b.append(logits[1:2].clone())
    eng.synchronize()
    assert eng.graph_replays > 100
    close(torch.cat(got_a), plain_logits(name, dtype, a)[20:], dtype, "a")
    close(torch.cat(got_b), plain_logits(name, dtype, b)[5:], dtype, "b")


def test_greedy_generation_through_the_scheduler():
    from kipp_b200.engine.llm import LLM
    name = "A"
    vocab = CONFIGS[name]["vocab"]
    prompts = [random_tokens(vocab, n, seed=60 + n) for n in (3, 41, 17)]
    llm = LLM(model_folder(name), dtype="float32", kv_tokens=512, max_requests=4, max_batch_tokens=64, chunk=16)
    out = llm.generate(prompts, decode=12)
    w = weights_for(name, "float32")
    for prompt, result in zip(prompts, out):
        seq = list(prompt)
        with torch.no_grad():
            for _ in range(12):
                seq.append(int(P.forward(CONFIGS[name], w, seq)[-1].argmax()))
        assert result.tokens == seq[len(prompt):]


def test_command_line_with_greedy_and_sampled_generation():
    """bin/kipp on a model folder (two prompts of unequal length beside one another, greedy: the
    plain model's continuation) and on the preset with random weights and sampling."""
    name = "D"
    vocab = CONFIGS[name]["vocab"]
    a, b = random_tokens(vocab, 9, seed=5), random_tokens(vocab, 27, seed=6)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kipp"), "--model", model_folder(name),
                           "--prompt-ids", ",".join(map(str, a)), "--prompt-ids", ",".join(map(str, b)),
                           "--decode", "5", "--dtype", "float32", "--chunk", "16", "--top", "0"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [[int(t) for t in line.split("\t")[1].split()] for line in proc.stdout.strip().splitlines()]
    w = weights_for(name, "float32")
    for prompt, tokens in zip((a, b), got):
        seq = list(prompt)
        with torch.no_grad():
            for _ in range(5):
                seq.append(int(P.forward(CONFIGS[name], w, seq)[-1].argmax()))
        assert tokens == seq[len(prompt):]
    assert "prefill_tokens=36" in proc.stderr and "decode_tokens=10" in proc.stderr
    sampled = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kipp"), "--random", "varunex-tiny",
                              "--prompt-ids", "1,2,3,4,5", "--decode", "8", "--temperature", "0.8", "--top-k", "20",
                              "--seed", "3", "--top", "0"], capture_output=True, text=True, timeout=600)
    assert sampled.returncode == 0, sampled.stderr[-2000:]
    tokens = [int(t) for t in sampled.stdout.strip().splitlines()[0].split("\t")[1].split()]
    assert len(tokens) == 8 and all(0 <= t < 384 for t in tokens)


def test_the_trace_program_runs_the_model_step_by_step(tmp_path):
    name = "B"
    toks = random_tokens(CONFIGS[name]["vocab"], 50, seed=77)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[30:49], "want": []},
                                     {"id": "y", "tokens": toks[:2], "want": [1]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[49:], "want": [0]}], "end": ["x"]}]
    out = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folder(name),
                           "--dtype", "float32", "--out", out, "--max-tokens", "128"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = plain_logits(name, "float32", toks)
    got = torch.cat([torch.frombuffer(bytearray(open(os.path.join(out, f"{s}.f32"), "rb").read()), dtype=torch.float32)
                     .view(-1, CONFIGS[name]["vocab"]) for s in (0, 2)])
    assert nmse(got, want[[0, 29, 49]]) <= BOUND["float32"]
