"""Venizen on the GPU against the plain float64 model (plain_venizen.py): each
mechanism alone; whole prompts; token-by-token decoding from the first token;
portions down to two tokens; batches of unequal requests; pages and slots used
again; keys at the edges of windows, of the kept first tokens and of pages;
long decoding through graphs; greedy generation through the scheduler; the
trace program."""
import json
import os
import subprocess
import sys
import tempfile

import pytest
import torch

import plain_venizen as P
from tiny import nmse, read_weights
from venizen_util import CONFIGS, INIT, model_folder, random_tokens, write_folder

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# float32: the engine against the float64 plain model.  bfloat16: against the plain model with
# the matrices rounded to bfloat16 (activations are not rounded there, so the bound is that of
# 16-bit activations through a few layers).
BOUND = {"float32": 1e-9, "bfloat16": 2e-3}


def weights_for(name, dtype):
    w = read_weights(model_folder(name))
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    return w


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


def close(got, want, dtype, what=""):
    e = nmse(got.cpu(), want)
    assert e <= BOUND[dtype], f"{what}: NMSE {e:.3e} > {BOUND[dtype]:.1e}"


# ------------------------------------------------------------------ each mechanism alone
def _mechanism_inputs(name, T, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, CONFIGS[name]["width"], generator=g, dtype=torch.float64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [("P", 1), ("P", 2), ("Q", 0), ("Q", 3), ("R", 0), ("R", 2)])
def test_attention_and_retention_branches_alone(name, layer, dtype):
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    run = [o["layer"] for o in eng.spec.plan["order"]].index(layer)
    T = 75
    h = _mechanism_inputs(name, T, 100 + layer)
    h_dev = h.to("cuda", eng.dtype).contiguous()
    h_ref = h_dev.double().cpu()
    w = {k: v.double() for k, v in weights_for(name, dtype).items()}
    mx, eps, p = cfg["layers"][layer]["mixer"], cfg["norm"]["eps"], f"l{layer}.mix."
    for branch, fn, scale in ((0, P.mixed_head_attention, mx["left_scale"]), (1, P.retention, mx["right_scale"])):
        side = "left" if branch == 0 else "right"
        want = scale * fn(w, p + side + ".", mx[side], h_ref, eps)
        out = torch.zeros(T, cfg["width"], device="cuda")
        # in two portions: the second reads the cache or the state the first left
        eng.run_part([StepEntry(f"b{branch}", [0] * 40, [])], run, f"mixer/{branch}", input=h_dev[:40].contiguous(),
                     residual=out[:40])
        eng.run_part([StepEntry(f"b{branch}", [0] * 35, [])], run, f"mixer/{branch}", input=h_dev[40:].contiguous(),
                     residual=out[40:])
        close(out, want, dtype, f"{name} layer {layer} {side}")
        eng.finish(f"b{branch}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [("P", 0), ("Q", 1), ("Q", 2), ("R", 1), ("R", 3)])
def test_delta_rule_alone(name, layer, dtype):
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    run = [o["layer"] for o in eng.spec.plan["order"]].index(layer)
    T = 60
    h_dev = _mechanism_inputs(name, T, 200 + layer).to("cuda", eng.dtype).contiguous()
    w = {k: v.double() for k, v in weights_for(name, dtype).items()}
    want = P.delta_rule(w, f"l{layer}.mix.", cfg["layers"][layer]["mixer"], h_dev.double().cpu(), cfg["norm"]["eps"])
    out = torch.zeros(T, cfg["width"], device="cuda")
    at = 0
    for n in (17, 1, 2, 40):
        eng.run_part([StepEntry("d", [0] * n, [])], run, "mixer", input=h_dev[at:at + n].contiguous(),
                     residual=out[at:at + n])
        at += n
    close(out, want, dtype, f"{name} layer {layer}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [("P", 2), ("Q", 2), ("R", 0)])
def test_polynorm_feed_forward_alone(name, layer, dtype):
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    run = [o["layer"] for o in eng.spec.plan["order"]].index(layer)
    T = 33
    h_dev = _mechanism_inputs(name, T, 300 + layer).to("cuda", eng.dtype).contiguous()
    w = {k: v.double() for k, v in weights_for(name, dtype).items()}
    want = P.polynorm_mlp(w, f"l{layer}.mlp.", h_dev.double().cpu(), cfg["norm"]["eps"])
    out = torch.zeros(T, cfg["width"], device="cuda")
    eng.run_part([StepEntry("f", [0] * T, [])], run, "feed_forward", input=h_dev, residual=out)
    close(out, want, dtype, f"{name} layer {layer}")


# ------------------------------------------------------------------ whole models
LENGTH = {"P": 90, "Q": 131, "R": 230, "S": 70, "T": 100}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_every_way_of_cutting_it(name, dtype):
    """Whole; token by token from the very first token; portions down to two
    tokens; most of it at once and the tail one by one: every position against
    the plain model, and (32-bit) the ways of cutting against one another."""
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
    # prompt steps of more than 64 tokens in bfloat16 run on the tensor-core kernel where the head
    # sizes are multiples of 16 (R: every attention layer; S: none), the others on CUDA cores
    used = eng.info()["counters"]["mix_mma_launches"]
    assert (used > 0) == (dtype == "bfloat16" and name != "S"), used


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
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
def needle_config(window, keep_first, page_aligned_dim=16):
    """One parallel layer whose attention is sharp (a large score scale), so that a
    key wrongly seen or wrongly dropped moves the logits far more than rounding."""
    from venizen_util import attention, parallel_layer, retention
    return {"architecture": "Venizen", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
            "layers": [parallel_layer(attention(3, 1, page_aligned_dim, 8, window, keep_first, 8, scale=6.0),
                                      retention(1, 8, 8, [0.5], 0), None, left_scale=2.0, right_scale=0.1)],
            "loop": {"start": 0, "stop": 0, "times": 1}}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,keep_first", [(16, 0), (17, 1), (32, 16), (33, 5), (5, 20), (1, 2), (30, 29)])
def test_keys_just_inside_and_outside_the_window_and_the_kept_tokens(window, keep_first, dtype, tmp_path):
    from kipp_b200.engine import Engine, StepEntry
    cfg = needle_config(window, keep_first)
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=window * 100 + keep_first, sigma=0.3, norm_jitter=0.1))
    w = read_weights(folder)
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    toks = random_tokens(97, 120, seed=window)
    with torch.no_grad():
        want = P.forward(cfg, w, toks)
        # the oracle itself tells a window that is one token off from the right one
        off = needle_config(window + 1, keep_first)
        assert nmse(P.forward(off, w, toks)[window + 1:], want[window + 1:]) > 3 * BOUND[dtype]
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=256, max_requests=2,
                             max_batch_tokens=256)
    whole = eng.step([StepEntry("w", toks, list(range(120)))], check=True).clone()
    close(whole, want, dtype, "prompt")
    # the same positions decoded one by one after a prompt portion that ends inside the first page
    first = eng.step([StepEntry("d", toks[:11], list(range(11)))]).clone()
    rows = [first] + [eng.step([StepEntry("d", [t], [0])]).clone() for t in toks[11:]]
    eng.synchronize()
    close(torch.cat(rows), want, dtype, "decoded")
    # each position on its own: the edges are single rows.  (In bfloat16 the sharp scores that make
    # a wrong key show also magnify the rounding of q and k: ten times the bound for a single row.)
    row_bound = BOUND[dtype] * (10 if dtype == "bfloat16" else 1)
    for pos in {window - 1, window, window + 1, keep_first + window - 1, keep_first + window, 15, 16, 17, 119} & set(range(120)):
        e = nmse(torch.cat(rows)[pos:pos + 1].cpu(), want[pos:pos + 1])
        assert e <= row_bound, f"position {pos}: NMSE {e:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_of_a_batch_through_graphs(dtype):
    """Two requests of unequal length decoded together for 150 steps (the steps are
    graph replays after the first); the state and the window move with every token."""
    from kipp_b200.engine import StepEntry
    name = "Q"
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
    name = "P"
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


def test_the_trace_program_runs_the_model_step_by_step(tmp_path):
    name = "Q"
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
    import numpy as np
    want = plain_logits(name, "float32", toks)
    vocab = CONFIGS[name]["vocab"]
    s0 = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(-1, vocab))
    s1 = torch.from_numpy(np.fromfile(os.path.join(out, "1.f32"), dtype="<f4").reshape(-1, vocab))
    s2 = torch.from_numpy(np.fromfile(os.path.join(out, "2.f32"), dtype="<f4").reshape(-1, vocab))
    close(s0, want[[0, 29]], "float32", "step 0")
    close(s1, want[[1]], "float32", "step 1")
    close(s2, want[[49]], "float32", "step 2")
