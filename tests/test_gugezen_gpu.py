"""Gugezen through the engine on the GPU against the plain whole-sequence model: the same requests whole, with their
last tokens decoded one by one, in portions down to two tokens, and mixed with other requests in a pool so small that
pages and state slots are used again; in 32-bit and in bfloat16; captured steps; greedy generation through the public
entry points and the scheduler; ``bin/trace_run`` and the command line as a user starts them."""

from __future__ import annotations

import functools
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import gugezen_tiny as pt
from tests import plain_gugezen as plain
from tests import schedules

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = {"A": [5, 18, 34, 70, 41, 64], "B": [1, 9, 40, 70, 97, 33], "C": [2, 129, 201, 70, 257, 64], "D": [4, 40, 22, 70, 33, 8]}
F32_REL = 3e-5          # of the largest expected logit of the request
BF16_REL = 3e-2


def requests_for(name, folder):
    cfg, _ = plain.read_folder(folder)
    return {f"r{i}": pt.random_ids(n, cfg["vocab"], 100 + i) for i, n in enumerate(LENGTHS[name])}


@functools.lru_cache(maxsize=None)
def _expected(name, tokens):
    """(the folder's weights depend on the name alone)"""
    import tempfile
    cfg, w = plain.read_folder(pt.make_tiny_folder(name, tempfile.mkdtemp()))
    return plain.forward(cfg, w, list(tokens))[0].numpy()


def expected_logits(name, reqs):
    return {rid: _expected(name, tuple(toks)) for rid, toks in reqs.items()}


def check(got, expected, dtype):
    """float32: every logit within F32_REL of the request's largest.  bfloat16 (against the 64-bit plain model): the
    root mean square of a position's differences within BF16_REL of the request's largest logit, and no single logit
    further off than twice that."""
    for rid, rows in got.items():
        top = float(np.abs(expected[rid]).max())
        for pos in sorted(rows):
            diff = rows[pos] - expected[rid][pos]
            if dtype == "float32":
                err, bound = float(np.abs(diff).max()), F32_REL * top
            else:
                err, bound = max(float(np.sqrt((diff ** 2).mean())), 0.5 * float(np.abs(diff).max())), BF16_REL * top
            assert err <= bound, f"first wrong place (request, position, error / bound): {(rid, pos, err / bound)}"


def replay(folder, name, steps, dtype, graphs=(), portions=(), page=None):
    from turingserve_b200 import kernels
    from turingserve_b200.engine.replay import Replayer
    kernels.use(None)
    rp = Replayer(folder, getattr(torch, dtype), schedules.peak_tokens(steps), "cuda", page_size=page or pt.page_size(name),
                  graph_batch_sizes=graphs, graph_portion_sizes=portions)
    outs = {}
    with torch.inference_mode():
        for s in steps:
            o = rp.step(s)
            if o is not None:
                outs[s["step"]] = o
            rp.cache.check()
    assert not rp.cache.live
    return schedules.collect(steps, outs), rp


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("schedule", ["whole", "decode_tail", "portions", "mixed"])
def test_schedules_match_plain(tmp_path, name, schedule, dtype):
    folder = pt.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    steps = getattr(schedules, schedule)(reqs)
    got, _ = replay(folder, name, steps, dtype)
    assert sum(len(v) for v in got.values()) == sum(len(t) for t in reqs.values())
    check(got, expected_logits(name, reqs), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_captured_steps_match_plain(tmp_path, name, dtype):
    """Single-token steps replayed from captured graphs of 1, 2 and 4 rows (3 live requests: a padding row that points at
    the null page and the null state slot), and steps of decoding requests beside one 16-token portion from graphs of
    (rows, portion): positions, slots and block tables all come from device arrays, so one capture serves every later
    step of its shape."""
    folder = pt.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    expected = expected_logits(name, reqs)
    got, rp = replay(folder, name, schedules.batched_tail(reqs), dtype, graphs=(1, 2, 4))
    assert rp.runner._graphs, "no step was captured"
    check(got, expected, dtype)
    got, rp = replay(folder, name, schedules.served(reqs), dtype, graphs=(1, 2, 4), portions=(16,))
    assert any(k[1] == 16 for k in rp.runner._graphs), "no step with a portion was captured"
    check(got, expected, dtype)


def test_results_do_not_depend_on_batch_mates_pages_or_slots(tmp_path):
    """float32: a request alone in a fresh pool and the same request among others in a small pool with other page sizes
    and handed-on state slots give the same logits to the last bits that the order of sums leaves."""
    folder = pt.make_tiny_folder("A", tmp_path)
    reqs = requests_for("A", folder)
    alone, _ = replay(folder, "A", schedules.whole(reqs), "float32", page=64)
    among, _ = replay(folder, "A", schedules.mixed(reqs, seed=3), "float32", page=8)
    for rid in reqs:
        for pos, row in alone[rid].items():
            assert float(np.abs(row - among[rid][pos]).max()) <= 2e-5 * float(np.abs(row).max()), (rid, pos)


def test_long_decoding(tmp_path):
    """A prompt of 20 tokens, then 300 tokens one by one: states carried over hundreds of single steps, keys hundreds of
    tokens back over many pages."""
    for name in ("A", "B", "C"):
        folder = pt.make_tiny_folder(name, tmp_path)
        cfg, _ = plain.read_folder(folder)
        reqs = {"long": pt.random_ids(320, cfg["vocab"], 7)}
        got, _ = replay(folder, name, schedules.decode_tail(reqs, tail=300), "float32", page={"A": 8, "B": 4, "C": 16}[name])
        check(got, expected_logits(name, reqs), "float32")


def engine(folder, dtype="float32", **kw):
    from turingserve_b200 import EngineConfig, LLMEngine, kernels
    kernels.use(None)
    opts = dict(num_blocks=200, max_num_seqs=8, max_num_batched_tokens=64, block_size=16, max_model_len=512)
    opts.update(kw)
    return LLMEngine.from_config(EngineConfig(model=folder, dtype=dtype, **opts))


def greedy(n):
    from turingserve_b200 import SamplingParams
    return SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)


def tokens_are_best(cfg, w, prompt, tokens, slack):
    ids = list(prompt)
    for tok in tokens:
        lg = plain.forward(cfg, w, ids)[0][-1]
        assert lg[tok] >= lg.max() - slack * lg.abs().max(), (len(ids), tok, int(lg.argmax()))
        ids.append(tok)


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_greedy_generation_float32_equals_plain(tmp_path, name):
    """Through LLMEngine.generate: the scheduler cuts the prompts into portions of at most 24 tokens beside the decoding
    requests; more requests than fit at once."""
    folder = pt.make_tiny_folder(name, tmp_path)
    cfg, w = plain.read_folder(folder)
    prompts = [pt.random_ids(n, cfg["vocab"], 20 + n) for n in (5, 17, 33, 1, 50)]
    eng = engine(folder, block_size=pt.page_size(name), max_num_batched_tokens=24, max_num_seqs=3)
    outs = eng.generate(prompts, greedy(8))
    for p, o in zip(prompts, outs):
        tokens_are_best(cfg, w, p, o.token_ids, 2e-5)
        assert o.finish_reason == "length" and len(o.token_ids) == 8 and o.prompt_tokens == len(p)
    assert not eng.cache.live and (not eng.cache.groups or eng.cache.min_free() == eng.cache.num_pages - 1)


def test_entry_point_and_long_decoding_from_the_first_token(tmp_path):
    """generate_greedy from a one-token prompt: 150 tokens decoded one by one through captured graphs, every one the plain
    model's choice (the first tokens of a sequence, then state and keys growing token by token)."""
    from turingserve_b200 import generate_greedy
    folder = pt.make_tiny_folder("B", tmp_path)
    cfg, w = plain.read_folder(folder)
    toks = generate_greedy(folder, [7], 150, dtype="float32", num_blocks=80, max_num_seqs=2, block_size=8, max_model_len=256)
    assert len(toks) == 150
    tokens_are_best(cfg, w, [7], toks, 2e-5)


def test_graphs_look_ahead_and_preemption_do_not_change_tokens(tmp_path):
    """bfloat16: graphs on or off, the next step launched ahead or not, and a pool so small that requests are preempted
    and recomputed (their state slots zeroed again): the same tokens."""
    from turingserve_b200 import SamplingParams
    folder = pt.make_tiny_folder("A", tmp_path)
    cfg, _ = plain.read_folder(folder)
    prompts = [pt.random_ids(n, cfg["vocab"], 40 + n) for n in (7, 21, 2, 50, 11, 33, 5)]
    params = [SamplingParams(temperature=0.0, max_tokens=m, ignore_eos=True) for m in (20, 3, 31, 9, 14, 1, 26)]
    runs = {}
    for graphs, ahead, pages in ((False, False, 200), (True, True, 200), (True, False, 200), (False, True, 200), (True, True, 14)):
        eng = engine(folder, "bfloat16", cuda_graphs=graphs, async_decode=ahead, block_size=8, max_num_seqs=8,
                     graph_batch_sizes=(1, 2, 4, 8), max_num_batched_tokens=32, num_blocks=pages)
        runs[(graphs, ahead, pages)] = [o.token_ids for o in eng.generate(prompts, params)]
        assert not eng.cache.live
    base = runs[(False, False, 200)]
    assert [len(t) for t in base] == [20, 3, 31, 9, 14, 1, 26]
    for key, got in runs.items():
        assert got == base, key


def test_trace_run_as_a_subprocess(tmp_path):
    folder = pt.make_tiny_folder("B", tmp_path)
    reqs = requests_for("B", folder)
    steps = schedules.mixed(reqs, seed=5)
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(schedules.peak_tokens(steps)), "--block-size", "16"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    cfg, _ = plain.read_folder(folder)
    outs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"]) for s in steps
            if any(e["want"] for e in s["entries"])}
    check(schedules.collect(steps, outs), expected_logits("B", reqs), "float32")


def test_command_line_generates_the_plain_models_tokens(tmp_path):
    """``python -m turingserve_b200.cli generate`` on a Gugezen folder: config.json alone chooses the model class."""
    folder = pt.make_tiny_folder("A", tmp_path)
    cfg, w = plain.read_folder(folder)
    prompt = pt.random_ids(6, cfg["vocab"], 12)
    r = subprocess.run([sys.executable, "-m", "turingserve_b200.cli", "generate", "--model", folder, "--dtype", "float32",
                        "--num-blocks", "32", "--max-num-seqs", "2", "--max-model-len", "128", "--prompt-ids",
                        ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0", "--ignore-eos"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    tokens_are_best(cfg, w, prompt, json.loads(r.stdout.strip().splitlines()[-1])["token_ids"], 2e-5)
