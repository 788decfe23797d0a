#!/usr/bin/env python3
"""Benchmark: decode tokens/s (default batch 8), prefill tokens/s at 2,048 tokens and roofline
fractions for a Qwen2.5-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--model qwen2.5-1.5b|qwen2.5-7b|qwen2.5-14b] [--batch 8] [--kv-block 16] [--phases ...]

One JSON line.  Beside the contract's keys: ``prefill``, ``roofline`` (the whole decode step against
the copy bandwidth), ``points`` (batch 1 and 64, and the headline batch with pages of 64 tokens),
``kernels`` (each dominant kernel alone against its roofline), ``graph_check`` (the captured decode
step against the same step launched kernel by kernel) and ``mixed`` (the Qwen2.5-14B shape with 32
decodes beside a 2,048-token prompt in portions of 512).

A "step" is one decode step of the whole batch.  ``value`` times K decode steps of the engine's
step function with CUDA events (inputs built on the host, copied to the device each step);
``e2e`` times the same through ``LLMEngine.step`` (scheduler, step function, sampler; host tokens
in, sampled tokens out).  The method follows the reference's micro benchmark
(benchmarks/micro/decode_speed.py:42-64: warm-up steps dropped, speed of light = bandwidth /
bytes per step), on synthetic uniform token ids and N(0, 0.02) weights.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE configs[2]: Qwen2.5-1.5B shape
SHAPES = {
    "qwen2.5-0.5b": dict(hidden_size=896, intermediate_size=4864, num_layers=24, num_heads=14, num_kv_heads=2,
                         head_dim=64, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                         tie_word_embeddings=True, max_position_embeddings=32768),
    "qwen2.5-1.5b": dict(hidden_size=1536, intermediate_size=8960, num_layers=28, num_heads=12, num_kv_heads=2,
                         head_dim=128, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                         tie_word_embeddings=True, max_position_embeddings=32768),
    "qwen2.5-3b": dict(hidden_size=2048, intermediate_size=11008, num_layers=36, num_heads=16, num_kv_heads=2,
                       head_dim=128, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                       tie_word_embeddings=True, max_position_embeddings=32768),
    "qwen2.5-7b": dict(hidden_size=3584, intermediate_size=18944, num_layers=28, num_heads=28, num_kv_heads=4,
                       head_dim=128, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6,
                       tie_word_embeddings=False, max_position_embeddings=32768),
    "qwen2.5-14b": dict(hidden_size=5120, intermediate_size=13824, num_layers=48, num_heads=40, num_kv_heads=8,
                        head_dim=128, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6,
                        tie_word_embeddings=False, max_position_embeddings=32768),
    "qwen2.5-32b": dict(hidden_size=5120, intermediate_size=27648, num_layers=64, num_heads=40, num_kv_heads=8,
                        head_dim=128, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-5,
                        tie_word_embeddings=False, max_position_embeddings=32768),
}
SHAPE_NAMES = {"qwen2.5-0.5b": "Qwen2.5-0.5B", "qwen2.5-1.5b": "Qwen2.5-1.5B", "qwen2.5-3b": "Qwen2.5-3B",
               "qwen2.5-7b": "Qwen2.5-7B", "qwen2.5-14b": "Qwen2.5-14B", "qwen2.5-32b": "Qwen2.5-32B"}


def metric_name(a) -> str:
    """The same words in both arms: the driver divides two lines only when their metrics read alike.
    The precision each arm computes in is in its ``dtype``."""
    return f"decode tok/s at batch {a.batch} ({SHAPE_NAMES[a.model]} shape, {a.prompt_len:,}-token prompts)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                p = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(p.get(k), (int, float)):
                    out[k] = float(p[k])
            return out, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.samples: list[list[str]] = []
        self.index = index
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                r = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                    "-i", str(self.index)], capture_output=True, text=True, timeout=5)
                if r.returncode == 0 and r.stdout.strip():
                    self.samples.append([x.strip() for x in r.stdout.strip().splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        mhz = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2:]) if v.lower().startswith("active")})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def model_numbers(kw: dict, layers: int) -> dict:
    h, I, H, KVH, D, V = (kw["hidden_size"], kw["intermediate_size"], kw["num_heads"], kw["num_kv_heads"],
                          kw["head_dim"], kw["vocab_size"])
    per_layer = h * (H + 2 * KVH) * D + (H + 2 * KVH) * D + H * D * h + 3 * h * I + 2 * h
    linear_params = layers * (h * (H + 2 * KVH) * D + H * D * h + 3 * h * I)
    head = V * h
    return dict(weight_bytes_decode=2 * (layers * per_layer + h + head),      # every weight a decode step reads
                kv_bytes_per_token=2 * layers * KVH * D * 2, linear_params=linear_params, head_params=head,
                attn_flops_per_layer=lambda T: 2.0 * T * T * D * H)             # causal: QK^T and PV, half each


def make_model(shape: str, layers: int, tmp: str) -> str:
    from turingserve_b200.models.qwen2 import make_config
    from turingserve_b200.weights.random_init import write_random_model
    kw = dict(SHAPES[shape])
    kw["num_layers"] = layers
    folder = os.path.join(tmp, f"{shape}-L{layers}")
    t0 = time.time()
    write_random_model(folder, make_config(**kw), seed=0)
    print(f"[bench] wrote random {shape} ({layers} layers) in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return folder


def build_engine_on_device(shape: str, layers: int, *, ctx_len: int, page: int, max_seqs: int, max_tokens: int,
                           graph_sizes: tuple[int, ...], model=None, portion_budget: int | None = None, mcfg=None):
    """An engine around a model whose N(0, 0.02) weights are drawn on the device (no checkpoint file:
    the 14B shape would be 30 GB of it); everything else as ``LLMEngine.from_config`` builds it."""
    import torch

    from turingserve_b200 import EngineConfig, LLMEngine
    from turingserve_b200.cache.manager import CacheManager
    from turingserve_b200.engine.runner import ModelRunner, run_needs
    from turingserve_b200.engine.scheduler import Scheduler
    from turingserve_b200.models.qwen2 import make_config
    from turingserve_b200.sampling.sampler import Sampler
    from turingserve_b200.weights.random_init import random_model_on_device

    if mcfg is None:
        kw = dict(SHAPES[shape])
        kw["num_layers"] = layers
        mcfg = make_config(**kw)
    device = torch.device("cuda", 0)
    if model is None:
        t0 = time.time()
        model = random_model_on_device(mcfg, torch.bfloat16, device, seed=0, max_positions=ctx_len)
        torch.cuda.synchronize()
        print(f"[bench] random {shape} ({layers} layers) on the device in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    cfg = EngineConfig(model=f"<random {shape}>", dtype="bfloat16", max_model_len=ctx_len, block_size=page,
                       num_blocks=max_seqs * (-(-ctx_len // page)) + 8, max_num_seqs=max_seqs,
                       max_num_batched_tokens=max_tokens, graph_batch_sizes=graph_sizes, watermark=0.0)
    if portion_budget is not None:
        cfg.graph_portion_budget = portion_budget
    cfg.validate(mcfg.max_position_embeddings)
    cache = CacheManager(run_needs(model), page, cfg.num_blocks, max_seqs, torch.bfloat16, device)
    portions = cfg.graph_portion_sizes() if graph_sizes else ()
    runner = ModelRunner(model, cache, max(max_tokens, max_seqs), max_seqs, ctx_len, cfg.graph_batch_sizes, portions)
    sched = Scheduler(cache, max_tokens, max_seqs, 0.0, runner.padded_decodes if portions else None)
    return LLMEngine(cfg, runner, cache, sched, Sampler(device), mcfg.eos_token_ids, ctx_len, mcfg.vocab_size)


def graph_check(runner, cache, rcs, tokens) -> dict:
    """One decode step replayed from its captured graph, then the same tokens at the same positions
    launched kernel by kernel (the cache is told to forget the step, whose keys and values are simply
    written again): the logits must agree to within bfloat16 rounding of a step's different split of
    the keys.  A wrong-but-finite output head or a stale graph input would show here."""
    import torch

    from turingserve_b200.engine.batch import StepEntry
    entries = [StepEntry(rc, [int(t)], [0]) for rc, t in zip(rcs, tokens)]
    with_graph = runner.step(entries).clone()
    for rc in rcs:
        rc.num_tokens -= 1
    sizes, runner.graph_batch_sizes = runner.graph_batch_sizes, ()
    try:
        without = runner.step([StepEntry(rc, [int(t)], [0]) for rc, t in zip(rcs, tokens)])
    finally:
        runner.graph_batch_sizes = sizes
    err = float((with_graph - without).abs().max())
    top = float(without.abs().max())
    rel = float((with_graph - without).norm() / without.norm())
    same = int((with_graph.argmax(-1) == without.argmax(-1)).sum())
    # The two runs split the keys differently (a captured step sizes its launch for the longest context),
    # so they differ by bfloat16 roundings carried through every layer: a few percent of the largest logit
    # at the worst of a million entries and about 3 % in the root mean square after 28 layers (some 200
    # roundings of 2^-9 each, added like a random walk).  A stale graph input or a wrong head gives
    # unrelated rows: a relative difference near 1.4.
    if not (rel <= 0.15):
        raise RuntimeError(f"the captured decode step disagrees with the same step launched kernel by kernel: "
                           f"relative difference {rel:.4g} (largest {err:.4g} against a largest logit of {top:.4g})")
    return {"rel_l2_diff": round(rel, 5), "max_abs_diff": round(err, 5), "max_logit": round(top, 3),
            "same_argmax": same, "rows": len(rcs)}


def run_ours(a) -> dict:
    import numpy as np
    import torch

    from turingserve_b200 import SamplingParams, kernels
    from turingserve_b200.engine.batch import StepEntry

    torch.cuda.set_device(0)
    ops = kernels.ops()
    pk, pk_src = peaks()
    kw = SHAPES[a.model]
    layers = a.layers or kw["num_layers"]
    nums = model_numbers(kw, layers)
    B, prompt_len, ctx_len = a.batch, a.prompt_len, a.context
    rng = np.random.default_rng(0)
    V = kw["vocab_size"]

    max_b = max(B, 64)
    ctx_len = max(ctx_len, a.prefill_tokens + 64, prompt_len + a.steps + max(3, a.warmup) + 64)
    eng = build_engine_on_device(a.model, layers, ctx_len=ctx_len, page=a.kv_block, max_seqs=max_b,
                                 max_tokens=max(2048, max_b, a.prefill_tokens), graph_sizes=(1, 8, 64, B))
    runner, cache = eng.runner, eng.cache

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---- prefill: one 2,048-token prompt in one step ------------------------------------------------
    def prefill_once(tokens):
        rc = cache.admit("prefill")
        e0, e1 = ev(), ev()
        e0.record()
        runner.step([StepEntry(rc, tokens, [len(tokens) - 1])])
        e1.record()
        torch.cuda.synchronize()
        cache.release(rc)
        return e0.elapsed_time(e1)

    phases = set(a.phases.split(","))
    prefill = None
    if "prefill" in phases:
        ptoks = rng.integers(0, V, size=a.prefill_tokens).tolist()
        for _ in range(3):
            prefill_once(ptoks)
        pms = sorted(prefill_once(ptoks) for _ in range(5))[2]
        T = a.prefill_tokens
        pflops = 2.0 * T * nums["linear_params"] + layers * nums["attn_flops_per_layer"](T) + 2.0 * nums["head_params"]
        prefill = {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                   "frac": round(pflops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                   "tflop": round(pflops / 1e12, 3)}

    # ---- decode through the step function -----------------------------------------------------------
    def decode_run(batch: int, steps: int, warmup: int):
        rcs = [cache.admit(f"d{i}") for i in range(batch)]
        for rc in rcs:                                           # prompts, one request per step
            runner.step([StepEntry(rc, rng.integers(0, V, size=prompt_len).tolist(), [])])
        toks = rng.integers(0, V, size=(warmup + steps, batch))
        if batch == B and not checks:
            checks.update(graph_check(runner, cache, rcs, rng.integers(0, V, size=batch)))
        for s in range(warmup):
            runner.step([StepEntry(rc, [int(toks[s, i])], [0]) for i, rc in enumerate(rcs)])
        torch.cuda.synchronize()
        l0 = ops.launches
        e0, e1 = ev(), ev()
        e0.record()
        for s in range(warmup, warmup + steps):
            runner.step([StepEntry(rc, [int(toks[s, i])], [0]) for i, rc in enumerate(rcs)])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = ops.launches - l0
        ctx_mid = prompt_len + warmup + steps / 2.0
        for rc in rcs:
            cache.release(rc)
        return ms, launches, ctx_mid

    steps, warmup = a.steps, max(3, a.warmup)
    checks: dict = {}
    with ClockSampler() as clocks:
        ms, launches, ctx_mid = decode_run(B, steps, warmup)
    value = B / (ms / 1e3)
    step_bytes = nums["weight_bytes_decode"] + B * ctx_mid * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms / 1e3) / 1e9
    points = {}
    if "points" in phases:
        for b in (1, 64):
            pms_, _, _ = decode_run(b, min(steps, 64), 3)
            points[f"decode_b{b}"] = round(b / (pms_ / 1e3), 1)

    # ---- end to end: LLMEngine.step with scheduler and sampler, host tokens in and out ----------------
    e2e = None
    if "e2e" in phases:
        prompts = [rng.integers(0, V, size=prompt_len).tolist() for _ in range(B)]
        params = SamplingParams(temperature=0.0, max_tokens=warmup + steps + B + 8, ignore_eos=True)
        for i, p in enumerate(prompts):
            eng.add_request(f"e{i}", p, params)
        while any(r.num_uncomputed > 1 for r in eng.requests.values()) or len(eng.scheduler.waiting):
            eng.step()
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n_tok = 0
        for _ in range(steps):
            n_tok += sum(len(o.delta_token_ids) for o in eng.step())
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        if n_tok != steps * B:
            raise RuntimeError(f"end-to-end run produced {n_tok} tokens in {steps} steps of {B} requests: a request "
                               "stopped early (bad logits?)")
        for rid in list(eng.requests):
            eng.abort(rid)
        eng.step()
        # per step: the input arena (ids, positions, request index, starts, lengths, slots, rows, slot
        # map, block tables) goes up (greedy rows need no sampler parameters); tokens and flags come back
        width = runner.max_pages
        h2d = 4 * (4 * B + (B + 1) + 3 * B + B * width)
        d2h = (2 * B + ops.STATUS_WORDS) * 4
        e2e = {"value": round(n_tok / e2e_s, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": round(1e3 * e2e_s / steps, 4)}

    kernel_points = None
    if "kernels" in phases:
        kernel_points = per_kernel(ops, kw, B, prompt_len + warmup + steps // 2, a.kv_block, a.prefill_tokens, pk)
    if "points" in phases and a.kv_block != 64:
        # the same decode step with pages of 64 tokens (one TMA box of the attention kernels a page)
        model = runner.model
        del eng, runner, cache
        torch.cuda.empty_cache()
        eng = build_engine_on_device(a.model, layers, ctx_len=ctx_len, page=64, max_seqs=B, max_tokens=max(2048, B),
                                     graph_sizes=(B,), model=model)
        runner, cache = eng.runner, eng.cache
        pms_, _, _ = decode_run(B, min(steps, 64), 3)
        points[f"decode_b{B}_page64"] = round(B / (pms_ / 1e3), 1)
    mixed = None
    if "mixed" in phases:
        del eng, runner, cache
        torch.cuda.empty_cache()
        try:
            mixed = run_mixed(a, pk)
        except Exception as e:                              # the 14B point must not take the headline down
            mixed = {"error": f"{type(e).__name__}: {str(e).splitlines()[0][:160] if str(e) else ''}"}

    return {
        "metric": metric_name(a),
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, N(0,0.02) random weights", "impl": "ours",
        "config": {"model": a.model, "layers": layers, "layers_of_model": kw["num_layers"],
                   "hidden": kw["hidden_size"], "heads": kw["num_heads"], "kv_heads": kw["num_kv_heads"],
                   "head_dim": kw["head_dim"], "intermediate": kw["intermediate_size"], "vocab": V,
                   "global_batch": B, "seq_len": ctx_len, "prompt_len": prompt_len, "new_tokens": warmup + steps,
                   "kv_block": a.kv_block, "parallelism": "single GPU", "cuda_graphs": True,
                   "l2": "inputs larger than L2 (weights %.2f GB per step)" % (nums["weight_bytes_decode"] / 1e9),
                   "peaks": pk_src},
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
        "graph_check": checks,
        "kernels": kernel_points,
        "mixed": mixed,
    }


def per_kernel(ops, kw: dict, B: int, ctx: int, page: int, prefill_tokens: int, pk: dict) -> dict:
    """Each dominant kernel alone at the step's shapes: mean time per launch with CUDA events around a
    CUDA graph of launches that rotate over enough copies of the weights (or caches) that they come from
    DRAM, the bytes (or FLOPs) the launch must move, and that rate over the measured peak (copy bandwidth;
    burst cuBLAS rate for the prompt attention, which is timed in isolation).  Inside a step the same
    kernels overlap their neighbours through programmatic dependent launch, so these times do not add up
    to the step; they say how far each is from its own roofline."""
    import torch

    from turingserve_b200 import kernels
    from turingserve_b200.engine.batch import streaming_decode

    h, I, H, KVH, D, V = (kw["hidden_size"], kw["intermediate_size"], kw["num_heads"], kw["num_kv_heads"],
                          kw["head_dim"], kw["vocab_size"])
    dev, bf = "cuda", torch.bfloat16
    out: dict = {"method": "CUDA events around a graph of rotating launches, each kernel alone"}

    def timed_graph(fn, copies: int) -> float:
        for i in range(copies):
            fn(i)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(copies):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * copies) * 1e3            # us per launch

    def record(name: str, us: float, nbytes: float = 0.0, flops: float = 0.0) -> None:
        r = {"us": round(us, 2)}
        if nbytes:
            r["GBps"] = round(nbytes / us / 1e3, 1)
            r["frac_hbm"] = round(nbytes / us / 1e3 / pk["hbm_gbs"], 4)
        if flops:
            r["TFLOPs"] = round(flops / us / 1e6, 1)
            r["frac_bf16"] = round(flops / us / 1e6 / pk["bf16_tflops"], 4)
        out[name] = r

    def weights(n: int, k: int):
        copies = max(2, int(300e6 // (n * k * 2)) + 1)
        return [torch.randn(n, k, device=dev, dtype=bf) * 0.02 for _ in range(copies)]

    x = torch.randn(B, h, device=dev, dtype=bf)
    positions = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    half = D // 2
    cos, sin = torch.ones(ctx + 8, half, device=dev), torch.zeros(ctx + 8, half, device=dev)
    slots = torch.full((B,), -1, dtype=torch.int32, device=dev)
    # K3: q/k/v product with bias, rotation and cache write (slots -1: nothing is written)
    nqkv = (H + 2 * KVH) * D
    ws, bias = weights(nqkv, h), torch.zeros(nqkv, device=dev, dtype=bf)
    qkv = torch.empty(B, nqkv, device=dev, dtype=bf)
    kc1 = torch.zeros(2, KVH, page, D, device=dev, dtype=bf)
    us = timed_graph(lambda i: ops.qkv_rope(qkv, x, ws[i % len(ws)], bias, positions, cos, sin, H, KVH, D, D, kc1, kc1,
                                            slots, page), len(ws))
    record("qkv_rope", us, nqkv * h * 2)
    del ws
    # K7, K10: output and down projections as the step runs them: a few tokens add themselves to the residual
    # rows (their K splits summed on chip), more leave partial sums for the norm kernel
    resid = torch.randn(B, h, device=dev, dtype=bf)
    for name, n, k in (("o_proj", h, H * D), ("down_proj", h, I)):
        ws = weights(n, k)
        xin = torch.randn(B, k, device=dev, dtype=bf) * 0.02
        o = torch.empty(B, n, device=dev, dtype=bf)

        def product(i):
            p = ops.linear(o, xin, ws[i % len(ws)], None, may_defer=True)
            if isinstance(p, kernels.LazyProduct) and not ops._into_residual(p, resid):
                ops._settle(p)

        record(name, timed_graph(product, len(ws)), n * k * 2)
        del ws
    # K8: gate/up product with the activation in its epilogue
    ws = weights(2 * I, h)
    act = torch.empty(B, I, device=dev, dtype=bf)
    group = 64 if I % 64 == 0 else 0
    record("gate_up_silu", timed_graph(lambda i: ops.gated_linear(act, x, ws[i % len(ws)], None, group), len(ws)), 2 * I * h * 2)
    del ws
    # K11: output head, 32-bit logits
    ws = weights(V, h)
    logits = torch.empty(B, V, device=dev, dtype=torch.float32)
    record("lm_head", timed_graph(lambda i: ops.linear(logits, x, ws[i % len(ws)], None), len(ws)), V * h * 2)
    del ws
    torch.cuda.empty_cache()

    class Step:
        pass

    def caches(batch: int, tokens: int, copies: int):
        per = -(-tokens // page)
        pages = batch * per + 1
        kv = [(torch.randn(pages, KVH, page, D, device=dev, dtype=bf), torch.randn(pages, KVH, page, D, device=dev, dtype=bf))
              for _ in range(copies)]
        table = (torch.randperm(pages - 1, device=dev).to(torch.int32) + 1).view(batch, per)
        return kv, table

    # K5: decode attention over the cache
    kv_bytes = B * (ctx + 1) * KVH * D * 2 * 2
    copies = max(2, min(28, int(300e6 // kv_bytes) + 1))
    kv, table = caches(B, ctx + 1, copies)
    st = Step()
    st.q_start = torch.arange(B + 1, dtype=torch.int32, device=dev)
    st.seq_lens = torch.full((B,), ctx + 1, dtype=torch.int32, device=dev)
    st.num_requests, st.max_q_len, st.max_seq_len, st.num_decode = B, 1, max(4096, ctx + 1), B
    st.streaming_decode = streaming_decode(B, ctx + 1)
    ao = torch.empty(B, H * D, device=dev, dtype=bf)
    record("decode_attention", timed_graph(lambda i: ops.attention(ao, qkv, kv[i % copies][0], kv[i % copies][1], table, st,
                                                                   H, KVH, D, page, D ** -0.5, None), copies), kv_bytes)
    del kv
    # K6: prompt attention, one prompt
    T = prefill_tokens
    kv, table = caches(1, T, 4)
    pq = torch.randn(T, nqkv, device=dev, dtype=bf)
    st = Step()
    st.q_start = torch.tensor([0, T], dtype=torch.int32, device=dev)
    st.seq_lens = torch.tensor([T], dtype=torch.int32, device=dev)
    st.num_requests, st.max_q_len, st.max_seq_len, st.num_decode, st.streaming_decode = 1, T, T, 0, False
    po = torch.empty(T, H * D, device=dev, dtype=bf)
    # pages shorter than a tile of 64 keys are fetched as one box where they lie one after the other
    # in the pool (a fresh pool hands them out so) and page by page where they do not
    in_order = torch.arange(1, table.numel() + 1, dtype=torch.int32, device=dev).view_as(table)
    for name, tab in (("prefill_attention", in_order), ("prefill_attention_shuffled_pages", table)):
        record(name, timed_graph(lambda i: ops.attention(po, pq, kv[i % 4][0], kv[i % 4][1], tab, st, H, KVH, D,
                                                         page, D ** -0.5, None), 4), flops=2.0 * T * T * D * H)
    return out


def run_mixed(a, pk: dict) -> dict:
    """The Qwen2.5-14B shape under a mixed step: 32 requests decode at about 2,048 tokens of context
    while a 2,048-token prompt arrives in portions of 512 (four steps a prompt).  Times the steps with
    CUDA events through the step function, and the same through ``LLMEngine.step`` with its scheduler
    (token budget 544: the decodes first, then the portion)."""
    import numpy as np
    import torch

    from turingserve_b200 import SamplingParams
    from turingserve_b200.engine.batch import StepEntry

    shape, nd, plen, chunk, ctx_len = "qwen2.5-14b", 32, 2048, 512, 4096
    kw = SHAPES[shape]
    layers = kw["num_layers"]
    V = kw["vocab_size"]
    rng = np.random.default_rng(1)
    # (steps of 32 decoding requests beside a 512-token portion are one captured graph, as in serving)
    eng = build_engine_on_device(shape, layers, ctx_len=ctx_len, page=a.kv_block, max_seqs=nd + 2, max_tokens=nd + chunk,
                                 graph_sizes=(nd,))
    runner, cache = eng.runner, eng.cache
    rcs = [cache.admit(f"d{i}") for i in range(nd)]
    for rc in rcs:
        for at in range(0, plen, chunk):
            runner.step([StepEntry(rc, rng.integers(0, V, size=chunk).tolist(), [])])

    def prompt_round(tag: str) -> float:
        rc = cache.admit(tag)
        ptoks = rng.integers(0, V, size=plen).tolist()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for at in range(0, plen, chunk):
            entries = [StepEntry(r, [int(rng.integers(0, V))], [0]) for r in rcs]
            entries.append(StepEntry(rc, ptoks[at:at + chunk], [chunk - 1] if at + chunk == plen else []))
            runner.step(entries)
        e1.record()
        torch.cuda.synchronize()
        cache.release(rc)
        return e0.elapsed_time(e1) / (plen // chunk)

    prompt_round("w0")
    prompt_round("w1")
    ms = sorted(prompt_round(f"p{i}") for i in range(3))[1]
    for rc in rcs:
        cache.release(rc)
    # the same through the engine: 32 running requests, prompts arriving one after the other
    # (while the later prompts arrive in portions the earlier requests already decode: a budget that lasts)
    params = SamplingParams(temperature=0.0, max_tokens=1024, ignore_eos=True)
    for i in range(nd):
        eng.add_request(f"e{i}", rng.integers(0, V, size=plen).tolist(), params)
    while any(r.num_uncomputed > 1 for r in eng.requests.values()) or len(eng.scheduler.waiting):
        eng.step()
    eng.add_request("x0", rng.integers(0, V, size=plen).tolist(), SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    for _ in range(4):
        eng.step()
    eng.add_request("x1", rng.integers(0, V, size=plen).tolist(), SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_tok = 0
    for _ in range(4):
        n_tok += sum(len(o.delta_token_ids) for o in eng.step())
    torch.cuda.synchronize()
    wall_ms = 1e3 * (time.perf_counter() - t0) / 4
    if n_tok < 4 * nd:
        raise RuntimeError(f"the mixed run through the engine produced {n_tok} tokens in 4 steps of {nd} decoding requests")
    for rid in list(eng.requests):
        eng.abort(rid)
    eng.step()
    nums = model_numbers(kw, layers)
    flops = 2.0 * (nd + chunk) * (nums["linear_params"] + 0) + 2.0 * (nd + 1) * nums["head_params"]
    return {"model": shape, "layers": layers, "decodes": nd, "prompt_tokens": plen, "portion": chunk,
            "ms_per_step": round(ms, 3), "tok_per_s": round((nd + chunk) / (ms / 1e3), 1),
            "e2e_ms_per_step": round(wall_ms, 3), "e2e_tokens_out": n_tok,
            "frac_bf16_products": round(flops / (ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}


class _StubTokenizer:
    """The reference's engine wants a tokenizer object; token ids go in and out, text is unused."""

    def decode(self, ids, skip_special_tokens=True):
        return ""


# ---- another design beside the flagship: Komirax (linear attention with a decaying state, two-map attention,
# dense and routed feed-forwards) at layer sizes of real models, next to Qwen2 layers of the same width --------
KOMIRAX_SIZES = {
    # width, heads, kv heads, key width per map / per linear head, value width, dense ff, experts, top, expert ff,
    # and the Qwen2 shape whose layers stand beside it
    "1.5b": dict(width=1536, heads=12, kv_heads=2, dim=64, vdim=128, ldim=128, ff=13440, experts=8, top=2, eff=2688,
                 beside="qwen2.5-1.5b"),
    "7b": dict(width=3584, heads=28, kv_heads=4, dim=64, vdim=128, ldim=128, ff=28416, experts=8, top=2, eff=7104,
               beside="qwen2.5-7b"),
}


def komirax_config(z: dict, groups: int, vocab: int):
    """``groups`` times four layers: (linear, dense), (linear, routed), (two-map attention, routed), (two-map
    attention, dense)."""
    from turingserve_b200.models.komirax import make_config
    lin = {"type": "lightning", "mixer": {"heads": z["heads"], "dim": z["ldim"], "vdim": z["vdim"],
                                          "decay": [1.0 - 2.0 ** -(2 + 6 * i / max(1, z["heads"] - 1)) for i in range(z["heads"])]}}
    att = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"],
                                          "diff": 0.5, "scale": z["dim"] ** -0.5}}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["eff"]}, "router": {"experts": z["experts"], "top": z["top"]}}
    four = [{**lin, "mlp": dense}, {**lin, "mlp": moe}, {**att, "mlp": moe}, {**att, "mlp": dense}]
    return make_config(width=z["width"], vocab=vocab, layers=four * groups, eps=1e-6)


def timed(fn, flush, reps: int = 7) -> float:
    """Median device time of ``fn`` in ms: captured once into a CUDA graph (so that the host's launch cost of a
    few-microsecond kernel is not what is timed) and replayed with the L2 flushed before every repetition
    (``flush`` writes a buffer larger than L2)."""
    import torch
    fn()                                                     # work buffers are made outside the capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    out = []
    for i in range(reps + 3):
        flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            out.append(e0.elapsed_time(e1))
    return sorted(out)[len(out) // 2]


def komirax_kernels(ops, z: dict, pk: dict, T: int, B: int, ctx: int, page: int) -> dict:
    """Each kernel of the new mechanisms alone: a portion of T tokens and B single tokens at context ``ctx``."""
    import torch
    from types import SimpleNamespace
    dev = torch.device("cuda", 0)
    big = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flush = lambda: big.fill_(1)
    H, G, D, V, LD, W = z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["ldim"], z["width"]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    out = {}
    FP32_PEAK = 148 * 128 * 2 * 1.965e9                      # FFMA lanes x 2 x the highest SM clock: nominal
    hbm = pk["hbm_gbs"] * 1e9

    # the state scan
    for name, rows, reqs in (("prefill", T, 1), ("decode", B, B)):
        proj = torch.randn(rows, 2 * H * LD + 2 * H * V, device=dev).to(torch.bfloat16)
        state = torch.zeros(reqs + 1, H, LD, V, device=dev)
        decay = torch.full((H,), 0.99, device=dev)
        o = torch.empty(rows, H * V, device=dev)
        per = rows // reqs
        step = SimpleNamespace(q_start=i32([i * per for i in range(reqs + 1)]), state_slots=i32(list(range(reqs))), num_requests=reqs)
        ms = timed(lambda: ops.lightning(o, proj, state, decay, step, H, LD, V), flush)
        flops = 5.0 * rows * H * LD * V
        byts = 2.0 * reqs * H * LD * V * 4 + rows * (2 * H * LD + H * V) * 2 + rows * H * V * 4
        out[f"state_scan_{name}"] = {"us": round(ms * 1e3, 1), "tflops_fp32": round(flops / ms / 1e9, 2),
                                     "frac_of_fp32_ffma_nominal": round(flops / (ms / 1e3) / FP32_PEAK, 3),
                                     "frac_of_hbm": round(byts / (ms / 1e3) / hbm, 3)}

    # the two-map attention
    pages = B * (-(-(ctx + 1) // page)) + -(-T // page) + 2
    kc = torch.randn(pages, G, page, 2 * D, device=dev).to(torch.bfloat16)
    vc = torch.randn(pages, G, page, V, device=dev).to(torch.bfloat16)
    width = -(-max(ctx + 1, T) // page)
    for name, reqs, per, seq in (("prefill", 1, T, T), ("decode", B, 1, ctx + 1)):
        rows = reqs * per
        proj = torch.randn(rows, H * 2 * D + G * 2 * D + G * V, device=dev).to(torch.bfloat16)
        tables = torch.zeros(reqs, width, dtype=torch.int32, device=dev)
        n = -(-seq // page)
        for r in range(reqs):
            tables[r, :n] = torch.arange(1 + r * n, 1 + (r + 1) * n, dtype=torch.int32, device=dev)
        step = SimpleNamespace(q_start=i32([i * per for i in range(reqs + 1)]), seq_lens=i32([seq] * reqs), num_requests=reqs,
                               max_q_len=per)
        o = torch.empty(rows, H * V, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.attention_diff(o, proj, kc, vc, tables, step, H, G, D, V, page, D ** -0.5, 0.4, 1e-6, 0.5), flush)
        flops = 2.0 * (2 * D + 2 * V) * H * (per * (per + 1) / 2 + per * (seq - per)) * reqs
        byts = reqs * seq * G * (2 * D + V) * 2.0
        out[f"two_map_attention_{name}"] = {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1),
                                            "frac_of_bf16": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
                                            "frac_of_hbm": round(byts / (ms / 1e3) / hbm, 3)}

    # the routed feed-forward: router + sort, the two grouped products
    E, top, ff = z["experts"], z["top"], z["eff"]
    w_up = (torch.randn(E, ff, W, device=dev) * 0.02).to(torch.bfloat16)
    w_down = (torch.randn(E, W, ff, device=dev) * 0.02).to(torch.bfloat16)
    wr = torch.randn(E, W, device=dev) * 0.05
    for name, rows in (("prefill", T), ("decode", B)):
        x = torch.randn(rows, W, device=dev).to(torch.bfloat16)
        idx = torch.empty(rows, top, dtype=torch.int32, device=dev)
        wts = torch.empty(rows, top, device=dev)
        a_ = torch.empty(rows * top, ff, dtype=torch.bfloat16, device=dev)
        y = torch.empty(rows * top, W, device=dev)
        ops.router_topk(idx, wts, x, wr, False, False)
        offsets, order, place, tiles = ops.moe_align(idx, E)
        ms_r = timed(lambda: (ops.router_topk(idx, wts, x, wr, False, False), ops.moe_align(idx, E)), flush)
        xs = torch.empty(rows * top, W, dtype=torch.bfloat16, device=dev)
        ms_g = timed(lambda: ops.moe_gather(xs, x, order, wts, top), flush)
        ms_u = timed(lambda: ops.grouped_linear(a_, xs, w_up, None, None, offsets, tiles, 1, "relu2"), flush)
        ms_d = timed(lambda: ops.grouped_linear(y, a_, w_down, None, None, offsets, tiles, 1), flush)
        flops = 2.0 * rows * top * ff * W
        used = min(E, rows * top)
        byts = used * ff * W * 2.0
        out[f"routed_ff_{name}"] = {
            "router_and_sort_us": round(ms_r * 1e3, 1), "gather_us": round(ms_g * 1e3, 1), "up_us": round(ms_u * 1e3, 1), "down_us": round(ms_d * 1e3, 1),
            "up_tflops": round(flops / ms_u / 1e9, 1), "down_tflops": round(flops / ms_d / 1e9, 1),
            "up_frac_of_bf16": round(flops / (ms_u / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
            "up_frac_of_hbm": round(byts / (ms_u / 1e3) / hbm, 3), "down_frac_of_hbm": round(byts / (ms_d / 1e3) / hbm, 3)}
    return out


# ---- Pizunex (gated delta rule, attention whose values are its keys with capped and biased scores and a window,
# latent attention) at layer sizes of real models, next to Komirax layers of the same width -----------------------
PIZUNEX_SIZES = {
    # width; attention heads, kv heads, head width, window; latent: heads, plain / rotated / value widths, latent sizes;
    # delta rule: heads, query/key heads, key and value widths; dense ff (squared ReLU, no gate)
    "1.5b": dict(width=1536, heads=12, kv_heads=2, dim=128, window=1024, lheads=12, nope=128, rope=64, lvdim=128, q_rank=768,
                 kv_rank=512, dheads=12, dkv=6, ddim=128, dvdim=128, ff=13440, beside="1.5b"),
    "7b": dict(width=3584, heads=28, kv_heads=4, dim=128, window=1024, lheads=28, nope=128, rope=64, lvdim=128, q_rank=1536,
               kv_rank=512, dheads=28, dkv=14, ddim=128, dvdim=128, ff=28416, beside="7b"),
}


def pizunex_config(z: dict, groups: int, vocab: int):
    """``groups`` times four layers: (attention, dense), (latent attention, dense), (delta rule, none), (delta rule, dense)."""
    from turingserve_b200.models.pizunex import make_config
    att = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                                          "scale": z["dim"] ** -0.5, "softcap": 30.0, "mask": {"size": z["window"]},
                                          "q_temp": {"coef": 0.1, "every": 128}}}
    lat = {"type": "latent_attention",
           "mixer": {"heads": z["lheads"], "dim": z["nope"], "rot_dim": z["rope"], "vdim": z["lvdim"], "q_rank": z["q_rank"],
                     "kv_rank": z["kv_rank"], "scale": (z["nope"] + z["rope"]) ** -0.5,
                     "rot": {"base": 10000.0, "dims": z["rope"],
                             "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}}
    dlt = {"type": "delta", "mixer": {"heads": z["dheads"], "kv_heads": z["dkv"], "dim": z["ddim"], "vdim": z["dvdim"], "conv": 4}}
    dense = {"kind": "dense", "ff": z["ff"]}
    four = [{**att, "mlp": dense}, {**lat, "mlp": dense}, {**dlt, "mlp": None}, {**dlt, "mlp": dense}]
    return make_config(width=z["width"], vocab=vocab, layers=four * groups, eps=1e-6)


def pizunex_kernels(ops, z: dict, pk: dict, T: int, B: int, ctx: int, page: int) -> dict:
    """Each kernel of the new mechanisms alone: a portion of T tokens and B single tokens at context ``ctx``."""
    import torch
    from types import SimpleNamespace
    dev = torch.device("cuda", 0)
    big = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flush = lambda: big.fill_(1)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    out = {}
    FP32_PEAK = 148 * 128 * 2 * 1.965e9                      # FFMA lanes x 2 x the highest SM clock: nominal
    hbm = pk["hbm_gbs"] * 1e9
    bf = torch.bfloat16

    # the delta rule: prepare (filter, unit length, gates) and the scan
    H, G, D, V, taps = z["dheads"], z["dkv"], z["ddim"], z["dvdim"], 4
    C = 2 * G * D + H * V
    for name, rows, reqs in (("prefill", T, 1), ("decode", B, B)):
        per = rows // reqs
        proj = torch.randn(rows, C + H * V + 2 * H, device=dev).to(bf)
        conv_w = torch.randn(C, taps, device=dev) * 0.5
        a_log, dt = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
        state = torch.zeros(reqs + 1, H * D * V + (taps - 1) * C, device=dev)
        ready = torch.empty(rows, C + 2 * H + G, device=dev)
        o = torch.empty(rows, H * V, device=dev)
        step = SimpleNamespace(q_start=i32([i * per for i in range(reqs + 1)]), state_slots=i32(list(range(reqs))),
                               num_requests=reqs, token_request=i32([r for r in range(reqs) for _ in range(per)]), max_q_len=per)
        ms_p = timed(lambda: ops.delta_prepare(ready, proj, conv_w, a_log, dt, state, step, H, G, D, V, taps, 1e-6), flush)
        ms = timed(lambda: ops.delta_scan(o, ready, proj, state, step, H, G, D, V, taps), flush)
        flops = 8.0 * rows * H * D * V                       # two sums, the decay and the write, 2 operations each
        byts = 2.0 * reqs * H * D * V * 4 + rows * (2 * G * D + H * V + 2 * H + G) * 4 + rows * H * V * 4
        out[f"delta_scan_{name}"] = {"us": round(ms * 1e3, 1), "prepare_us": round(ms_p * 1e3, 1),
                                     "tflops_fp32": round(flops / ms / 1e9, 2),
                                     "frac_of_fp32_ffma_nominal": round(flops / (ms / 1e3) / FP32_PEAK, 3),
                                     "frac_of_hbm": round(byts / (ms / 1e3) / hbm, 3)}

    def tables_for(reqs, seq, width):
        t = torch.zeros(reqs, width, dtype=torch.int32, device=dev)
        n = -(-seq // page)
        for r in range(reqs):
            t[r, :n] = torch.arange(1 + r * n, 1 + (r + 1) * n, dtype=torch.int32, device=dev)
        return t

    pages = B * (-(-(ctx + 1) // page)) + -(-T // page) + 2
    width = -(-max(ctx + 1, T) // page)
    # attention with capped, biased scores and a window; values of the keys' width
    H, G, D, win = z["heads"], z["kv_heads"], z["dim"], z["window"]
    kc = torch.randn(pages, G, page, D, device=dev).to(bf)
    vc = torch.randn(pages, G, page, D, device=dev).to(bf)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
    for name, reqs, per, seq in (("prefill", 1, T, T), ("decode", B, 1, ctx + 1)):
        rows = reqs * per
        q = torch.randn(rows, H, D, device=dev).to(bf)
        o = torch.empty(rows, H, D, dtype=bf, device=dev)
        step = SimpleNamespace(q_start=i32([i * per for i in range(reqs + 1)]), seq_lens=i32([seq] * reqs), num_requests=reqs,
                               num_decode=reqs if per == 1 else 0, max_q_len=per, max_seq_len=seq)
        bt = tables_for(reqs, seq, width)
        ms = timed(lambda: ops.attention_biased(o, q, kc, vc, bt, step, G, page, D ** -0.5, 30.0, slopes, win), flush)
        seen = sum(min(i + 1, win) for i in range(seq - per, seq))       # keys a request's queries see
        flops = 4.0 * D * H * seen * reqs
        byts = reqs * min(seq, win + per) * G * 2 * D * 2.0
        out[f"capped_attention_{name}"] = {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1),
                                           "frac_of_bf16": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
                                           "frac_of_hbm": round(byts / (ms / 1e3) / hbm, 3)}
    # latent attention: every head over the one cached row a token (keys of kv_rank + rot_dim, values its first kv_rank)
    H, rank, R = z["lheads"], z["kv_rank"], z["rope"]
    kc = torch.randn(pages, 1, page, rank + R, device=dev).to(bf)
    for name, reqs, per, seq in (("prefill", 1, T, T), ("decode", B, 1, ctx + 1)):
        rows = reqs * per
        q = torch.randn(rows, H, rank + R, device=dev).to(bf)
        o = torch.empty(rows, H, rank, dtype=bf, device=dev)
        step = SimpleNamespace(q_start=i32([i * per for i in range(reqs + 1)]), seq_lens=i32([seq] * reqs), num_requests=reqs,
                               num_decode=reqs if per == 1 else 0, max_q_len=per, max_seq_len=seq)
        bt = tables_for(reqs, seq, width)
        ms = timed(lambda: ops.attention_biased(o, q, kc, None, bt, step, 1, page, 0.07, 0.0, None, None), flush)
        seen = sum(i + 1 for i in range(seq - per, seq))
        flops = 2.0 * (2 * rank + R) * H * seen * reqs      # scores over rank + R columns, values over rank
        byts = reqs * seq * (rank + R) * 2.0
        out[f"latent_attention_{name}"] = {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1),
                                           "frac_of_bf16": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
                                           "frac_of_hbm": round(byts / (ms / 1e3) / hbm, 3)}
    return out


# ---- Vofinex (parallel layers on one layer norm, attention in blocks of positions with a sink, q and k rotated by
# halves and normed head by head, gated experts beside identity outputs) at layer sizes of real models, next to Komirax
# layers of the same width and weight count ---------------------------------------------------------------------------
VOFINEX_SIZES = {
    # width; heads, kv heads, head width (keys and values), rotated dimensions, block of positions; gated dense ff;
    # experts with tensors, identity outputs, top, gated expert ff (three matrices: two thirds of Komirax's widths).
    # Blocks of 1,536 positions: a prompt of 2,048 tokens crosses one edge, and a token decoded at 2,048 sees 513 keys
    "1.5b": dict(width=1536, heads=12, kv_heads=2, dim=128, rot=64, size=1536, ff=8960, experts=8, identity=4, top=4, eff=1792,
                 beside="1.5b"),
    "7b": dict(width=3584, heads=28, kv_heads=4, dim=128, rot=64, size=1536, ff=18944, experts=8, identity=4, top=4, eff=4736,
               beside="7b"),
}


def vofinex_config(z: dict, groups: int, vocab: int):
    """``groups`` times four parallel layers: (attention, dense), (attention, routed), (attention, routed), (attention,
    dense); the whole stack is one span that runs once (its vector is added to the stream)."""
    from turingserve_b200.models.vofinex import make_config
    att = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                                          "scale": z["dim"] ** -0.5, "mask": {"size": z["size"]},
                                          "rot": {"base": 500000.0, "dims": z["rot"]}}}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["eff"]},
           "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"]}}
    four = [{**att, "mlp": dense}, {**att, "mlp": moe}, {**att, "mlp": moe}, {**att, "mlp": dense}]
    return make_config(width=z["width"], vocab=vocab, layers=four * groups, eps=1e-6, residual_mult=0.5, embedding_scale=4.0,
                       logit_scale=0.5, loop={"start": 0, "stop": 4 * groups, "times": 1})


def vofinex_kernels(ops, z: dict, pk: dict, T: int, B: int, ctx: int, page: int) -> dict:
    """Each kernel of the new mechanisms alone: a portion of T tokens and B single tokens at context ``ctx``."""
    import torch
    from types import SimpleNamespace
    dev = torch.device("cuda", 0)
    big = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flush = lambda: big.fill_(1)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    out = {}
    hbm = pk["hbm_gbs"] * 1e9
    bf = torch.bfloat16
    H, G, D, W, size, rot = z["heads"], z["kv_heads"], z["dim"], z["width"], z["size"], z["rot"]

    # the stream's layer norm: two branch outputs and the pass vector into the 32-bit stream, then the norm
    for name, rows in (("prefill", T), ("decode", B)):
        stream = torch.randn(rows, W, device=dev)
        a_, b_ = torch.randn(rows, W, device=dev).to(bf), torch.randn(rows, W, device=dev).to(bf)
        w_, nb, row = torch.ones(W, device=dev), torch.zeros(W, device=dev), torch.zeros(W, device=dev)
        o = torch.empty(rows, W, dtype=bf, device=dev)
        ms = timed(lambda: ops.rmsnorm_stream(o, stream, a_, b_, w_, 1e-6, False, alpha=0.5, row=row, norm_bias=nb), flush)
        ms_r = timed(lambda: ops.rmsnorm_stream(o, stream, a_, None, w_, 1e-6, False), flush)
        byts = rows * W * (4 + 4 + 2 + 2 + 2.0)
        out[f"stream_layer_norm_{name}"] = {"us": round(ms * 1e3, 1), "frac_of_hbm": round(byts / (ms / 1e3) / hbm, 3),
                                            "beside_rms_norm_us": round(ms_r * 1e3, 1),
                                            "beside_frac_of_hbm": round(rows * W * 12.0 / (ms_r / 1e3) / hbm, 3)}

    pages = B * (-(-(ctx + 1) // page)) + -(-T // page) + 2
    width = -(-max(ctx + 1, T) // page)
    kc = torch.randn(pages, G, page, D, device=dev).to(bf)
    vc = torch.randn(pages, G, page, D, device=dev).to(bf)
    # rotation by halves, unit heads, cache write
    freq = (500000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(dev)
    for name, rows in (("prefill", T), ("decode", B)):
        proj = torch.randn(rows, (H + 2 * G) * D, device=dev).to(bf)
        pos = i32(list(range(rows)))
        slots = i32(list(range(page, page + rows)))
        ms = timed(lambda: ops.rope_headnorm_write(proj, H * D, (H + G) * D, pos, freq, rot, 1e-6, kc, vc, slots, H, G, D, D, page), flush)
        byts = rows * (2 * H * D + 2 * 2 * G * D) * 2.0
        # beside it the rotation by a table and cache write of the Qwen2 layers (full heads, no norm) on the same rows
        cos, sin = torch.ones(rows, D // 2, device=dev), torch.zeros(rows, D // 2, device=dev)
        ms_q = timed(lambda: ops.rope_kv_write(proj, pos, cos, sin, H, G, D, D, kc, vc, slots, page), flush)
        out[f"rotate_norm_write_{name}"] = {"us": round(ms * 1e3, 1), "frac_of_hbm": round(byts / (ms / 1e3) / hbm, 3),
                                            "beside_table_rotation_us": round(ms_q * 1e3, 1),
                                            "beside_frac_of_hbm": round(byts / (ms_q / 1e3) / hbm, 3)}

    # attention in blocks with a sink
    sinks = torch.zeros(H, device=dev)
    for name, reqs, per, seq in (("prefill", 1, T, T), ("decode", B, 1, ctx + 1)):
        rows = reqs * per
        q = torch.randn(rows, H, D, device=dev).to(bf)
        o = torch.empty(rows, H, D, dtype=bf, device=dev)
        bt = torch.zeros(reqs, width, dtype=torch.int32, device=dev)
        n = -(-seq // page)
        for r in range(reqs):
            bt[r, :n] = torch.arange(1 + r * n, 1 + (r + 1) * n, dtype=torch.int32, device=dev)
        for tag, c in (("", size), ("_no_blocks", None)):
            sq = seq
            if c and per == 1:
                sq = (seq - 1) // c * c                    # a single token at its block's last position: a full block of keys
            step = SimpleNamespace(q_start=i32([i * per for i in range(reqs + 1)]), seq_lens=i32([sq] * reqs), num_requests=reqs,
                                   num_decode=reqs if per == 1 else 0, max_q_len=per, max_seq_len=sq)
            ms = timed(lambda: ops.attention_biased(o, q, kc, vc, bt, step, G, page, D ** -0.5, 0.0, None, None, chunk=c,
                                                    sinks=sinks), flush)
            seen = sum(i % c + 1 if c else i + 1 for i in range(sq - per, sq))       # keys a request's queries see
            flops = 4.0 * D * H * seen * reqs
            held = min(sq, (sq - 1) % c + 1 + (per - 1 if per > 1 else 0)) if c else sq
            byts = reqs * held * G * 2 * D * 2.0 + rows * H * D * 4.0
            out[f"sink_attention{tag}_{name}"] = {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1),
                                                  "frac_of_bf16": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
                                                  "frac_of_hbm": round(byts / (ms / 1e3) / hbm, 3)}

    # the routed feed-forward: router (softmax, correction) + sort, gather, gate/up product, activation, down product, sum
    E, ident, top, ff = z["experts"], z["identity"], z["top"], z["eff"]
    w_up = (torch.randn(E, 2 * ff, W, device=dev) * 0.02).to(bf)
    w_down = (torch.randn(E, W, ff, device=dev) * 0.02).to(bf)
    wr = torch.randn(E + ident, W, device=dev) * 0.05
    corr = torch.randn(E + ident, device=dev) * 0.01
    for name, rows in (("prefill", T), ("decode", B)):
        x = torch.randn(rows, W, device=dev).to(bf)
        idx = torch.empty(rows, top, dtype=torch.int32, device=dev)
        wts = torch.empty(rows, top, device=dev)
        a_ = torch.empty(rows * top, 2 * ff, dtype=bf, device=dev)
        g_ = torch.empty(rows * top, ff, dtype=bf, device=dev)
        y = torch.zeros(rows * top, W, device=dev)
        o = torch.empty(rows, W, dtype=bf, device=dev)
        ops.router_topk(idx, wts, x, wr, True, False, corr)
        offsets, order, place, tiles = ops.moe_align(idx, E + ident, E)
        real = int(offsets[E])                                   # pairs that go to experts with tensors
        ms_r = timed(lambda: (ops.router_topk(idx, wts, x, wr, True, False, corr), ops.moe_align(idx, E + ident, E)), flush)
        xs = torch.empty(rows * top, W, dtype=bf, device=dev)
        ms_g = timed(lambda: ops.moe_gather(xs, x, order, None, top), flush)
        ms_u = timed(lambda: ops.grouped_linear(a_, xs, w_up, None, None, offsets, tiles, 1), flush)
        ms_a = timed(lambda: ops.silu_mul(g_, a_, 0), flush)
        ms_d = timed(lambda: ops.grouped_linear(y, g_, w_down, None, None, offsets, tiles, 1), flush)
        ms_c = timed(lambda: ops.moe_combine(o, y, place, wts, top, x=x, pass_from=offsets[E:E + 1]), flush)
        flops_u, flops_d = 4.0 * real * ff * W, 2.0 * real * ff * W
        used = min(E, max(1, real))
        out[f"routed_ff_{name}"] = {
            "pairs_with_tensors": real, "pairs": rows * top,
            "router_and_sort_us": round(ms_r * 1e3, 1), "gather_us": round(ms_g * 1e3, 1), "up_us": round(ms_u * 1e3, 1),
            "activation_us": round(ms_a * 1e3, 1), "down_us": round(ms_d * 1e3, 1), "sum_us": round(ms_c * 1e3, 1),
            "up_tflops": round(flops_u / ms_u / 1e9, 1), "down_tflops": round(flops_d / ms_d / 1e9, 1),
            "up_frac_of_bf16": round(flops_u / (ms_u / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
            "down_frac_of_bf16": round(flops_d / (ms_d / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
            "up_frac_of_hbm": round(used * 2 * ff * W * 2.0 / (ms_u / 1e3) / hbm, 3),
            "down_frac_of_hbm": round(used * ff * W * 2.0 / (ms_d / 1e3) / hbm, 3)}
    return out


# ---- Gugezen (a stream in several copies, attention with a sink and an output gate beside linear attention, the
# state-space mixer, gated GELU and routed feed-forwards with a shared expert) beside Komirax layers ----------------
GUGEZEN_SIZES = {
    # width; attention half: heads, kv heads, head width, rotated dimensions; linear half: heads (key and value width as the
    # attention's); state-space mixer: heads, head width, state rows, groups, taps, norm parts; gated dense ff (three
    # matrices: two thirds of the Komirax width for the same weight count); experts, top, expert ff, shared expert ff
    "1.5b": dict(width=1536, heads=12, kv_heads=2, dim=128, rot=128, lheads=6, sheads=48, sdim=64, state=128, sgroups=2, taps=4,
                 parts=2, ff=8960, experts=8, top=2, eff=2688, shared=1344, streams=2, beside="1.5b"),
    "7b": dict(width=3584, heads=28, kv_heads=4, dim=128, rot=128, lheads=14, sheads=112, sdim=64, state=128, sgroups=2, taps=4,
               parts=2, ff=18944, experts=8, top=2, eff=7104, shared=3552, streams=2, beside="7b"),
}


def gugezen_config(z: dict, groups: int, vocab: int):
    """``groups`` times four layers: (state-space, dense), (attention + linear attention, routed), (state-space, routed),
    (attention + linear attention, dense)."""
    from turingserve_b200.models.gugezen import make_config
    pair = {"type": "parallel", "mixer": {
        "left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
                 "rot": {"base": 500000.0, "dims": z["rot"], "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}},
        "right": {"heads": z["lheads"], "dim": z["dim"], "vdim": z["dim"],
                  "decay": [1.0 - 2.0 ** -(2 + 6 * i / max(1, z["lheads"] - 1)) for i in range(z["lheads"])]},
        "left_scale": 0.7, "right_scale": 1.1}}
    ssm = {"type": "mamba2", "mixer": {"heads": z["sheads"], "vdim": z["sdim"], "state": z["state"], "groups": z["sgroups"],
                                       "conv": z["taps"], "norm_groups": z["parts"]}}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["eff"]}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared"]}}
    four = [{**ssm, "mlp": dense}, {**pair, "mlp": moe}, {**ssm, "mlp": moe}, {**pair, "mlp": dense}]
    return make_config(width=z["width"], vocab=vocab, layers=four * groups, eps=1e-6, streams=z["streams"], embedding_scale=4.0,
                       logit_scale=0.5)


def gugezen_kernels(ops, z: dict, pk: dict, T: int, B: int, ctx: int, page: int) -> dict:
    """Each kernel of the new mechanisms alone, beside the like kernel of the closest design: a portion of T tokens and B
    single tokens at context ``ctx``."""
    import torch
    from types import SimpleNamespace
    dev = torch.device("cuda", 0)
    big = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flush = lambda: big.fill_(1)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    out = {}
    hbm = pk["hbm_gbs"] * 1e9
    FP32_PEAK = 148 * 128 * 2 * 1.965e9                      # FFMA lanes x 2 x the highest SM clock: nominal
    bf = torch.bfloat16
    W, S = z["width"], z["streams"]
    H, G, D, rot = z["heads"], z["kv_heads"], z["dim"], z["rot"]
    frac = lambda byts, ms: round(byts / (ms / 1e3) / hbm, 3)

    # the norm over the stream's copies (write-back of the pending output, read, norm) beside the one-copy stream norm
    for name, rows in (("prefill", T), ("decode", B)):
        streams = torch.randn(rows, S, W, device=dev)
        one = torch.randn(rows, W, device=dev)
        y = torch.randn(rows, W, device=dev).to(bf)
        w_ = torch.ones(W, device=dev)
        mix, wo, wi = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.full((S,), 1.0 / S, device=dev)
        o = torch.empty(rows, W, dtype=bf, device=dev)
        ms = timed(lambda: ops.hyper_norm(o, streams, y, mix, wo, wi, w_, 1e-6), flush)
        ms_r = timed(lambda: ops.rmsnorm_stream(o, one, y, None, w_, 1e-6, False), flush)
        out[f"stream_copies_norm_{name}"] = {"us": round(ms * 1e3, 1), "frac_of_hbm": frac(rows * W * (8.0 * S + 4), ms),
                                             "beside_stream_norm_us": round(ms_r * 1e3, 1),
                                             "beside_frac_of_hbm": frac(rows * W * 12.0, ms_r)}

    pages = B * (-(-(ctx + 1) // page)) + -(-T // page) + 2
    width = -(-max(ctx + 1, T) // page)
    kc = torch.randn(pages, G, page, D, device=dev).to(bf)
    vc = torch.randn(pages, G, page, D, device=dev).to(bf)
    # rotation of neighbouring pairs + cache write, beside the rotation by halves with the per-head norm
    freq = (500000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(dev)
    n_left = (2 * H + 2 * G) * D                             # q | k | v | gate
    for name, rows in (("prefill", T), ("decode", B)):
        proj = torch.randn(rows, n_left, device=dev).to(bf)
        pos = i32(list(range(rows)))
        slots = i32(list(range(page, page + rows)))
        ms = timed(lambda: ops.rope_pairs_write(proj, H * D, (H + G) * D, pos, freq, 1.0, rot, kc, vc, slots, H, G, D, D, page), flush)
        byts = rows * (2 * H * D + 2 * 2 * G * D) * 2.0
        ms_h = timed(lambda: ops.rope_headnorm_write(proj, H * D, (H + G) * D, pos, freq, rot, 1e-6, kc, vc, slots, H, G, D, D, page), flush)
        out[f"rotate_pairs_write_{name}"] = {"us": round(ms * 1e3, 1), "frac_of_hbm": frac(byts, ms),
                                             "beside_rotation_by_halves_us": round(ms_h * 1e3, 1), "beside_frac_of_hbm": frac(byts, ms_h)}

    # attention with a sink (no blocks of positions), then the output gate
    sinks = torch.zeros(H, device=dev)
    for name, reqs, per, seq in (("prefill", 1, T, T), ("decode", B, 1, ctx + 1)):
        rows = reqs * per
        q = torch.randn(rows, H, D, device=dev).to(bf)
        o = torch.empty(rows, H, D, dtype=bf, device=dev)
        gate = torch.randn(rows, H * D, device=dev).to(bf)
        heads = torch.empty(rows, H * D, dtype=bf, device=dev)
        bt = torch.zeros(reqs, width, dtype=torch.int32, device=dev)
        n = -(-seq // page)
        for r in range(reqs):
            bt[r, :n] = torch.arange(1 + r * n, 1 + (r + 1) * n, dtype=torch.int32, device=dev)
        step = SimpleNamespace(q_start=i32([i * per for i in range(reqs + 1)]), seq_lens=i32([seq] * reqs), num_requests=reqs,
                               num_decode=reqs if per == 1 else 0, max_q_len=per, max_seq_len=seq)
        ms = timed(lambda: ops.attention_biased(o, q, kc, vc, bt, step, G, page, D ** -0.5, 0.0, None, None, chunk=None, sinks=sinks), flush)
        ms_g = timed(lambda: ops.gate_mul(heads, o.view(rows, H * D), gate, "sigmoid", 0.7), flush)
        seen = sum(i + 1 for i in range(seq - per, seq))
        flops = 4.0 * D * H * seen * reqs
        byts = reqs * seq * G * 2 * D * 2.0 + rows * H * D * 4.0
        out[f"sink_attention_{name}"] = {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1),
                                         "frac_of_bf16": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
                                         "frac_of_hbm": frac(byts, ms), "gate_us": round(ms_g * 1e3, 1),
                                         "gate_frac_of_hbm": frac(rows * H * D * 6.0, ms_g)}

    # the state-space mixer: prepare (filter, SiLU, dt, decay) and scan, beside the linear attention's scan at the same
    # number of state values a layer
    SH, P, N, SG, taps, parts = z["sheads"], z["sdim"], z["state"], z["sgroups"], z["taps"], z["parts"]
    inner, channels = SH * P, SH * P + 2 * SG * N
    n_in = 2 * inner + 2 * SG * N + SH
    conv_w, conv_b = torch.randn(channels, taps, device=dev) * 0.3, torch.zeros(channels, device=dev)
    a_log, dt_bias, skip = torch.zeros(SH, device=dev), torch.zeros(SH, device=dev), torch.ones(SH, device=dev)
    norm_w = torch.ones(inner, device=dev)
    LH = z["lheads"]
    decay = torch.full((LH,), 0.99, device=dev)
    for name, reqs, per in (("prefill", 1, T), ("decode", B, 1)):
        rows = reqs * per
        proj = torch.randn(rows, n_in, device=dev).to(bf)
        state = torch.zeros(reqs + 1, SH * N * P + (taps - 1) * channels, device=dev)
        step = SimpleNamespace(q_start=i32([i * per for i in range(reqs + 1)]), state_slots=i32(list(range(reqs))), num_requests=reqs,
                               token_request=i32([r for r in range(reqs) for _ in range(per)]), max_q_len=per)
        ready = torch.empty(rows, channels + 2 * SH, device=dev)
        y = torch.empty(rows, inner, device=dev)
        g_ = torch.empty(rows, inner, dtype=bf, device=dev)
        ms_p = timed(lambda: ops.ssm_prepare(ready, proj, inner, inner + channels, conv_w, conv_b, a_log, dt_bias, state, SH * N * P,
                                             step, SH, channels, taps), flush)
        ms_s = timed(lambda: ops.ssm_scan(y, ready, proj, inner, state, skip, step, SH, SG, N, P, taps), flush)
        ms_n = timed(lambda: ops.gated_group_rmsnorm(g_, y, proj[:, :inner], norm_w, 1e-6, parts, "silu", True), flush)
        flops = 5.0 * rows * SH * N * P                       # decay, write (two), read (two) a state value
        # the linear attention of the paired mixer (and of Komirax): D x D states
        lproj = torch.randn(rows, 4 * LH * D, device=dev).to(bf)
        lstate = torch.zeros(reqs + 1, LH, D, D, device=dev)
        lo = torch.empty(rows, LH * D, device=dev)
        ms_l = timed(lambda: ops.lightning(lo, lproj, lstate, decay, step, LH, D, D), flush)
        lflops = 5.0 * rows * LH * D * D
        lg = torch.empty(rows, LH * D, dtype=bf, device=dev)
        lw = torch.ones(LH * D, device=dev).to(bf)
        ms_ln = timed(lambda: ops.gated_rmsnorm(lg, lo, lproj[:, 3 * LH * D:], lw, 1e-6), flush)
        out[f"state_space_{name}"] = {
            "prepare_us": round(ms_p * 1e3, 1), "prepare_frac_of_hbm": frac(rows * (channels * 2.0 + (channels + 2 * SH) * 4.0), ms_p),
            "scan_us": round(ms_s * 1e3, 1), "scan_tflops_fp32": round(flops / ms_s / 1e9, 2),
            "scan_frac_of_fp32_nominal": round(flops / (ms_s / 1e3) / FP32_PEAK, 3),
            "scan_frac_of_hbm": frac(reqs * SH * N * P * 8.0 + rows * (channels + inner) * 4.0, ms_s),
            "gated_norm_us": round(ms_n * 1e3, 1), "gated_norm_frac_of_hbm": frac(rows * inner * 8.0, ms_n),
            "beside_linear_attention_scan_us": round(ms_l * 1e3, 1), "beside_scan_tflops_fp32": round(lflops / ms_l / 1e9, 2),
            "beside_scan_frac_of_fp32_nominal": round(lflops / (ms_l / 1e3) / FP32_PEAK, 3),
            "beside_scan_frac_of_hbm": frac(reqs * LH * D * D * 8.0 + rows * LH * D * (3 * 2.0 + 4.0), ms_l),
            "beside_gated_norm_us": round(ms_ln * 1e3, 1), "beside_gated_norm_frac_of_hbm": frac(rows * LH * D * 8.0, ms_ln)}

    # the gated dense feed-forward's activation beside the SiLU one
    ff = z["ff"]
    for name, rows in (("prefill", T), ("decode", B)):
        gu = torch.randn(rows, 2 * ff, device=dev).to(bf)
        a_ = torch.empty(rows, ff, dtype=bf, device=dev)
        ms = timed(lambda: ops.act_mul(a_, gu, "gelu_tanh", 64), flush)
        ms_q = timed(lambda: ops.silu_mul(a_, gu, 64), flush)
        out[f"gelu_gate_{name}"] = {"us": round(ms * 1e3, 1), "frac_of_hbm": frac(rows * ff * 6.0, ms),
                                    "beside_silu_us": round(ms_q * 1e3, 1), "beside_frac_of_hbm": frac(rows * ff * 6.0, ms_q)}
    return out


def run_design(a) -> dict:
    """``--design komirax``: prefill and decode throughput of Komirax layers beside Qwen2 layers of the same
    width and count (random weights, bfloat16, through the step function), and each new kernel alone."""
    import numpy as np
    import torch

    from turingserve_b200 import kernels
    from turingserve_b200.engine.batch import StepEntry

    torch.cuda.set_device(0)
    ops = kernels.ops()
    pk, pk_src = peaks()
    rng = np.random.default_rng(0)
    B, T, ctx, page = a.batch, a.prefill_tokens, a.prompt_len, 64
    steps, warmup = min(a.steps, 64), max(3, a.warmup)
    vocab = 32768
    result = {"design": a.design, "dtype": "bfloat16", "data": "synthetic", "peaks": pk_src, "batch": B,
              "prefill_tokens": T, "context": ctx, "page": page, "sizes": {}}

    def measure(eng):
        runner, cache = eng.runner, eng.cache
        toks = rng.integers(0, vocab, size=T).tolist()
        times = []
        for i in range(6):
            rc = cache.admit("p")
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step([StepEntry(rc, toks, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            cache.release(rc)
            if i >= 3:
                times.append(e0.elapsed_time(e1))
        pms = sorted(times)[1]
        rcs = [cache.admit(f"d{i}") for i in range(B)]
        for rc in rcs:
            runner.step([StepEntry(rc, rng.integers(0, vocab, size=ctx).tolist(), [])])
        dt = rng.integers(0, vocab, size=(warmup + steps, B))
        for s_ in range(warmup):
            runner.step([StepEntry(rc, [int(dt[s_, i])], [0]) for i, rc in enumerate(rcs)])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s_ in range(warmup, warmup + steps):
            runner.step([StepEntry(rc, [int(dt[s_, i])], [0]) for i, rc in enumerate(rcs)])
        e1.record()
        torch.cuda.synchronize()
        dms = e0.elapsed_time(e1) / steps
        for rc in rcs:
            cache.release(rc)
        return {"prefill_ms": round(pms, 3), "prefill_tok_s": round(T / (pms / 1e3), 1), "decode_ms_per_step": round(dms, 4),
                "decode_tok_s": round(B / (dms / 1e3), 1)}

    for name in a.design_sizes.split(","):
        groups = a.layers // 4 if a.layers else 2
        ctx_len = max(ctx + warmup + steps + 64, T + 64)
        if a.design == "vofinex":
            # beside Komirax layers of the same width and weight count, the closest design the engine has (a 32-bit
            # stream, an attention with key and value widths of its own, dense and routed feed-forwards)
            z = VOFINEX_SIZES[name]
            eng = build_engine_on_device(f"vofinex-{name}", 4 * groups, ctx_len=ctx_len, page=page, max_seqs=B,
                                         max_tokens=max(T, ctx), graph_sizes=(B,), mcfg=vofinex_config(z, groups, vocab))
            ours = measure(eng)
            del eng
            torch.cuda.empty_cache()
            eng = build_engine_on_device(f"komirax-{z['beside']}", 4 * groups, ctx_len=ctx_len, page=page, max_seqs=B,
                                         max_tokens=max(T, ctx), graph_sizes=(B,),
                                         mcfg=komirax_config(KOMIRAX_SIZES[z["beside"]], groups, vocab))
            beside = measure(eng)
            del eng
            torch.cuda.empty_cache()
            entry = {"layers": 4 * groups, "width": z["width"], "vofinex": ours, "beside": f"komirax-{z['beside']}", "komirax": beside,
                     "prefill_ratio": round(ours["prefill_tok_s"] / beside["prefill_tok_s"], 3),
                     "decode_ratio": round(ours["decode_tok_s"] / beside["decode_tok_s"], 3)}
            if "kernels" in a.phases.split(","):
                entry["kernels"] = vofinex_kernels(ops, z, pk, T, B, ctx, page)
                entry["komirax_kernels"] = komirax_kernels(ops, KOMIRAX_SIZES[z["beside"]], pk, T, B, ctx, page)
            result["sizes"][name] = entry
            continue
        if a.design == "gugezen":
            # beside Komirax layers of the same width and about the same weight count, the closest design the engine has (a
            # 32-bit stream, linear attention with a decaying state, an attention of its own, dense and routed feed-forwards)
            z = GUGEZEN_SIZES[name]
            eng = build_engine_on_device(f"gugezen-{name}", 4 * groups, ctx_len=ctx_len, page=page, max_seqs=B,
                                         max_tokens=max(T, ctx), graph_sizes=(B,), mcfg=gugezen_config(z, groups, vocab))
            ours = measure(eng)
            del eng
            torch.cuda.empty_cache()
            eng = build_engine_on_device(f"komirax-{z['beside']}", 4 * groups, ctx_len=ctx_len, page=page, max_seqs=B,
                                         max_tokens=max(T, ctx), graph_sizes=(B,),
                                         mcfg=komirax_config(KOMIRAX_SIZES[z["beside"]], groups, vocab))
            beside = measure(eng)
            del eng
            torch.cuda.empty_cache()
            entry = {"layers": 4 * groups, "width": z["width"], "gugezen": ours, "beside": f"komirax-{z['beside']}", "komirax": beside,
                     "prefill_ratio": round(ours["prefill_tok_s"] / beside["prefill_tok_s"], 3),
                     "decode_ratio": round(ours["decode_tok_s"] / beside["decode_tok_s"], 3)}
            if "kernels" in a.phases.split(","):
                entry["kernels"] = gugezen_kernels(ops, z, pk, T, B, ctx, page)
            result["sizes"][name] = entry
            continue
        if a.design == "pizunex":
            # beside Komirax layers of the same width, the closest design the engine has (a 32-bit stream, a recurrent
            # mixer with a matrix state, an attention of its own, feed-forwards without a gate)
            z = PIZUNEX_SIZES[name]
            eng = build_engine_on_device(f"pizunex-{name}", 4 * groups, ctx_len=ctx_len, page=page, max_seqs=B,
                                         max_tokens=max(T, ctx), graph_sizes=(B,), mcfg=pizunex_config(z, groups, vocab))
            ours = measure(eng)
            del eng
            torch.cuda.empty_cache()
            eng = build_engine_on_device(f"komirax-{z['beside']}", 4 * groups, ctx_len=ctx_len, page=page, max_seqs=B,
                                         max_tokens=max(T, ctx), graph_sizes=(B,),
                                         mcfg=komirax_config(KOMIRAX_SIZES[z["beside"]], groups, vocab))
            beside = measure(eng)
            del eng
            torch.cuda.empty_cache()
            entry = {"layers": 4 * groups, "width": z["width"], "pizunex": ours, "beside": f"komirax-{z['beside']}", "komirax": beside,
                     "prefill_ratio": round(ours["prefill_tok_s"] / beside["prefill_tok_s"], 3),
                     "decode_ratio": round(ours["decode_tok_s"] / beside["decode_tok_s"], 3)}
            if "kernels" in a.phases.split(","):
                entry["kernels"] = pizunex_kernels(ops, z, pk, T, B, ctx, page)
            result["sizes"][name] = entry
            continue
        z = KOMIRAX_SIZES[name]
        kcfg = komirax_config(z, groups, vocab)
        eng = build_engine_on_device(f"komirax-{name}", 4 * groups, ctx_len=ctx_len, page=page, max_seqs=B,
                                     max_tokens=max(T, ctx), graph_sizes=(B,), mcfg=kcfg)
        ours = measure(eng)
        del eng
        torch.cuda.empty_cache()
        qkw = dict(SHAPES[z["beside"]])
        qkw.update(num_layers=4 * groups, vocab_size=vocab, tie_word_embeddings=False)
        from turingserve_b200.models.qwen2 import make_config as qwen_config
        eng = build_engine_on_device(z["beside"], 4 * groups, ctx_len=ctx_len, page=page, max_seqs=B,
                                     max_tokens=max(T, ctx), graph_sizes=(B,), mcfg=qwen_config(**qkw))
        beside = measure(eng)
        del eng
        torch.cuda.empty_cache()
        entry = {"layers": 4 * groups, "width": z["width"], "komirax": ours, "beside": z["beside"], "qwen2": beside,
                 "prefill_ratio": round(ours["prefill_tok_s"] / beside["prefill_tok_s"], 3),
                 "decode_ratio": round(ours["decode_tok_s"] / beside["decode_tok_s"], 3)}
        if "kernels" in a.phases.split(","):
            entry["kernels"] = komirax_kernels(ops, z, pk, T, B, ctx, page)
        result["sizes"][name] = entry
    result["gpu_launches"] = ops.launches
    return result


def run_reference(a) -> dict:
    """The unmodified reference from baseline/_ref through its own ``build_engine`` /
    ``LLMEngine.step``: float16 (it has no bfloat16), Triton kernels, CUDA graphs, same workload."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "turingserve")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed"}
    sys.path.insert(0, ref)
    import numpy as np
    import torch

    kw = SHAPES[a.model]
    layers = a.layers or kw["num_layers"]
    B, prompt_len, ctx_len = a.batch, a.prompt_len, a.context
    rng = np.random.default_rng(0)
    try:
        from turingserve.config import EngineConfig as RefConfig
        from turingserve.engine.builder import build_engine
        from turingserve.engine.sampling_params import SamplingParams as RefParams
        with tempfile.TemporaryDirectory() as tmp:
            folder = make_model(a.model, layers, tmp)
            cfg = RefConfig(model=folder, dtype="float16", device="cuda", kernels="triton", max_model_len=ctx_len,
                            num_blocks=B * (-(-ctx_len // 16)) + 64, max_num_seqs=B, max_num_batched_tokens=2048,
                            cuda_graphs=True, graph_batch_sizes=(B,), prefix_caching=False, autopilot="off",
                            log_level="warning")
            eng = build_engine(cfg, tokenizer=_StubTokenizer())
        steps, warmup = a.steps, max(3, a.warmup)
        params = RefParams(temperature=0.0, max_tokens=warmup + steps + B + 8, ignore_eos=True)
        for i in range(B):
            eng.add_request(f"r{i}", rng.integers(0, kw["vocab_size"], size=prompt_len).tolist(), params)
        while eng.scheduler.waiting or any(s.num_uncomputed > 1 for s in eng.scheduler.running):
            eng.step()
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        with ClockSampler() as clocks:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record()
            n_tok = 0
            for _ in range(steps):
                n_tok += sum(len(o.delta_token_ids) for o in eng.step())
            e1.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
        ms = e0.elapsed_time(e1) / steps
        # per step its input builder copies ids, positions, slots and sample rows (int64), query starts and
        # lengths (int32), the block table at its live width, and the all-greedy flag; tokens and bad flags
        # (int64) and that flag's answer come back (turingserve/runner/input_builder.py:138-144,
        # turingserve/sampling/sampler.py:88-89,105-106)
        width = -(-(prompt_len + warmup + steps) // 16)
        h2d = 8 * 4 * B + 4 * (B + 1) + 4 * B + 4 * B * width + B
        d2h = 2 * 8 * B + 1
        return {"metric": metric_name(a),
                "value": round(n_tok / (ms * steps / 1e3), 1), "unit": "tok/s", "n_gpus": 1, "steps": steps,
                "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "fp16", "data": "synthetic: uniform random token ids, N(0,0.02) random weights",
                "impl": "reference",
                "config": {"model": a.model, "layers": layers, "global_batch": B, "seq_len": ctx_len,
                           "prompt_len": prompt_len, "parallelism": "single GPU", "cuda_graphs": True,
                           "kernels": "triton"},
                "clocks": clocks.summary(),
                "e2e": {"value": round(n_tok / wall, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": d2h}}
    except Exception as e:                                   # the reference targets Turing + torch 2.6/triton 3.2
        return {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e).splitlines()[0][:200] if str(e) else ''}"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen2.5-1.5b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0 = all)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--kv-block", type=int, default=16, help="tokens per cache page (the reference's 16)")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--phases", default="prefill,decode,points,e2e,kernels,mixed",
                    help="which measurements to run (decode always runs); fewer for a profiler capture")
    ap.add_argument("--design", default="", choices=["", "komirax", "pizunex", "vofinex", "gugezen"],
                    help="instead of the default workload: layers of this design beside layers of the closest other one (Komirax "
                         "beside Qwen2, Pizunex beside Komirax) at the same width "
                         "(prefill and decode throughput, and each of the design's kernels alone)")
    ap.add_argument("--design-sizes", default="1.5b,7b", help="which of the design's layer sizes to run")
    a = ap.parse_args()
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.design:
        print(json.dumps(run_design(a)))
        return 0
    out = run_reference(a) if a.impl == "reference" else run_ours(a)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
