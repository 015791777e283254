#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen3-8B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch (default: 8 sequences, 512-token
prompts, context cap 4096).  Prints ONE JSON line:
  value    decoded tokens per second, timed on the device with CUDA events over
           exactly K steps after W warm-up steps (synthetic token ids fed from
           the host each step, no read-back inside the timed region);
  e2e      the same through the Python entry point Engine.generate: host token
           lists in, host token lists out, a device-to-host read every step;
  prefill  one 2,048-token prompt in one step;
  roofline the decode step against the HBM copy bandwidth: every weight it uses
           once plus the live requests' cache, divided by its time;
  points   decode at batch 1 and 64.
Peaks come from MEASURED_PEAKS.json beside this file when it exists.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: the Qwen3-8B shape
SHAPE_8B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1e6,
                rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960)
WEIGHT_SEED = 5
CONTEXT = 4096
PROMPT = 512
PREFILL_TOKENS = 2048

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"]))}, "measured"
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        clocks = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        maxes = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None,
                "sm_max_mhz": max(maxes) if maxes else None, "reasons": reasons, "samples": len(clocks)}


def count_params(cfg, n_layers):
    d, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * (qd + 2 * kvd) + qd * d + 3 * d * I
    return per_layer, V * d  # layer matrices; head (the embedding table is read by rows only)


def decode_bytes(cfg, n_layers, batch, ctx_tokens):
    """Bytes a decode step has to read: every matrix once (bfloat16) and the live cache."""
    per_layer, head = count_params(cfg, n_layers)
    weights = 2 * (per_layer * n_layers + head)
    kv = 2 * 2 * n_layers * cfg["num_key_value_heads"] * cfg["head_dim"] * ctx_tokens * batch
    return weights + kv


def prefill_flops(cfg, n_layers, T):
    per_layer, head = count_params(cfg, n_layers)
    gemm = 2 * T * per_layer * n_layers + 2 * head  # logits at the last place only
    attn = 4 * cfg["num_attention_heads"] * cfg["head_dim"] * (T * (T + 1) // 2) * n_layers
    return gemm + attn


def run_decode(engine, batch, steps, warmup, vocab, seed=1):
    """Device-timed decode: returns (tokens/s, ms/step, mean context length, kernel launches)."""
    import numpy as np
    import torch
    from odin_infer_b200 import StepEntry
    from odin_infer_b200.csrc import ops
    rng = np.random.default_rng(seed)
    slots = [engine.take_slot() for _ in range(batch)]
    try:
        prompts = [rng.integers(0, vocab, PROMPT).tolist() for _ in range(batch)]
        engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        feed = rng.integers(0, vocab, (warmup + steps, batch))
        for i in range(warmup):
            engine.step([StepEntry(s, [int(feed[i, b])], [0]) for b, s in enumerate(slots)])
        torch.cuda.synchronize()
        ctx0 = engine.cache.lengths[slots[0]]
        launches0 = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warmup, warmup + steps):
            engine.step([StepEntry(s, [int(feed[i, b])], [0]) for b, s in enumerate(slots)])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = ops.launch_count() - launches0
        mean_ctx = ctx0 + (steps + 1) / 2
        return batch * steps / (ms / 1e3), ms / steps, mean_ctx, launches
    finally:
        for s in slots:
            engine.give_back_slot(s)


def run_prefill(engine, vocab, reps=3):
    import numpy as np
    import torch
    from odin_infer_b200 import StepEntry
    rng = np.random.default_rng(7)
    best = None
    for r in range(reps + 1):
        toks = rng.integers(0, vocab, PREFILL_TOKENS).tolist()
        slot = engine.take_slot()
        try:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([StepEntry(slot, toks, [len(toks) - 1])])
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
        finally:
            engine.give_back_slot(slot)
        if r > 0:  # the first run warms up
            best = ms if best is None else min(best, ms)
    return best


def run_e2e(engine, batch, steps, vocab):
    """Through Engine.generate: host token lists in and out, one read-back per step.  Returns the statistics of a
    call of `steps` decode steps and, when that is short, of one of 256 steps as well: the first ~20 decode steps
    after a prompt step run 12 to 15 % slower than the later ones (the prompt step runs at the power cap and the
    SM clock takes ~80 ms to come back), so a short call measures mostly that."""
    import numpy as np
    from odin_infer_b200 import GenerationStats
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, vocab, PROMPT).tolist() for _ in range(batch)]
    engine.generate(prompts, max_new_tokens=4, temperature=0.0, stop_token_ids=[])  # warm-up (graphs, allocator)
    stats = GenerationStats()
    out = engine.generate(prompts, max_new_tokens=steps + 1, temperature=0.0, stop_token_ids=[], stats=stats)
    assert all(len(o.tokens) == steps + 1 for o in out)
    steady = None
    if steps < 128:
        steady = GenerationStats()
        engine.generate(prompts, max_new_tokens=257, temperature=0.0, stop_token_ids=[], stats=steady)
    return stats, steady


SHAPE_1P7B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=2048, intermediate_size=6144, num_hidden_layers=28,
                  num_attention_heads=16, num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1e6,
                  rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=40960)
SHAPE_32B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=5120, intermediate_size=25600, num_hidden_layers=64,
                 num_attention_heads=64, num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1e6,
                 rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960)


def other_workload(which: str) -> int:
    """BASELINE.json configs[3] and configs[4]; one JSON line each, device-timed unless said otherwise."""
    import time

    import numpy as np
    import torch
    from odin_infer_b200 import Engine, Engine_Opts, StepEntry
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.engine.generate import GenerationStats
    peaks, peak_source = load_peaks()
    if which == "1.7b-mixed":
        raw = dict(SHAPE_1P7B)
        rng = np.random.default_rng(11)
        lens = rng.integers(16, 2049, 64)
        prompts = [rng.integers(0, raw["vocab_size"], int(n)).tolist() for n in lens]
        need = sum((int(n) + 128 + 63) // 64 * 64 for n in lens)
        e = Engine.random(config_from_dict(raw), 6, Engine_Opts(max_ctx=4096, max_tokens=need, max_batch=64,
                                                                dtype="bfloat16", verbose=False))
        e.generate(prompts, max_new_tokens=128, stop_token_ids=[])  # warm-up: the same requests once (kernels, graphs)
        st = GenerationStats()
        t0 = time.perf_counter()
        e.generate(prompts, max_new_tokens=128, stop_token_ids=[], stats=st)
        total = time.perf_counter() - t0
        out = {"metric": "Qwen3-1.7B shape, bf16: 64 prompts of 16..2048 tokens in one batch, 128 new tokens each, "
                         "through Engine.generate (host clock, second pass over the same requests)", "prompt_tokens": int(lens.sum()),
               "ttft_ms": round(st.ttft_s * 1e3, 1), "prefill_tokens_per_s": round(float(lens.sum()) / st.ttft_s),
               "decode_tokens_per_s": round(st.decode_tokens_per_s), "total_s": round(total, 3), "batches": st.n_batches}
    else:
        raw = dict(SHAPE_32B)
        e = Engine.random(config_from_dict(raw), 7, Engine_Opts(max_ctx=8192, max_tokens=8 * 8192, max_batch=8,
                                                                dtype="bfloat16", verbose=False))
        rng = np.random.default_rng(12)
        L = raw["num_hidden_layers"]
        out = {"metric": "Qwen3-32B shape, bf16, 64 layers: a 2,048-token prompt; decoding at context 8192", "peak_source": peak_source}
        for _ in range(3):
            s = e.take_slot()
            p = rng.integers(0, raw["vocab_size"], 2048).tolist()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            e.step([StepEntry(s, p, [2047])])
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b)
            e.give_back_slot(s)
        out["prefill"] = {"tokens": 2048, "ms": round(ms, 2), "value": round(2048 / ms * 1e3),
                          "frac": round(prefill_flops(raw, L, 2048) / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
        for B in (1, 8):
            slots = [e.take_slot() for _ in range(B)]
            ctx0 = 8192 - 72
            for a0 in range(0, ctx0, 2048):  # the context, in pieces of 2,048 tokens
                n = min(2048, ctx0 - a0)
                e.step([StepEntry(s, rng.integers(0, raw["vocab_size"], n).tolist(), []) for s in slots])
            feed = rng.integers(0, raw["vocab_size"], (72, B))
            for i in range(8):
                e.step([StepEntry(s, [int(feed[i, b])], [0]) for b, s in enumerate(slots)])
            torch.cuda.synchronize()
            a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(8, 72):
                e.step([StepEntry(s, [int(feed[i, b])], [0]) for b, s in enumerate(slots)])
            b2.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b2) / 64
            out[f"decode_b{B}"] = {"ms_per_step": round(ms, 3), "value": round(B / ms * 1e3, 1), "context": 8192 - 32,
                                   "hbm_frac": round(decode_bytes(raw, L, B, 8192 - 32) / (ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4)}
            for s in slots:
                e.give_back_slot(s)
    ops.gemm_tc_check()
    ops.attention_prefill_check()
    ops.attention_decode_check()
    print(json.dumps(out))
    return 0


# --------------------------------------------------------------------------------------------------------------
# --workload tovalix: the Tovalix design beside the Qwen3 dense decoder at equal sizes
# --------------------------------------------------------------------------------------------------------------
TOVALIX_SIZES = {
    # width, ff, attention heads / kv heads / head size, recurrence heads x sizes, token input, layers
    "2048": dict(width=2048, ff=6144, heads=16, kv=8, hd=128, wkv_heads=32, wkv_dim=64, hg_heads=16, hg_dim=128, hg_v=128,
                 side=256, layers=8, vocab=32768, chunk=1024, rank=64),
    "4096": dict(width=4096, ff=12288, heads=32, kv=8, hd=128, wkv_heads=64, wkv_dim=64, hg_heads=32, hg_dim=128, hg_v=128,
                 side=256, layers=4, vocab=32768, chunk=1024, rank=128),
}


def tovalix_config(z: dict) -> dict:
    att = {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["hd"], "vdim": z["hd"], "scale": z["hd"] ** -0.5, "softcap": 30.0,
           "rot": {"dims": z["hd"], "base": 1e6}, "mask": {"size": z["chunk"]}}
    mlp = {"kind": "dense", "ff": z["ff"]}
    cycle = [("attention", att), ("wkv", {"heads": z["wkv_heads"], "dim": z["wkv_dim"], "decay_rank": z["rank"]}),
             ("hgrn2", {"heads": z["hg_heads"], "dim": z["hg_dim"], "vdim": z["hg_v"]}), ("attention", dict(att, kv_from=0))]
    layers = []
    for i in range(z["layers"]):
        kind, mixer = cycle[i % 4]
        if "kv_from" in mixer:
            mixer = dict(mixer, kv_from=i - 3)
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Tovalix", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5, "groups": 2},
            "token_side": {"dim": z["side"]}, "layers": layers}


def qwen3_config_like(z: dict) -> dict:
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=z["width"], intermediate_size=z["ff"], num_hidden_layers=z["layers"],
                num_attention_heads=z["heads"], num_key_value_heads=z["kv"], head_dim=z["hd"], vocab_size=z["vocab"],
                rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False)


def _timed(fn, flush, reps=5, inner=1):
    """Median device time of fn() in microseconds, L2 flushed before every run."""
    import torch
    times = []
    for r in range(reps + 2):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(inner):
            fn()
        b.record()
        torch.cuda.synchronize()
        if r >= 2:
            times.append(a.elapsed_time(b) * 1e3 / inner)
    return statistics.median(times)


def tovalix_kernels(z: dict, T: int, peaks: dict) -> dict:
    """Every kernel that the design adds, alone at this size for T token rows (one sequence of T tokens, or T
    sequences of one token after a context of 512), beside the like kernel of the Qwen3 decoder; microseconds,
    and the algorithmic bytes (or FLOPs) over the time as a fraction of the measured copy bandwidth (or cuBLAS rate)."""
    import torch
    from odin_infer_b200.csrc import ops
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    d, ff = z["width"], z["ff"]
    decode = T <= 64
    out = {}
    def _timed_replayed(fn, flush, reps=5, inner=20):
        """Kernels of a few rows: `inner` launches captured in a CUDA graph and replayed, so that the device's time is
        read and not the host's time to launch (their data is far smaller than L2 in any case)."""
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(inner):
                fn()
        return _timed(graph.replay, flush, reps) / inner
    timed = _timed_replayed if decode else _timed

    def note(name, us, nbytes=None, flops=None):
        rec = {"us": round(us, 1)}
        if nbytes is not None:
            rec["of_hbm"] = round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 3)
        if flops is not None:
            rec["of_bf16"] = round(flops / (us * 1e-6) / 1e12 / peaks["bf16_tflops"], 3)
        out[name] = rec

    x = torch.randn(T, d, device=dev)
    delta = torch.randn(T, d, device=dev)
    w = torch.ones(d, dtype=bf, device=dev)
    h = torch.empty(T, d, dtype=bf, device=dev)
    row_bytes = T * d * (4 + 4 + 4 + 2)
    note("norm: add + RMSNorm (Qwen3)", timed(lambda: ops.add_rmsnorm(x, delta, w, 1e-5, h), flush), row_bytes)
    note("norm: add + RMSNorm in 2 groups", timed(lambda: ops.row_update(x, delta, None, w, 1e-5, 2, h), flush), row_bytes)
    note("token input: settle + convert", timed(lambda: ops.row_update(x, delta, None, None, 0.0, 1, h, normalise=False), flush), row_bytes)
    note("token input: x += w * unit(y)", timed(lambda: ops.normed_add(x, delta, w, 1e-5), flush), T * d * 12)
    gu = torch.randn(T, 2 * ff, device=dev).to(bf)
    act = torch.empty(T, ff, dtype=bf, device=dev)
    pq = torch.tensor([0.3, -0.2], dtype=bf, device=dev)
    note("feed-forward: SwiGLU (Qwen3)", timed(lambda: ops.swiglu(gu, act), flush), T * ff * 6)
    note("feed-forward: xIELU", timed(lambda: ops.activation(gu[:, :ff], "xielu", act, pq), flush), T * ff * 4)
    sd = z["side"]
    gate = torch.randn(T, sd, device=dev)
    table = torch.randn(z["vocab"], sd * z["layers"], device=dev).to(bf)
    ids = torch.randint(0, z["vocab"], (T,), dtype=torch.int32, device=dev)
    g_out = torch.empty(T, sd, dtype=bf, device=dev)
    note("token input: gelu(gate) * table row", timed(lambda: ops.gated_lookup(gate, "gelu_tanh", table, sd, ids, g_out), flush), T * sd * 8)

    # sequences: one of T tokens (prompt) or T of one token each
    n_seq = T if decode else 1
    starts = torch.arange(0, T + 1, 1 if decode else T, dtype=torch.int32, device=dev)
    slots = torch.arange(n_seq, dtype=torch.int32, device=dev)
    seq = (torch.arange(T, dtype=torch.int32, device=dev) if decode else torch.zeros(T, dtype=torch.int32, device=dev))
    mu = torch.rand(5, d, device=dev).to(bf)
    streams = torch.empty(5, T, d, dtype=bf, device=dev)
    for name, mode, H, dk, dv in (("wkv", "bonus", z["wkv_heads"], z["wkv_dim"], z["wkv_dim"]),
                                  ("hgrn2", "gated", z["hg_heads"], z["hg_dim"], z["hg_v"])):
        n_state = H * dk * dv
        state = torch.zeros(n_seq, n_state + d, device=dev)
        q, k, g = (torch.randn(T, H * dk, device=dev) for _ in range(3))
        v, o = torch.randn(T, H * dv, device=dev), torch.empty(T, H * dv, device=dev)
        c0, c1 = torch.randn(H * dk, dtype=bf, device=dev) - 2, torch.rand(H * dk, dtype=bf, device=dev)
        nbytes = 4 * (T * H * (3 * dk + 2 * dv) + 2 * n_seq * n_state)
        flops = 5 * T * H * dk * dv
        us = timed(lambda: ops.linear_recurrence(mode, q, k if mode == "bonus" else None, g, v, c0, c1, o, state[:, :n_state],
                                                  starts, slots, n_seq, H, dk, dv), flush)
        note(f"{name}: recurrence ({H} heads of {dk} x {dv})" + (", token by token" if not decode else ""), us, nbytes)
        if not decode:
            us = timed(lambda: ops.linear_recurrence(mode, q, k if mode == "bonus" else None, g, v, c0, c1, o, state[:, :n_state],
                                                     starts, slots, n_seq, H, dk, dv, block_len=128, max_new=T), flush)
            note(f"{name}: recurrence ({H} heads of {dk} x {dv}), blocks of 128 tokens (what a prompt runs)", us,
                 nbytes + 4 * (2 * T * H * dk + 3 * (T // 128) * n_state))
            out[f"{name}: recurrence ({H} heads of {dk} x {dv}), blocks of 128 tokens (what a prompt runs)"]["gflops"] = round(flops / us / 1e3, 1)
        y = torch.empty(T, H * dv, dtype=bf, device=dev)
        wn = torch.ones(H * dv, dtype=bf, device=dev)
        note(f"{name}: head norm, weight" + (", gate" if mode == "bonus" else ""),
             timed(lambda: ops.head_unit_scale(o, wn, True, g if (mode == "bonus" and dk == dv) else None, 1e-5, y, H, dv), flush),
             T * H * dv * (4 + 2 + (4 if mode == "bonus" else 0)))
        if mode == "bonus":
            note("wkv: token shift (5 streams)", timed(lambda: ops.token_shift(h, state[:, n_state:], mu, streams, seq, starts, slots), flush),
                 T * d * 2 * 6)

    # attention: 512 tokens of context before the T rows when decoding, one prompt of T tokens else
    Hq, Hkv, hd = z["heads"], z["kv"], z["hd"]
    ctx = 512 if decode else 0
    per_seq = (ctx + 1 + 63) // 64 if decode else (T + 63) // 64
    n_pages = n_seq * per_seq
    kc = torch.randn(n_pages, Hkv, 64, hd, device=dev).to(bf)
    vc = torch.randn(n_pages, Hkv, 64, hd, device=dev).to(bf)
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev).reshape(n_seq, per_seq)
    pos = (torch.full((T,), ctx, dtype=torch.int32, device=dev) if decode else torch.arange(T, dtype=torch.int32, device=dev))
    qkv = torch.randn(T, (Hq + 2 * Hkv) * hd, device=dev).to(bf)
    bias = torch.randn((Hq + 2 * Hkv) * hd, device=dev).to(bf)
    qn = torch.ones(hd, dtype=bf, device=dev)
    cos = torch.randn(max(T, ctx + 1), hd // 2, device=dev)
    q_out = torch.empty(T, Hq * hd, dtype=bf, device=dev)
    hp_bytes = T * (Hq + 2 * Hkv) * hd * 4
    note("attention: head preparation (Qwen3)", timed(lambda: ops.head_prep(qkv, Hq, Hkv, hd, qn, qn, 1e-6, cos, cos, hd, pos, seq, bt, kc, vc, q_out=q_out), flush), hp_bytes)
    note("attention: head preparation (bias, unit norm after rotation)",
         timed(lambda: ops.head_prep(qkv, Hq, Hkv, hd, None, None, 1e-5, cos, cos, hd, pos, seq, bt, kc, vc, q_out=q_out, bias=bias,
                                      unit_norm_after=True), flush), hp_bytes)
    ao = torch.empty(T, Hq * hd, dtype=bf, device=dev)
    if decode:
        n_split = 4
        scratch = torch.empty(ops.attention_decode_scratch(T, Hq, hd, n_split), device=dev)
        kv_bytes = 2 * 2 * T * Hkv * hd * (ctx + 1)
        note("attention: decode over 512 keys (Qwen3)", timed(lambda: ops.attention_decode(q_out, ao, Hq, Hkv, hd, kc, vc, pos, seq, bt, 0, scratch, n_split), flush), kv_bytes)
        note("attention: decode over 512 keys, chunk + capped scores",
             timed(lambda: ops.attention_decode(q_out, ao, Hq, Hkv, hd, kc, vc, pos, seq, bt, 0, scratch, n_split, z["chunk"], hd ** -0.5, 30.0), flush), kv_bytes)
    else:
        lens = torch.tensor([T], dtype=torch.int32, device=dev)
        full = 4 * Hq * hd * (T * (T + 1) // 2)
        c = z["chunk"]
        inside = sum(min(c, T - a) * (min(c, T - a) + 1) // 2 for a in range(0, T, c)) * 4 * Hq * hd
        note("attention: prompt (Qwen3)", timed(lambda: ops.attention_prefill(q_out, ao, 1, T, Hq, Hkv, hd, kc, vc, starts, lens, bt, 0), flush), flops=full)
        note("attention: prompt, capped scores", timed(lambda: ops.attention_prefill(q_out, ao, 1, T, Hq, Hkv, hd, kc, vc, starts, lens, bt, 0, 0, hd ** -0.5, 30.0), flush), flops=full)
        note(f"attention: prompt, chunks of {c} + capped scores",
             timed(lambda: ops.attention_prefill(q_out, ao, 1, T, Hq, Hkv, hd, kc, vc, starts, lens, bt, 0, c, hd ** -0.5, 30.0), flush), flops=inside)
    ops.attention_prefill_check()
    ops.attention_decode_check()
    return out


def tovalix_workload(steps: int, warmup: int) -> int:
    """The Tovalix design at two sizes that resemble a real model's layers, beside the Qwen3 dense decoder of the same
    width, feed-forward size, attention heads, number of layers and vocabulary (random weights): a prompt of 2,048
    tokens in one step, decoding at batch 8 after 512-token prompts (device-timed), and every new kernel alone."""
    import torch
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.csrc import ops
    peaks, peak_source = load_peaks()
    result = {"metric": "Tovalix beside the Qwen3 dense decoder at equal sizes: prompt of 2,048 tokens, decode at batch 8 "
                        "(512-token prompts), bf16, random weights", "peak_source": peak_source, "sizes": {}}
    steps = min(steps, 64)
    for name, z in TOVALIX_SIZES.items():
        entry = {}
        for model, raw in (("tovalix", tovalix_config(z)), ("qwen3", qwen3_config_like(z))):
            need = PROMPT + warmup + steps + 72
            engine = Engine.random(config_from_dict(raw), WEIGHT_SEED, Engine_Opts(
                max_ctx=CONTEXT, max_tokens=max(8 * ((need + 63) // 64 * 64), PREFILL_TOKENS + 64), max_batch=8,
                dtype="bfloat16", verbose=False))
            ms_pf = run_prefill(engine, z["vocab"])
            tps, ms_step, _, launches = run_decode(engine, 8, steps, warmup, z["vocab"])
            entry[model] = {"layers": z["layers"], "weights_gib": round(engine.weight_bytes / 2 ** 30, 2),
                            "prefill_2048": {"ms": round(ms_pf, 3), "tokens_per_s": round(PREFILL_TOKENS / ms_pf * 1e3)},
                            "decode_b8": {"ms_per_step": round(ms_step, 4), "tokens_per_s": round(tps, 1),
                                          "weights_over_time_of_hbm": round(engine.weight_bytes / (ms_step / 1e3) / 1e9 / peaks["hbm_gbs"], 3),
                                          "launches_per_step": launches // steps}}
            engine.destroy()
            del engine
            torch.cuda.empty_cache()
        entry["kernels_prompt_2048_rows"] = tovalix_kernels(z, PREFILL_TOKENS, peaks)
        entry["kernels_decode_8_rows"] = tovalix_kernels(z, 8, peaks)
        result["sizes"][name] = entry
    ops.gemm_tc_check()
    print(json.dumps(result))
    return 0


# --------------------------------------------------------------------------------------------------------------
# --workload nufupel: the Nufupel design beside the Qwen3 dense decoder at equal sizes
# --------------------------------------------------------------------------------------------------------------
NUFUPEL_SIZES = {
    # width, heads / kv heads / head size, experts x inner (top of them per token) beside a shared expert; the dense
    # layers' and the Qwen3 decoder's inner size is what a token uses of an expert layer (top x inner + shared)
    "2048": dict(width=2048, heads=16, kv=8, hd=128, experts=32, top=4, eff=768, shared=1536, layers=8, vocab=32768,
                 window=1024),
    "4096": dict(width=4096, heads=32, kv=8, hd=128, experts=64, top=6, eff=1024, shared=2048, layers=4, vocab=32768,
                 window=1024),
}


def nufupel_config(z: dict) -> dict:
    ff = z["top"] * z["eff"] + z["shared"]
    base = {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["hd"], "vdim": z["hd"], "scale": z["hd"] ** -0.5,
            "mask": {"size": z["window"]}}
    rot = {"dims": z["hd"] // 2, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    moe = {"kind": "moe", "expert": {"ff": z["eff"]}, "router": {"experts": z["experts"], "top": z["top"]}, "shared": {"ff": z["shared"]}}
    layers = []
    for i in range(z["layers"]):
        if i % 4 == 0:
            layers.append({"type": "attention_2", "mixer": dict(base, rot=rot), "mlp": {"kind": "dense", "ff": ff} if i == 0 else moe})
        elif i % 4 == 1:
            layers.append({"type": "attention", "mixer": dict(base, mask={"size": z["window"] // 2}), "mlp": moe})
        else:
            layers.append(dict(layers[i - i % 4 + 1], weights_of=i - i % 4 + 1))
    return {"architecture": "Nufupel", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": float(z["width"]) ** 0.5}, "logit_softcap": 30.0, "layers": layers}


def nufupel_kernels(z: dict, T: int, peaks: dict) -> dict:
    """Every kernel that the design adds, alone at this size for T token rows, beside the like kernel of the Qwen3
    decoder: microseconds, and algorithmic bytes (or FLOPs) over the time as a fraction of the measured peaks."""
    import torch
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.engine import runtime as R
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    d, hd, Hq, Hkv = z["width"], z["hd"], z["heads"], z["kv"]
    E, top, eff = z["experts"], z["top"], z["eff"]
    always = z["shared"] // eff
    ff = top * eff + z["shared"]
    decode = T <= 64
    out = {}

    def replayed(fn, flush, reps=5, inner=20):
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(inner):
                fn()
        return _timed(graph.replay, flush, reps) / inner
    timed = replayed if decode else _timed

    def note(name, us, nbytes=None, flops=None):
        e = {"us": round(us, 2)}
        if nbytes is not None:
            e["of_hbm"] = round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 3)
        if flops is not None:
            e["tflops"] = round(flops / (us * 1e-6) / 1e12, 1)
            e["of_bf16"] = round(flops / (us * 1e-6) / 1e12 / peaks["bf16_tflops"], 3)
        out[name] = e
    rt = R.Runtime(dev, bf)
    torch.manual_seed(0)
    h = torch.randn(T, d, device=dev).to(bf)
    x = torch.randn(T, d, device=dev)
    w1 = torch.randn(d, device=dev)
    hb = torch.empty(T, d, dtype=bf, device=dev)
    # norm: one update against three
    d1 = torch.randn(2, T, d, device=dev)
    d2 = torch.randn(T, d, device=dev)
    note("add_rmsnorm (qwen3)", timed(lambda: ops.add_rmsnorm(x, d1, w1, 1e-6, hb), flush), nbytes=T * d * (4 * 4 + 2))
    note("add_rmsnorm, three updates", timed(lambda: ops.row_update(x, [d1, d2, d1], None, w1, 1e-6, 1, hb), flush),
         nbytes=T * d * (4 * 7 + 2))
    # gate on the heads, gated activations
    o = torch.randn(T, Hq * hd, device=dev).to(bf)
    wide = torch.randn(2 if decode else 1, T, (Hq + 2 * Hkv) * hd + Hq * hd, device=dev)
    if not decode:
        wide = wide[0].to(bf)
    g0 = (Hq + 2 * Hkv) * hd
    note("sigmoid gate per element", timed(lambda: ops.sigmoid_gate(o, wide[..., g0:], Hq, hd, False), flush),
         nbytes=T * Hq * hd * (4 + wide.element_size() * (wide.shape[0] if wide.dim() == 3 else 1)))
    note("sigmoid gate per head", timed(lambda: ops.sigmoid_gate(o, wide[..., g0:g0 + Hq], Hq, hd, True), flush), nbytes=T * Hq * hd * 4)
    gu = torch.randn(2, T, 2 * ff, device=dev) if decode else torch.randn(T, 2 * ff, device=dev).to(bf)
    act = torch.empty(T, ff, dtype=bf, device=dev)
    nb = gu.numel() * gu.element_size() + act.numel() * 2
    note("swiglu (qwen3)", timed(lambda: ops.swiglu(gu, act), flush), nbytes=nb)
    note("geglu", timed(lambda: ops.gated_activation(gu, "gelu_tanh", act), flush), nbytes=nb)
    # gate|up with the activation in the epilogue
    if not decode:
        wgu = (torch.randn(2 * ff, d, device=dev) * 0.02).to(bf)
        fl = 2.0 * T * 2 * ff * d
        note("gate|up product + swiglu epilogue (qwen3)", timed(lambda: ops.gemm_tc2_swiglu(h, wgu, act, "silu"), flush), flops=fl)
        note("gate|up product + geglu epilogue", timed(lambda: ops.gemm_tc2_swiglu(h, wgu, act, "gelu_tanh"), flush), flops=fl)
    # router and experts
    wr = (torch.randn(E, d, device=dev) / d ** 0.5).to(bf)
    ids = torch.empty(T, top + always, dtype=torch.int32, device=dev)
    wts = torch.empty(T, top + always, dtype=torch.float32, device=dev)
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    def route():   # as the feed-forward part does it: the logits of many tokens as a tensor-core product
        lg = rt.linear(h, wr, out_dtype=torch.float32) if T > 64 else None
        ops.moe_router(h, wr, None, top, always, seq, ids, wts, lg)
    note("router (logits, choice, weights)", timed(route, flush), nbytes=T * d * 2 + E * d * 2)
    n_e = E + always
    wg = (torch.randn(n_e, 2 * eff, d, device=dev) * 0.02).to(bf)
    wd = (torch.randn(n_e, d, eff, device=dev) * 0.02).to(bf)
    used = len(torch.unique(ids))
    fl = 2.0 * T * (top + always) * 3 * eff * d
    note("experts (all their launches)", timed(lambda: rt.experts(h, wg, wd, ids, wts, "silu"), flush), flops=fl,
         nbytes=used * 3 * eff * d * 2)
    out["experts (all their launches)"]["experts_used"] = used
    # the dense feed-forward of what a token uses of the experts, as the Qwen3 decoder runs it
    wgu = (torch.randn(2 * ff, d, device=dev) * 0.02).to(bf)
    wdn = (torch.randn(d, ff, device=dev) * 0.02).to(bf)
    note("dense feed-forward of equal active size (qwen3)",
         timed(lambda: rt.linear(rt.gated_linear(h, wgu, ff), wdn, out_dtype=torch.float32, may_split=True), flush),
         flops=2.0 * T * 3 * ff * d, nbytes=3 * ff * d * 2)
    # attention with and without the sink
    ctx = T if not decode else 512
    n_pages = (ctx + 63) // 64 * (1 if not decode else T) + 2
    kc = (torch.randn(n_pages, Hkv, 64, hd, device=dev) * 0.3).to(bf)
    vc = (torch.randn(n_pages, Hkv, 64, hd, device=dev) * 0.3).to(bf)
    q = (torch.randn(T, Hq * hd, device=dev) * 0.3).to(bf)
    ao = torch.empty(T, Hq * hd, dtype=bf, device=dev)
    sink = torch.randn(Hq, device=dev)
    if decode:
        per_seq = (ctx + 63) // 64
        bt = torch.arange(T * per_seq, dtype=torch.int32, device=dev).reshape(T, per_seq).contiguous()
        pos = torch.full((T,), ctx - 1, dtype=torch.int32, device=dev)
        sq = torch.arange(T, dtype=torch.int32, device=dev)
        n_split = R.decode_key_splits(T, Hkv, ctx)
        scratch = torch.empty(ops.attention_decode_scratch(T, Hq, hd, n_split), dtype=torch.float32, device=dev)
        nb = T * ctx * Hkv * hd * 2 * 2
        for name, sk in (("decode attention (qwen3)", None), ("decode attention with a sink", sink)):
            note(name, timed(lambda: ops.attention_decode(q, ao, Hq, Hkv, hd, kc, vc, pos, sq, bt, 0, scratch, n_split, 0, hd ** -0.5, 0.0, sk), flush), nbytes=nb)
    else:
        bt = torch.arange((ctx + 63) // 64, dtype=torch.int32, device=dev).reshape(1, -1).contiguous()
        starts = torch.tensor([0, T], dtype=torch.int32, device=dev)
        lens = torch.tensor([T], dtype=torch.int32, device=dev)
        fl = 4.0 * Hq * hd * (T * (T + 1) // 2)
        w = z["window"]
        inside = 4.0 * Hq * hd * (w * (w + 1) // 2 + (T - w) * w) if T > w else fl
        note("prompt attention (qwen3)", timed(lambda: ops.attention_prefill(q, ao, 1, T, Hq, Hkv, hd, kc, vc, starts, lens, bt, 0, 0, hd ** -0.5, 0.0), flush), flops=fl)
        note("prompt attention with a sink", timed(lambda: ops.attention_prefill(q, ao, 1, T, Hq, Hkv, hd, kc, vc, starts, lens, bt, 0, 0, hd ** -0.5, 0.0, sink), flush), flops=fl)
        note("prompt attention with a sink and the window", timed(lambda: ops.attention_prefill(q, ao, 1, T, Hq, Hkv, hd, kc, vc, starts, lens, bt, w, 0, hd ** -0.5, 0.0, sink), flush), flops=inside)
    torch.cuda.synchronize()
    ops.attention_prefill_check()
    ops.attention_decode_check()
    ops.moe_tc_check()
    return out


def nufupel_workload(steps: int, warmup: int) -> int:
    """The Nufupel design at two sizes that resemble a real model's layers, beside the Qwen3 dense decoder of the same
    width, attention heads, number of layers and vocabulary, whose feed-forward has the size that a token uses of an
    expert layer (random weights): a prompt of 2,048 tokens in one step, decoding at batch 8 after 512-token prompts
    (device-timed), and every new kernel alone."""
    import torch
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.csrc import ops
    peaks, peak_source = load_peaks()
    result = {"metric": "Nufupel beside the Qwen3 dense decoder at equal sizes: prompt of 2,048 tokens, decode at batch 8 "
                        "(512-token prompts), bf16, random weights", "peak_source": peak_source, "sizes": {}}
    steps = min(steps, 64)
    for name, z in NUFUPEL_SIZES.items():
        entry = {}
        ff = z["top"] * z["eff"] + z["shared"]
        like = dict(z, ff=ff)
        for model, raw in (("nufupel", nufupel_config(z)), ("qwen3", qwen3_config_like(like))):
            need = PROMPT + warmup + steps + 72
            engine = Engine.random(config_from_dict(raw), WEIGHT_SEED, Engine_Opts(
                max_ctx=CONTEXT, max_tokens=max(8 * ((need + 63) // 64 * 64), PREFILL_TOKENS + 64), max_batch=8,
                dtype="bfloat16", verbose=False))
            ms_pf = run_prefill(engine, z["vocab"])
            tps, ms_step, _, launches = run_decode(engine, 8, steps, warmup, z["vocab"])
            entry[model] = {"layers": z["layers"], "weights_gib": round(engine.weight_bytes / 2 ** 30, 2),
                            "prefill_2048": {"ms": round(ms_pf, 3), "tokens_per_s": round(PREFILL_TOKENS / ms_pf * 1e3)},
                            "decode_b8": {"ms_per_step": round(ms_step, 4), "tokens_per_s": round(tps, 1),
                                          "launches_per_step": launches // steps}}
            engine.destroy()
            del engine
            torch.cuda.empty_cache()
        entry["kernels_prompt_2048_rows"] = nufupel_kernels(z, PREFILL_TOKENS, peaks)
        entry["kernels_decode_8_rows"] = nufupel_kernels(z, 8, peaks)
        result["sizes"][name] = entry
    ops.gemm_tc_check()
    print(json.dumps(result))
    return 0


# --------------------------------------------------------------------------------------------------------------
# --workload nikonex: the Nikonex design beside the Nufupel design (the closest: parallel blocks, windows, experts)
# --------------------------------------------------------------------------------------------------------------
NIKONEX_SIZES = {
    # the Nufupel sizes' width, experts, layers and vocabulary; latent attention whose cached row is 128 elements
    # (kv_rank + rot_dim), retention heads of 128 x 128, experts in groups
    "2048": dict(NUFUPEL_SIZES["2048"], lat_heads=16, lat_dim=64, rot_dim=64, lat_v=64, q_rank=512, kv_rank=64,
                 ret_heads=16, ret_dim=128, ret_v=128, groups=4, keep=2),
    "4096": dict(NUFUPEL_SIZES["4096"], lat_heads=16, lat_dim=128, rot_dim=64, lat_v=128, q_rank=768, kv_rank=64,
                 ret_heads=32, ret_dim=128, ret_v=128, groups=8, keep=4),
}


def nikonex_config(z: dict) -> dict:
    lat = {"heads": z["lat_heads"], "dim": z["lat_dim"], "rot_dim": z["rot_dim"], "vdim": z["lat_v"], "q_rank": z["q_rank"],
           "kv_rank": z["kv_rank"], "scale": (z["lat_dim"] + z["rot_dim"]) ** -0.5, "mask": {"size": z["window"]},
           "rot": {"dims": z["rot_dim"], "base": 500000.0,
                   "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}
    ret = {"heads": z["ret_heads"], "dim": z["ret_dim"], "vdim": z["ret_v"],
           "decay": [math.exp(-1.0 / (8.0 * 2.0 ** (8.0 * i / max(z["ret_heads"] - 1, 1)))) for i in range(z["ret_heads"])],  # memories of 8 to 2,048 tokens
           "rot": {"dims": z["ret_dim"], "base": 500000.0}}
    moe = {"kind": "moe", "expert": {"ff": z["eff"]}, "shared": {"ff": z["shared"]},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 2.5, "groups": {"count": z["groups"], "keep": z["keep"]}}}
    layers = [{"type": "retention" if i % 2 == 0 else "latent_attention", "mixer": ret if i % 2 == 0 else lat, "mlp": moe}
              for i in range(z["layers"])]
    return {"architecture": "Nikonex", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.6,
            "layers": layers}


def nikonex_kernels(z: dict, T: int, peaks: dict) -> dict:
    """Every kernel that the design adds (or runs with options of its own), alone at this size for T token rows (one
    prompt of T tokens, or T sequences of one token after 512), beside the like kernel of the closest existing path:
    microseconds, and algorithmic bytes (or FLOPs) over the time as a fraction of the measured peaks."""
    import torch
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.engine import runtime as R
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    d, E, top, eff = z["width"], z["experts"], z["top"], z["eff"]
    H, e, r, ev, qr, kvr = z["lat_heads"], z["lat_dim"], z["rot_dim"], z["lat_v"], z["q_rank"], z["kv_rank"]
    L = kvr + r
    always = z["shared"] // eff
    decode = T <= 64
    out = {}

    def replayed(fn, flush, reps=5, inner=20):
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(inner):
                fn()
        return _timed(graph.replay, flush, reps) / inner
    timed = replayed if decode else _timed

    def note(name, us, nbytes=None, flops=None, **more):
        rec = {"us": round(us, 2)}
        if nbytes is not None:
            rec["of_hbm"] = round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 3)
        if flops is not None:
            rec["tflops"] = round(flops / (us * 1e-6) / 1e12, 2)
            rec["of_bf16"] = round(flops / (us * 1e-6) / 1e12 / peaks["bf16_tflops"], 3)
        rec.update(more)
        out[name] = rec
    rt = R.Runtime(dev, bf)
    torch.manual_seed(0)
    h = torch.randn(T, d, device=dev).to(bf)
    x = torch.randn(T, d, device=dev)
    w1 = torch.randn(d, device=dev).to(bf)
    hb = torch.empty(T, d, dtype=bf, device=dev)
    # norms: two updates with and without the factor; the second norm of the same x
    d1, d2 = torch.randn(T, d, device=dev), torch.randn(T, d, device=dev)
    nb = T * d * (4 * 4 + 2)
    note("add + RMSNorm of two updates (nufupel)", timed(lambda: ops.row_update(x, [d1, d2], None, w1, 1e-6, 1, hb), flush), nbytes=nb)
    note("add + RMSNorm of two updates times a factor", timed(lambda: ops.row_update(x, [d1, d2], None, w1, 1e-6, 1, hb, scale=0.6), flush), nbytes=nb)
    note("the second norm of the same x", timed(lambda: ops.row_update(x, None, None, w1, 1e-6, 1, hb), flush), nbytes=T * d * 6)
    w2, hb2 = torch.randn(d, device=dev).to(bf), torch.empty(T, d, dtype=bf, device=dev)
    note("add + both norms of two updates times a factor, one kernel",
         timed(lambda: ops.row_update(x, [d1, d2], None, w1, 1e-6, 1, hb, scale=0.6, weight2=w2, out2=hb2), flush), nbytes=nb + T * d * 2)
    # sequences and pages: one prompt of T tokens, or T sequences of one token after 512
    ctx = 512 if decode else 0
    n_seq = T if decode else 1
    per_seq = (ctx + 1 + 63) // 64 if decode else (T + 63) // 64
    n_pages = n_seq * per_seq
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev).reshape(n_seq, per_seq).contiguous()
    pos = torch.full((T,), ctx, dtype=torch.int32, device=dev) if decode else torch.arange(T, dtype=torch.int32, device=dev)
    seq = torch.arange(T, dtype=torch.int32, device=dev) if decode else torch.zeros(T, dtype=torch.int32, device=dev)
    starts = torch.arange(0, T + 1, 1 if decode else T, dtype=torch.int32, device=dev)
    slots = torch.arange(n_seq, dtype=torch.int32, device=dev)
    # preparation of rows: the latent one beside the heads' one
    Hq, Hkv, hd = z["heads"], z["kv"], z["hd"]
    down = torch.randn(T, qr + L, device=dev).to(bf)
    cq = torch.empty(T, qr, dtype=bf, device=dev)
    qn, cn = torch.ones(qr, dtype=bf, device=dev), torch.ones(kvr, dtype=bf, device=dev)
    cos, sin = torch.randn(max(T, ctx + 1), r // 2, device=dev), torch.randn(max(T, ctx + 1), r // 2, device=dev)
    rows = (torch.randn(n_pages, 1, 64, L, device=dev) * 0.3).to(bf)
    note("latent preparation (two norms, rotation, cache row)",
         timed(lambda: ops.latent_prep(down, qr, kvr, r, True, qn, cn, 1e-6, cq, cos, sin, pos, seq, bt, rows), flush), nbytes=T * (qr + L) * 4)
    kc = (torch.randn(n_pages, Hkv, 64, hd, device=dev) * 0.3).to(bf)
    vc = (torch.randn(n_pages, Hkv, 64, hd, device=dev) * 0.3).to(bf)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * hd, device=dev).to(bf)
    hn = torch.ones(hd, dtype=bf, device=dev)
    ch = torch.randn(max(T, ctx + 1), hd // 2, device=dev)
    q_out = torch.empty(T, Hq * hd, dtype=bf, device=dev)
    note("head preparation (nufupel)", timed(lambda: ops.head_prep(qkv, Hq, Hkv, hd, hn, hn, 1e-6, ch, ch, hd, pos, seq, bt, kc, vc, q_out=q_out), flush),
         nbytes=T * (Hq + 2 * Hkv) * hd * 4)
    # the products per head around attention, and the queries' rotation into the wide row
    q = (torch.randn(T, H * (e + r), device=dev) * 0.3).to(bf)
    w_uk = (torch.randn(H, e, kvr, device=dev) / e ** 0.5).to(bf)
    w_uv = (torch.randn(H, kvr, ev, device=dev) / kvr ** 0.5).to(bf)
    qf = torch.empty(T, H * L, dtype=bf, device=dev)
    note("queries onto the latent, a product per head", timed(lambda: ops.heads_linear(q, e + r, w_uk, qf, L), flush),
         flops=2.0 * T * H * e * kvr, nbytes=T * H * (e + kvr) * 2 + w_uk.numel() * 2)
    note("queries' rotated part into the wide row", timed(lambda: ops.rope_heads(q[:, e:], e + r, qf[:, kvr:], L, H, r, r, True, cos, sin, pos), flush),
         nbytes=T * H * r * 4)
    o = torch.empty(T, H * L, dtype=bf, device=dev)
    ov = torch.empty(T, H * ev, dtype=bf, device=dev)
    note("values from the latent, a product per head", timed(lambda: ops.heads_linear(o, L, w_uv, ov, ev), flush),
         flops=2.0 * T * H * kvr * ev, nbytes=T * H * (kvr + ev) * 2 + w_uv.numel() * 2)
    # attention: every head over one shared row of L elements, beside grouped-query attention
    win = z["window"]
    if decode:
        for name, qq, oo, nq, nkv, dim, k_, v_ in (("decode attention over 512 keys (nufupel)", q_out, torch.empty_like(q_out), Hq, Hkv, hd, kc, vc),
                                                    ("decode attention over 512 shared rows", qf, o, H, 1, L, rows, rows)):
            n_split = R.decode_key_splits(T, nkv, ctx + 1)
            scratch = torch.empty(ops.attention_decode_scratch(T, nq, dim, n_split), dtype=torch.float32, device=dev)
            nbytes = T * (ctx + 1) * nkv * dim * 2 * (2 if k_ is not v_ else 1)
            note(name, timed(lambda: ops.attention_decode(qq, oo, nq, nkv, dim, k_, v_, pos, seq, bt, win, scratch, n_split, 0, dim ** -0.5, 0.0), flush), nbytes=nbytes)
    else:
        lens = torch.tensor([T], dtype=torch.int32, device=dev)
        pairs_seen = win * (win + 1) // 2 + (T - win) * win if T > win else T * (T + 1) // 2
        note("prompt attention in the window (nufupel)",
             timed(lambda: ops.attention_prefill(q_out, torch.empty_like(q_out), 1, T, Hq, Hkv, hd, kc, vc, starts, lens, bt, win, 0, hd ** -0.5, 0.0), flush),
             flops=4.0 * Hq * hd * pairs_seen)
        note("prompt attention in the window over shared rows",
             timed(lambda: ops.attention_prefill(qf, o, 1, T, H, 1, L, rows, rows, starts, lens, bt, win, 0, L ** -0.5, 0.0), flush),
             flops=4.0 * H * L * pairs_seen)
    # retention's recurrence beside the gated recurrence (Tovalix) at equal heads and sizes
    RH, dk, dv = z["ret_heads"], z["ret_dim"], z["ret_v"]
    n_state = RH * dk * dv
    state = torch.zeros(n_seq, n_state, device=dev)
    qkvg = torch.randn(T, RH * (2 * dk + 2 * dv), device=dev)
    rq, rk, rv, rg = qkvg[:, :RH * dk], qkvg[:, RH * dk:2 * RH * dk], qkvg[:, 2 * RH * dk:2 * RH * dk + RH * dv], qkvg[:, 2 * RH * dk + RH * dv:]
    ro = torch.empty(T, RH * dv, device=dev)
    decay = torch.full((RH,), 0.99, device=dev)
    c0, c1 = torch.randn(RH * dk, device=dev) - 2, torch.rand(RH * dk, device=dev)
    cr, sr = torch.randn(max(T, ctx + 1), dk // 2, device=dev), torch.randn(max(T, ctx + 1), dk // 2, device=dev)
    both = qkvg[:, :2 * RH * dk]
    note("rotation of q and k in place, k scaled", timed(lambda: ops.rope_heads(both, dk, both, dk, 2 * RH, dk, dk, False, cr, sr, pos, scale=dk ** -0.5, scale_from_head=RH), flush),
         nbytes=T * 2 * RH * dk * 8)
    qkvg.normal_()
    blocks = dict(block_len=128, max_new=T) if not decode else {}
    nbytes = 4 * (T * RH * (2 * dk + 2 * dv) + 2 * n_seq * n_state)
    if not decode:
        nbytes += 4 * (2 * T * RH * dk + 3 * (T // 128) * n_state)
    tag = " in blocks of 128 tokens" if not decode else ""
    note(f"recurrence with a forget gate ({RH} heads of {dk} x {dv}; tovalix)" + tag,
         timed(lambda: ops.linear_recurrence("gated", rq, None, rk, rv, c0, c1, ro, state, starts, slots, n_seq, RH, dk, dv, **blocks), flush),
         nbytes=nbytes - 4 * T * RH * dk)
    note(f"recurrence with a fixed decay ({RH} heads of {dk} x {dv})" + tag,
         timed(lambda: ops.linear_recurrence("fixed", rq, rk, None, rv, decay, decay, ro, state, starts, slots, n_seq, RH, dk, dv, **blocks), flush),
         nbytes=nbytes)
    y = torch.empty(T, RH * dv, dtype=bf, device=dev)
    wn = torch.ones(dv, dtype=bf, device=dev)
    note("heads' norm with a weight (tovalix)", timed(lambda: ops.head_unit_scale(ro, wn, False, None, 1e-5, y, RH, dv), flush), nbytes=T * RH * dv * 6)
    note("heads' unit norm times silu(gate)", timed(lambda: ops.head_unit_scale(ro, None, False, rg, 1e-5, y, RH, dv), flush), nbytes=T * RH * dv * 10)
    # router: softmax over the chosen beside sigmoid scores in groups with the shared expert's gate as one more row
    wr = (torch.randn(E + 1, d, device=dev) / d ** 0.5).to(bf)
    ids = torch.empty(T, top + always, dtype=torch.int32, device=dev)
    wts = torch.empty(T, top + always, dtype=torch.float32, device=dev)

    def route(score, **kw):
        w = wr if kw.get("gate_row") else wr[:E]
        lg = rt.linear(h, w, out_dtype=torch.float32) if T > 64 else None
        ops.moe_router(h, w, None, top, always, seq, ids, wts, lg, score=score, **kw)
    rb = T * d * 2 + E * d * 2
    note("router, softmax of the chosen (nufupel)", timed(lambda: route("softmax_of_chosen"), flush), nbytes=rb)
    note("router, sigmoid scores in groups, the shared expert's gate",
         timed(lambda: route("sigmoid_in_groups", groups=z["groups"], keep=z["keep"], route_scale=2.5, gate_row=True), flush), nbytes=rb)
    # experts: relu^2 without a gate matrix beside silu with one
    n_e = E + always
    used = len(torch.unique(ids))
    wg = (torch.randn(n_e, 2 * eff, d, device=dev) * 0.02).to(bf)
    wd = (torch.randn(n_e, d, eff, device=dev) * 0.02).to(bf)
    note("experts with a gate matrix, silu (nufupel; all their launches)", timed(lambda: rt.experts(h, wg, wd, ids, wts, "silu"), flush),
         flops=2.0 * T * (top + always) * 3 * eff * d, nbytes=used * 3 * eff * d * 2, experts_used=used)
    wu = wg[:, :eff].contiguous()
    note("experts without one, relu squared (all their launches)", timed(lambda: rt.experts(h, wu, wd, ids, wts, "relu2", gated=False), flush),
         flops=2.0 * T * (top + always) * 2 * eff * d, nbytes=used * 2 * eff * d * 2, experts_used=used)
    torch.cuda.synchronize()
    ops.attention_prefill_check()
    ops.attention_decode_check()
    ops.moe_tc_check()
    return out


def nikonex_workload(steps: int, warmup: int) -> int:
    """The Nikonex design at two sizes that resemble a real model's layers, beside the Nufupel design of the same
    width, layers, vocabulary, window and experts (random weights): a prompt of 2,048 tokens in one step, decoding at
    batch 8 after 512-token prompts (device-timed), and every kernel of the design alone beside its like."""
    import torch
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.csrc import ops
    peaks, peak_source = load_peaks()
    result = {"metric": "Nikonex beside Nufupel at equal sizes: prompt of 2,048 tokens, decode at batch 8 (512-token prompts), "
                        "bf16, random weights", "peak_source": peak_source, "sizes": {}}
    steps = min(steps, 64)
    for name, z in NIKONEX_SIZES.items():
        entry = {}
        for model, raw in (("nikonex", nikonex_config(z)), ("nufupel", nufupel_config(z))):
            need = PROMPT + warmup + steps + 72
            engine = Engine.random(config_from_dict(raw), WEIGHT_SEED, Engine_Opts(
                max_ctx=CONTEXT, max_tokens=max(8 * ((need + 63) // 64 * 64), PREFILL_TOKENS + 64), max_batch=8,
                dtype="bfloat16", verbose=False))
            ms_pf = run_prefill(engine, z["vocab"])
            tps, ms_step, _, launches = run_decode(engine, 8, steps, warmup, z["vocab"])
            entry[model] = {"layers": z["layers"], "weights_gib": round(engine.weight_bytes / 2 ** 30, 2),
                            "prefill_2048": {"ms": round(ms_pf, 3), "tokens_per_s": round(PREFILL_TOKENS / ms_pf * 1e3)},
                            "decode_b8": {"ms_per_step": round(ms_step, 4), "tokens_per_s": round(tps, 1),
                                          "launches_per_step": launches // steps}}
            engine.destroy()
            del engine
            torch.cuda.empty_cache()
        entry["kernels_prompt_2048_rows"] = nikonex_kernels(z, PREFILL_TOKENS, peaks)
        entry["kernels_decode_8_rows"] = nikonex_kernels(z, 8, peaks)
        result["sizes"][name] = entry
    ops.gemm_tc_check()
    print(json.dumps(result))
    return 0


# --------------------------------------------------------------------------------------------------------------
# --workload meropel: the Meropel design beside the Nikonex design (the closest: recurrences, attention, experts in groups)
# --------------------------------------------------------------------------------------------------------------
MEROPEL_SIZES = {
    # the Nikonex sizes' width, layers, vocabulary and experts; attention of 16 query heads on 8 kv heads of 128 (the
    # tensor-core kernels' head size), a selective scan of twice the width with 16 states per channel, a recurrence over
    # heads of 128 states x 64 (twice the width in all), gated linear attention with keys of half and values of the width
    "2048": dict(NIKONEX_SIZES["2048"], scan_inner=4096, scan_state=16, dt_rank=128, ssd_heads=64, ssd_dim=64, ssd_state=128,
                 ssd_groups=8, gla_heads=8, gla_dim=128, gla_v=256, identity=4),
    "4096": dict(NIKONEX_SIZES["4096"], scan_inner=8192, scan_state=16, dt_rank=256, ssd_heads=128, ssd_dim=64, ssd_state=128,
                 ssd_groups=8, gla_heads=16, gla_dim=128, gla_v=256, identity=8),
}


def meropel_config(z: dict) -> dict:
    att = {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["hd"], "vdim": z["hd"], "scale": z["hd"] ** -0.5}
    par = {"left": dict(att, rot={"dims": z["hd"] // 2, "base": 10000.0}), "left_scale": 0.7, "right_scale": 0.6,
           "right": {"inner": z["scan_inner"], "state": z["scan_state"], "dt_rank": z["dt_rank"], "conv": 4}}
    par2 = {"left": dict(att, rot={"dims": z["hd"], "base": 1000000.0}),
            "right": {"heads": z["ssd_heads"], "vdim": z["ssd_dim"], "state": z["ssd_state"], "groups": z["ssd_groups"],
                      "norm_groups": z["ssd_groups"], "conv": 4}}
    gla = {"heads": z["gla_heads"], "dim": z["gla_dim"], "vdim": z["gla_v"], "tau": 8.0}
    moe = {"kind": "moe", "expert": {"ff": z["eff"]}, "shared": {"ff": z["shared"]},
           "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"], "scale": 2.5,
                      "groups": {"count": z["groups"], "keep": z["keep"]}}}
    kinds = [("parallel", par), ("parallel_2", par2), ("gla", gla)]
    layers = [{"type": kinds[i % 3][0], "mixer": kinds[i % 3][1], "mlp": moe} for i in range(z["layers"])]
    return {"architecture": "Meropel", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "logit_scale": 0.5,
            "embedding": {"bigram": {"buckets": 99991, "mul_prev": 131, "mul_cur": 31}}, "layers": layers}


def meropel_kernels(z: dict, T: int, peaks: dict) -> dict:
    """Every kernel that the design adds (or runs with options of its own), alone at this size for T token rows (one
    prompt of T tokens, or T sequences of one token after 512), beside the like kernel of the closest existing path:
    microseconds, and algorithmic bytes (or FLOPs) over the time as a fraction of the measured peaks."""
    import torch
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.engine import runtime as R
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    d, E, top, eff, ident = z["width"], z["experts"], z["top"], z["eff"], z["identity"]
    always = z["shared"] // eff
    decode = T <= 64
    out = {}

    def replayed(fn, flush, reps=5, inner=20):
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(inner):
                fn()
        return _timed(graph.replay, flush, reps) / inner
    timed = replayed if decode else _timed

    def note(name, us, nbytes=None, flops=None, **more):
        rec = {"us": round(us, 2)}
        if nbytes is not None:
            rec["of_hbm"] = round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 3)
        if flops is not None:
            rec["tflops"] = round(flops / (us * 1e-6) / 1e12, 2)
        rec.update(more)
        out[name] = rec
    rt = R.Runtime(dev, bf)
    torch.manual_seed(0)
    ctx = 512 if decode else 0
    n_seq = T if decode else 1
    per_seq = (ctx + 1 + 63) // 64 if decode else (T + 63) // 64
    n_pages = n_seq * per_seq
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev).reshape(n_seq, per_seq).contiguous()
    pos = torch.full((T,), ctx, dtype=torch.int32, device=dev) if decode else torch.arange(T, dtype=torch.int32, device=dev)
    seq = torch.arange(T, dtype=torch.int32, device=dev) if decode else torch.zeros(T, dtype=torch.int32, device=dev)
    starts = torch.arange(0, T + 1, 1 if decode else T, dtype=torch.int32, device=dev)
    slots = torch.arange(n_seq, dtype=torch.int32, device=dev)
    h = torch.randn(T, d, device=dev).to(bf)
    x = torch.randn(T, d, device=dev)
    w1, w2 = torch.randn(d, device=dev).to(bf), torch.randn(d, device=dev).to(bf)
    hb = torch.empty(T, d, dtype=bf, device=dev)
    # the residual stream: two terms, the update's own norm, the add, the next norm, beside the add of two updates and a norm
    d1, d2 = torch.randn(T, d, device=dev), torch.randn(T, d, device=dev)
    nb = T * d * (4 * 4 + 2)
    note("add + RMSNorm of two updates (nikonex)", timed(lambda: ops.row_update(x, [d1, d2], None, w1, 1e-6, 1, hb), flush), nbytes=nb)
    note("two terms with factors, their norm, the add, the next norm", timed(
        lambda: ops.combine_add(x, [ops.Term(d1, 0.7), ops.Term(d2, 0.6)], w2, 1e-6, w1, 1e-6, hb), flush), nbytes=nb)
    note("two terms each with a norm of its own, their norm, the add, the next norm", timed(
        lambda: ops.combine_add(x, [ops.Term(d1, 0.5, None, w1, 1e-6), ops.Term(d2, 0.5, None, w2, 1e-6)], w2, 1e-6, w1, 1e-6, hb), flush), nbytes=nb)
    # the embedding: a row of the token table, beside that plus a row of the pair table and the token before
    V, buckets = z["vocab"], 99991
    table, pairs = torch.randn(V, d, device=dev).to(bf), torch.randn(buckets + 1, d, device=dev).to(bf)
    tok = torch.randint(0, V, (T,), dtype=torch.int32, device=dev)
    before = torch.zeros(n_seq, 64, dtype=torch.int32, device=dev)
    note("embedding (nikonex)", timed(lambda: ops.embed(table, tok, x), flush), nbytes=T * d * 6)
    note("embedding plus the row of the pair (token before, token), with its memory", timed(
        lambda: ops.embed_pair(table, pairs, tok, seq, starts, slots, before, n_seq, buckets, 131, 31, x, single_rows=decode), flush), nbytes=T * d * 8)
    # head preparation: biases, the norm over the whole projection, rotation in pairs, beside the per-head norm
    Hq, Hkv, hd = z["heads"], z["kv"], z["hd"]
    kc = (torch.randn(n_pages, Hkv, 64, hd, device=dev) * 0.3).to(bf)
    vc = (torch.randn(n_pages, Hkv, 64, hd, device=dev) * 0.3).to(bf)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * hd, device=dev).to(bf)
    bias = torch.randn((Hq + 2 * Hkv) * hd, device=dev).to(bf)
    hn, qn, kn = torch.ones(hd, dtype=bf, device=dev), torch.ones(Hq * hd, dtype=bf, device=dev), torch.ones(Hkv * hd, dtype=bf, device=dev)
    ch = torch.randn(max(T, ctx + 1), hd // 2, device=dev)
    q_out = torch.empty(T, Hq * hd, dtype=bf, device=dev)
    hb_ = T * (Hq + 2 * Hkv) * hd * 4
    note("head preparation with a norm per head (nikonex's neighbour nufupel)", timed(
        lambda: ops.head_prep(qkv, Hq, Hkv, hd, hn, hn, 1e-6, ch, ch, hd, pos, seq, bt, kc, vc, q_out=q_out), flush), nbytes=hb_)
    note("head preparation with biases and a unit norm after the rotation (tovalix)", timed(
        lambda: ops.head_prep(qkv, Hq, Hkv, hd, None, None, 1e-6, ch, ch, hd, pos, seq, bt, kc, vc, q_out=q_out, bias=bias, unit_norm_after=True), flush), nbytes=hb_)
    note("head preparation with biases, the norm over the whole projection, rotation in pairs", timed(
        lambda: ops.head_prep(qkv, Hq, Hkv, hd, qn, kn, 1e-6, ch, ch, hd, pos, seq, bt, kc, vc, q_out=q_out, bias=bias, whole_norm=True, pairs=True), flush), nbytes=hb_)
    # the causal convolution with its memory
    C, taps = z["scan_inner"], 4
    xz = torch.randn(T, 2 * C, device=dev).to(bf)
    cw, cb = torch.randn(C, taps, device=dev).to(bf), torch.randn(C, device=dev).to(bf)
    cstate = torch.zeros(n_seq, (taps - 1) * C, device=dev)
    xc = torch.empty(T, C, dtype=bf, device=dev)
    note(f"causal convolution of {taps} taps over {C} channels with SiLU, and its memory", timed(
        lambda: ops.causal_conv(xz[:, :C], cw, cb, True, cstate, seq, starts, slots, n_seq, xc, single_rows=decode), flush),
        nbytes=T * C * 4 + 2 * n_seq * (taps - 1) * C * 4)
    # the recurrences: retention's (nikonex) beside the three of this design, decoding and a prompt
    RH, dk, dv = z["ret_heads"], z["ret_dim"], z["ret_v"]
    blocks = dict(block_len=128, max_new=T) if not decode else {}
    tag = " in blocks of 128 tokens" if not decode else ""

    def rec_bytes(H_, dk_, dv_, qk_cols):
        nbytes = 4 * (T * (qk_cols + 2 * H_ * dv_) + 2 * n_seq * H_ * dk_ * dv_)
        if not decode:
            nbytes += 4 * (2 * T * H_ * dk_ + 3 * (T // 128) * H_ * dk_ * dv_)
        return nbytes
    state = torch.zeros(n_seq, RH * dk * dv, device=dev)
    qkvg = torch.randn(T, RH * (2 * dk + 2 * dv), device=dev)
    rq, rk, rv = qkvg[:, :RH * dk], qkvg[:, RH * dk:2 * RH * dk], qkvg[:, 2 * RH * dk:2 * RH * dk + RH * dv]
    ro = torch.empty(T, RH * dv, device=dev)
    decay = torch.full((RH,), 0.99, device=dev)
    note(f"recurrence with a fixed decay ({RH} heads of {dk} x {dv}; nikonex)" + tag, timed(
        lambda: ops.linear_recurrence("fixed", rq, rk, None, rv, decay, decay, ro, state, starts, slots, n_seq, RH, dk, dv, **blocks), flush),
        nbytes=rec_bytes(RH, dk, dv, 2 * RH * dk))
    GH, gk, gv = z["gla_heads"], z["gla_dim"], z["gla_v"]
    gstate = torch.zeros(n_seq, GH * gk * gv, device=dev)
    gq, gkk, graw = (torch.randn(T, GH * gk, device=dev) for _ in range(3))
    gvv, go = torch.randn(T, GH * gv, device=dev), torch.empty(T, GH * gv, device=dev)
    gb, gt = torch.randn(GH * gk, device=dev) + 2, torch.full((GH * gk,), 1 / 8.0, device=dev)
    note(f"gated linear attention's recurrence ({GH} heads of {gk} x {gv})" + tag, timed(
        lambda: ops.linear_recurrence("gla", gq, gkk, graw, gvv, gb, gt, go, gstate, starts, slots, n_seq, GH, gk, gv, q_scale=gk ** -0.5, **blocks), flush),
        nbytes=rec_bytes(GH, gk, gv, 3 * GH * gk))
    SH, sp, sn, sg = z["ssd_heads"], z["ssd_dim"], z["ssd_state"], z["ssd_groups"]
    sstate = torch.zeros(n_seq, SH * sn * sp, device=dev)
    xbc = torch.randn(T, SH * sp + 2 * sg * sn, device=dev)
    sx, sB, sC = xbc[:, :SH * sp], xbc[:, SH * sp:SH * sp + sg * sn], xbc[:, SH * sp + sg * sn:]
    sdt, so = torch.randn(T, SH, device=dev), torch.empty(T, SH * sp, device=dev)
    sa, sbias = torch.randn(SH, device=dev) * 0.5, torch.randn(SH, device=dev) - 2
    note(f"state-space recurrence over heads ({SH} heads of {sn} x {sp}, {sg} groups)" + tag, timed(
        lambda: ops.linear_recurrence("ssd", sC, sB, sdt, sx, sa, sbias, so, sstate, starts, slots, n_seq, SH, sn, sp, heads_per_group=SH // sg, **blocks), flush),
        nbytes=rec_bytes(SH, sn, sp, 2 * sg * sn))
    inner, N = z["scan_inner"], z["scan_state"]
    cst = torch.zeros(n_seq, inner * N, device=dev)
    dt = torch.randn(T, inner, device=dev)
    bc = torch.randn(T, 2 * N, device=dev)
    a_log, dd, dtb = torch.randn(inner, N, device=dev) * 0.5, torch.randn(inner, device=dev), torch.randn(inner, device=dev) - 2
    yb = torch.empty(T, inner, dtype=bf, device=dev)
    note(f"selective scan ({inner} channels of {N} states) with skip and gate" + tag, timed(
        lambda: ops.selective_scan(xc, dt, dtb, bc[:, :N], bc[:, N:], a_log, dd, xz[:, C:], cst, yb, starts, slots, n_seq, **blocks), flush),
        nbytes=T * inner * (2 + 4 + 2 + 2) + T * 2 * N * 4 + 2 * n_seq * inner * N * 4 + inner * N * 4,
        flops=T * inner * N * 4.0)
    # what follows a recurrence: the heads' norm with a weight and a gate, beside skip, gate and a norm in groups
    y = torch.empty(T, RH * dv, dtype=bf, device=dev)
    rg = qkvg[:, 2 * RH * dk + RH * dv:]
    note("heads' unit norm times silu(gate) (nikonex)", timed(lambda: ops.head_unit_scale(ro, None, False, rg, 1e-5, y, RH, dv), flush), nbytes=T * RH * dv * 10)
    wv = torch.ones(gv, dtype=bf, device=dev)
    gg, gy = torch.randn(T, GH * gv, device=dev), torch.empty(T, GH * gv, dtype=bf, device=dev)
    note("heads' norm with a shared weight times silu(gate)", timed(lambda: ops.head_unit_scale(go, wv, False, gg, 1e-5, gy, GH, gv), flush), nbytes=T * GH * gv * 10)
    sz, sw, sy = torch.randn(T, SH * sp, device=dev), torch.ones(SH * sp, device=dev), torch.empty(T, SH * sp, dtype=bf, device=dev)
    note("skip, silu(gate) and a norm in groups", timed(lambda: ops.skip_gate_norm(so, sx, sa, sp, sz, sw, sg, 1e-5, sy), flush), nbytes=T * SH * sp * 14)
    # router: sigmoid scores in groups (nikonex) beside corrected softmax scores in groups with pass-through rows
    rows_r = E + ident
    wr = (torch.randn(rows_r + 1, d, device=dev) / d ** 0.5).to(bf)
    ids = torch.empty(T, top + always, dtype=torch.int32, device=dev)
    wts = torch.empty(T, top + always, dtype=torch.float32, device=dev)
    passed = torch.empty(T, dtype=torch.float32, device=dev)
    corr = torch.randn(rows_r, device=dev) * 0.01

    def route(score, w, **kw):
        lg = rt.linear(h, w, out_dtype=torch.float32) if T > 64 else None
        ops.moe_router(h, w, kw.pop("bias", None), top, always, seq, ids, wts, lg, score=score, **kw)
    rb = T * d * 2 + E * d * 2
    note("router, sigmoid scores in groups, the shared expert's gate (nikonex)", timed(
        lambda: route("sigmoid_in_groups", wr[:E + 1], groups=z["groups"], keep=z["keep"], route_scale=2.5, gate_row=True), flush), nbytes=rb)
    note("router, corrected softmax scores in groups, rows that hand the input through", timed(
        lambda: route("softmax_corrected_in_groups", wr[:rows_r], bias=corr, groups=z["groups"], keep=z["keep"], route_scale=2.5,
                      n_real=E, pass_out=passed), flush), nbytes=rb)
    torch.cuda.synchronize()
    return out


def meropel_workload(steps: int, warmup: int) -> int:
    """The Meropel design at two sizes that resemble a real model's layers, beside the Nikonex design of the same
    width, layers, vocabulary and experts (random weights): a prompt of 2,048 tokens in one step, decoding at batch 8
    after 512-token prompts (device-timed), and every kernel of the design alone beside its like."""
    import torch
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.csrc import ops
    peaks, peak_source = load_peaks()
    result = {"metric": "Meropel beside Nikonex at equal sizes: prompt of 2,048 tokens, decode at batch 8 (512-token prompts), "
                        "bf16, random weights", "peak_source": peak_source, "sizes": {}}
    steps = min(steps, 64)
    for name, z in MEROPEL_SIZES.items():
        entry = {}
        for model, raw in (("meropel", meropel_config(z)), ("nikonex", nikonex_config(z))):
            need = PROMPT + warmup + steps + 72
            engine = Engine.random(config_from_dict(raw), WEIGHT_SEED, Engine_Opts(
                max_ctx=CONTEXT, max_tokens=max(8 * ((need + 63) // 64 * 64), PREFILL_TOKENS + 64), max_batch=8,
                dtype="bfloat16", verbose=False))
            ms_pf = run_prefill(engine, z["vocab"])
            tps, ms_step, _, launches = run_decode(engine, 8, steps, warmup, z["vocab"])
            entry[model] = {"layers": z["layers"], "weights_gib": round(engine.weight_bytes / 2 ** 30, 2),
                            "prefill_2048": {"ms": round(ms_pf, 3), "tokens_per_s": round(PREFILL_TOKENS / ms_pf * 1e3)},
                            "decode_b8": {"ms_per_step": round(ms_step, 4), "tokens_per_s": round(tps, 1),
                                          "launches_per_step": launches // steps}}
            engine.destroy()
            del engine
            torch.cuda.empty_cache()
        entry["kernels_prompt_2048_rows"] = meropel_kernels(z, PREFILL_TOKENS, peaks)
        entry["kernels_decode_8_rows"] = meropel_kernels(z, 8, peaks)
        result["sizes"][name] = entry
    ops.gemm_tc_check()
    ops.attention_prefill_check()
    ops.attention_decode_check()
    ops.moe_tc_check()
    print(json.dumps(result))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--no-graphs", action="store_true", help="launch the decode step's kernels one by one (for profilers)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end run (for profilers)")
    ap.add_argument("--workload", default="8b", choices=["8b", "1.7b-mixed", "32b-long", "tovalix", "nufupel", "nikonex", "meropel"],
                    help="8b: the contract's run (default).  The others are further workloads of the baseline's list and "
                         "print a line of their own: 1.7b-mixed = Qwen3-1.7B shape, 64 prompts of 16..2048 tokens, 128 new "
                         "tokens each; 32b-long = Qwen3-32B shape, a 2,048-token prompt, decoding 1 and 8 sequences at context 8192; "
                         "tovalix = the Tovalix design beside the Qwen3 decoder at equal sizes, and its kernels alone; "
                         "nufupel = the same for the Nufupel design; nikonex = the Nikonex design beside Nufupel at equal sizes, "
                         "and its kernels alone; meropel = the Meropel design beside Nikonex at equal sizes, and its kernels alone")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is written in Odin (CPU) and Metal (macOS GPU); this image has no Odin compiler, "
                          "it is no Python package, and it has no batched or CUDA path to run"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)
    if args.workload == "tovalix":
        return tovalix_workload(args.steps, warmup)
    if args.workload == "nufupel":
        return nufupel_workload(args.steps, warmup)
    if args.workload == "nikonex":
        return nikonex_workload(args.steps, warmup)
    if args.workload == "meropel":
        return meropel_workload(args.steps, warmup)
    if args.workload != "8b":
        return other_workload(args.workload)

    import torch
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.csrc import ops

    cfg_raw = dict(SHAPE_8B)
    full_layers = cfg_raw["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg_raw["num_hidden_layers"] = n_layers
    cfg = config_from_dict(cfg_raw)
    peaks, peak_source = load_peaks()
    vocab = cfg_raw["vocab_size"]

    max_batch = 64 if not args.no_points else args.batch
    need = PROMPT + max(warmup, 32) + args.steps + 8
    max_tokens = max(max_batch * ((need + 63) // 64 * 64), ((PREFILL_TOKENS + 63) // 64) * 64)
    engine = Engine.random(cfg, WEIGHT_SEED, Engine_Opts(max_ctx=CONTEXT, max_tokens=max_tokens, max_batch=max_batch,
                                                         dtype="bfloat16", verbose=False,
                                                         cuda_graphs=not args.no_graphs))

    sampler = ClockSampler()
    sampler.start()
    tps, ms_step, mean_ctx, launches = run_decode(engine, args.batch, args.steps, warmup, vocab)
    clocks = sampler.stop()
    ops.gemm_tc_check()
    ops.attention_prefill_check()
    ops.attention_decode_check()

    bytes_step = decode_bytes(cfg_raw, n_layers, args.batch, mean_ctx)
    achieved = bytes_step / (ms_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peak_source}

    if args.no_e2e:
        e2e = None
    else:
        stats, steady = run_e2e(engine, args.batch, args.steps, vocab)
        e2e = {"value": round(stats.decode_tokens_per_s, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": int(engine.last_step_h2d_bytes), "d2h_bytes_per_step": 4 * args.batch,
               "ttft_ms": round(stats.ttft_s * 1e3, 2), "steps": args.steps}
        if steady is not None:
            e2e["value_at_256_steps"] = round(steady.decode_tokens_per_s, 1)

    out = {
        "metric": "decode tokens/s (Qwen3-8B shape, bf16, batch %d, 512-token prompts)" % args.batch,
        "value": round(tps, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights N(0,0.02) seed 5)",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": n_layers, "layers_of_config": full_layers,
                   "hidden": cfg_raw["hidden_size"], "q_heads": cfg_raw["num_attention_heads"],
                   "kv_heads": cfg_raw["num_key_value_heads"], "head_dim": cfg_raw["head_dim"],
                   "intermediate": cfg_raw["intermediate_size"], "vocab": vocab, "global_batch": args.batch,
                   "prompt_len": PROMPT, "seq_len": CONTEXT, "decode_ctx_mean": round(mean_ctx, 1),
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (%.1f GB read per step)" % (bytes_step / 1e9),
                   "cuda_graphs": not args.no_graphs},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline,
    }
    if not args.no_points:
        ms_pf = run_prefill(engine, vocab)
        flops = prefill_flops(cfg_raw, n_layers, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (ms_pf / 1e3), 1), "tokens": PREFILL_TOKENS,
                          "ms": round(ms_pf, 3), "frac": round(flops / (ms_pf / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
        pts = {}
        for b in (1, 64):
            # The prompt step of 64 x 512 tokens runs for 0.4 s at the power cap, and the SM clock needs ~80 ms of
            # decoding to come back: at least 32 untimed steps, so that the point is the steady decode rate.
            t, m, c, _ = run_decode(engine, b, min(args.steps, 128), max(warmup, 32), vocab, seed=b)
            pts[f"decode_b{b}"] = round(t, 1)
            pts[f"decode_b{b}_hbm_frac"] = round(decode_bytes(cfg_raw, n_layers, b, c) / (m / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        out["points"] = pts
        ops.gemm_tc_check()
        ops.attention_prefill_check()
        ops.attention_decode_check()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
