"""Benchmark: decode tok/s at batch 8 (also 1 and 64) and prefill tok/s at 2,048 tokens, Llama 3.2 1B
shape, bfloat16, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference|plain-cpu]
                    [--shape 1b|3b|8b] [--layers N] [--batch B] [--only decode|prefill] [--no-graphs]

`--impl plain-cpu` times the plain float32 implementation under tests/ on the CPU (no GPU needed), with
the reference's own protocol: wall-clock prefill and generation times and tokens a second
(models/llm/generate.go:227-229,275-282).

A "step" is one decode step of the whole batch.  Prints ONE JSON line.  The weights a step reads
(2.47 GB) are far larger than the L2 cache, which is stated in `config` as the timing hygiene rule asks.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the benchmark model: Llama 3.2 1B shape (random weights, seed 2)
MODEL = dict(
    architectures=["LlamaForCausalLM"], hidden_size=2048, num_hidden_layers=16, intermediate_size=8192,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=128256, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    rms_norm_eps=1e-5, max_position_embeddings=131072, tie_word_embeddings=True)
# further shapes for extra measurements (`--shape`); the contract's line is measured at the default
SHAPES = {
    "1b": {},
    "3b": dict(hidden_size=3072, num_hidden_layers=28, intermediate_size=8192, num_attention_heads=24,
               num_key_value_heads=8, head_dim=128),
    "8b": dict(hidden_size=4096, num_hidden_layers=32, intermediate_size=14336, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, tie_word_embeddings=False,
               rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                 original_max_position_embeddings=8192)),
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", "0", "-lms", "25"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6 or not (t0 - 0.05 <= ts <= t1 + 0.15):
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def make_model_dir(tmp):
    import torch
    from dlgo_b200.config import config_from_dict
    from dlgo_b200.weights import write_random_model
    cfg = config_from_dict(MODEL)
    t0 = time.time()
    write_random_model(cfg, 2, tmp, device="cuda" if torch.cuda.is_available() else "cpu")
    print(f"[bench] wrote the random model in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return tmp


PROMPT_LEN = 0     # > 0: every prompt has this many tokens (extra measurements at long contexts)
PROMPT_RANGE = (128, 1024)     # prompt lengths are uniform in this range (inclusive), seed 3


def prompts_for(batch, seed=3):
    import torch
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(PROMPT_RANGE[0], PROMPT_RANGE[1] + 1, (batch,), generator=g).tolist()
    if PROMPT_LEN > 0:
        lens = [PROMPT_LEN] * batch
    return [torch.randint(0, MODEL["vocab_size"], (n,), generator=g).tolist() for n in lens]


def decode_run(llm, batch, steps, warmup, sample_clocks=False):
    """Device-timed decode: prompts in, `warmup` untimed steps, then exactly `steps` timed steps."""
    import torch
    from dlgo_b200.csrc import kernels
    eng = llm.engine
    prompts = prompts_for(batch)
    slots = [eng.take_slot() for _ in prompts]
    logits = eng.step(slots, prompts)
    nxt = kernels.argmax(logits).cpu().tolist()
    for _ in range(warmup):
        logits = eng.step(slots, [[t] for t in nxt])
        nxt = kernels.argmax(logits).cpu().tolist()
    sampler = ClockSampler() if sample_clocks else None
    if sampler:
        sampler.start()
    # the prompts of a large batch are a tensor-core burst of ~100 ms that leaves the GPU at its power
    # cap; decode steps timed right behind it came out up to 15 % slower than the same steps a moment later
    torch.cuda.synchronize()
    time.sleep(0.3)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    launches0 = kernels.LAUNCHES
    t0 = time.time()
    start.record()
    feed = [[t] for t in nxt]
    for _ in range(steps):
        # device-timed: the step and the argmax are queued without waiting for their result (the
        # ids fed are fixed; the end-to-end number below feeds back what was sampled)
        logits = eng.step(slots, feed)
        kernels.argmax(logits)
    end.record()
    torch.cuda.synchronize()
    t1 = time.time()
    ms = start.elapsed_time(end)
    clocks = sampler.stop(t0, t1) if sampler else None
    lens = [eng.length(s) for s in slots]
    for s in slots:
        eng.free_slot(s)
    return dict(ms_per_step=ms / steps, tok_s=batch * steps / (ms / 1e3), launches=kernels.LAUNCHES - launches0,
                clocks=clocks, mean_context=sum(lens) / len(lens) - steps / 2)


def prefill_run(llm, n_tokens, reps=5, lens=None):
    """Median time (ms) of one prompt step: one prompt of `n_tokens`, or, with `lens`, a packed batch of
    prompts of those lengths (what generate() runs first)."""
    import torch
    eng = llm.engine
    g = torch.Generator().manual_seed(11)
    times = []
    lens = list(lens) if lens else [n_tokens]
    for r in range(reps + 2):
        toks = [torch.randint(0, MODEL["vocab_size"], (n,), generator=g).tolist() for n in lens]
        slots = [eng.take_slot() for _ in lens]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        eng.step(slots, toks)
        end.record()
        torch.cuda.synchronize()
        for s in slots:
            eng.free_slot(s)
        if r >= 2:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def prefill_flops(n_tokens, lens=None):
    m = MODEL
    d, f, hq, hkv, hd, L = (m["hidden_size"], m["intermediate_size"], m["num_attention_heads"],
                            m["num_key_value_heads"], m["head_dim"], m["num_hidden_layers"])
    lens = list(lens) if lens else [n_tokens]
    per_token = 2 * d * (hq * hd + 2 * hkv * hd) + 2 * hq * hd * d + 2 * d * 2 * f + 2 * f * d
    gemm = sum(lens) * per_token * L + len(lens) * 2 * d * m["vocab_size"]   # the head runs for each prompt's last row
    attn = sum(L * hq * hd * 2 * 2 * (n * (n + 1) // 2) for n in lens)       # causal QK^T and PV
    return gemm + attn


def e2e_run(llm, batch, steps):
    """The same metric through the public entry point: host token ids in, host token ids out."""
    prompts = prompts_for(batch)
    llm.generate(prompts, max_tokens=4, greedy=True, ignore_eos=True)          # warm-up (graphs, pages)
    res = llm.generate_detailed(prompts, max_tokens=steps + 1, greedy=True, ignore_eos=True)
    return batch * steps / (res.generate_ms / 1e3)


def sampled_run(llm, batch, steps) -> dict:
    """Decode tokens a second through the public entry point (host ids in and out, the prompts' step not
    counted) for greedy choice, the reference's default sampler (temperature 0.7, top-k 40, top-p 0.9,
    repetition penalty 1.1: ops/sampling.go:19-27), and temperature alone."""
    prompts = prompts_for(batch)
    out = {"only": "sampled", "batch": batch, "steps": steps}
    for name, opts in (("greedy", dict(greedy=True)), ("default_sampler", dict(seed=1)),
                       ("temperature_only", dict(seed=1, temperature=0.7, top_k=0, top_p=1.0, repetition_penalty=1.0))):
        llm.generate(prompts, max_tokens=4, ignore_eos=True, **opts)          # warm-up (graphs, pages)
        res = llm.generate_detailed(prompts, max_tokens=steps + 1, ignore_eos=True, **opts)
        out[name] = round(batch * steps / (res.generate_ms / 1e3), 1)
    return out


def plain_cpu_baseline() -> dict:
    """The plain implementation (tests/plain_llama.py: whole sequences, no cache, float32, CPU) timed as the
    reference times itself: prefill = the prompt's forward pass, generation = the tokens after the first,
    tokens a second over the generation time (models/llm/generate.go:227-229,275-282).  Tiny A and Tiny B
    with their workloads, and one single-token forward pass at the benchmark's layer sizes."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_llama as P
    from tiny_configs import random_tokens, write_tiny
    out = {"impl": "plain-cpu", "threads": torch.get_num_threads()}
    for name, lens, n_new in (("A", (5, 17, 32), 16), ("B", (1, 9, 70, 130), 24)):
        with tempfile.TemporaryDirectory() as tmp:
            cfg, w = P.read_model(write_tiny(name, tmp))
        pre = gen = 0.0
        toks = 0
        for i, n in enumerate(lens):
            seq = random_tokens(n, cfg["vocab_size"], 100 + i)
            t0 = time.perf_counter()
            nxt = P.argmax(P.forward(cfg, w, seq)[-1])
            t1 = time.perf_counter()
            for _ in range(n_new - 1):
                seq.append(nxt)
                nxt = P.argmax(P.forward(cfg, w, seq)[-1])     # no cache: the whole sequence again
            t2 = time.perf_counter()
            pre += t1 - t0
            gen += t2 - t1
            toks += n_new - 1
        out[f"tiny_{name}"] = {"requests": len(lens), "prompt_tokens": sum(lens), "new_tokens": n_new,
                               "prefill_ms": round(pre * 1e3, 1), "generate_ms": round(gen * 1e3, 1),
                               "tok_s": round(toks / gen, 2)}
    # one token through all layers at the benchmark's sizes (what a decode step computes, without a cache to read)
    m = MODEL
    torch.manual_seed(2)
    d, f, hq, hkv, hd = (m["hidden_size"], m["intermediate_size"], m["num_attention_heads"],
                         m["num_key_value_heads"], m["head_dim"])
    w = {"model.embed_tokens.weight": torch.randn(m["vocab_size"], d) * 0.02, "model.norm.weight": torch.ones(d)}
    for i in range(m["num_hidden_layers"]):
        p = f"model.layers.{i}."
        for n, shape in (("self_attn.q_proj", (hq * hd, d)), ("self_attn.k_proj", (hkv * hd, d)),
                         ("self_attn.v_proj", (hkv * hd, d)), ("self_attn.o_proj", (d, hq * hd)),
                         ("mlp.gate_proj", (f, d)), ("mlp.up_proj", (f, d)), ("mlp.down_proj", (d, f))):
            w[p + n + ".weight"] = torch.randn(shape) * 0.02
        w[p + "input_layernorm.weight"] = torch.ones(d)
        w[p + "post_attention_layernorm.weight"] = torch.ones(d)
    times = []
    for r in range(4):
        t0 = time.perf_counter()
        P.forward(m, w, [r + 1])
        times.append(time.perf_counter() - t0)
    ms = statistics.median(times[1:]) * 1e3
    out["llama_1b_one_token"] = {"ms": round(ms, 1), "tok_s": round(1e3 / ms, 2), "weights_gb_fp32": round(
        sum(t.numel() for t in w.values()) * 4 / 1e9, 2)}
    return out


def phase_stamps(llm, batch):
    """Phase timing of the persistent decode kernel (csrc/decode_layers.cu), which stamps the global timer at
    its phase boundaries when built with -DDLGO_TIMING.  Run as
        DLGO_FUSED_DECODE=1 DLGO_NVCC_FLAGS=-DDLGO_TIMING python bench.py --only phases --layers 4 --batch 8
    Prints, for the launch's second layer, when each phase ended (us after the first CTA began the layer;
    minimum, median and maximum over the CTAs)."""
    import ctypes
    import torch
    from dlgo_b200.csrc import build, kernels
    eng = llm.engine
    if not eng.model.fused_runs or "DLGO_TIMING" not in os.environ.get("DLGO_NVCC_FLAGS", ""):
        print("bench.py --only phases needs DLGO_FUSED_DECODE=1 and DLGO_NVCC_FLAGS=-DDLGO_TIMING in the environment")
        return 2
    prompts = prompts_for(batch)
    slots = [eng.take_slot() for _ in prompts]
    nxt = kernels.argmax(eng.step(slots, prompts)).cpu().tolist()
    for _ in range(6):
        eng.step(slots, [[t] for t in nxt])
    torch.cuda.synchronize()
    lib = build.load_library("decode_layers")
    buf = (ctypes.c_ulonglong * (256 * 16))()
    if lib.dlgo_decode_layers_times(buf) != 0:
        return 1
    grid = kernels.decode_layers_grid()
    rows = [[buf[c * 16 + k] for k in range(15)] for c in range(grid)]
    t0 = min(r[0] for r in rows)
    names = ["layer begins", "P1 operand built", "P1 epilogue done", "barrier 1 passed", "P2 attention done",
             "barrier 2 passed", "P3 operand built", "P3 epilogue done", "barrier 3 passed", "P4 operand built",
             "P4 epilogue done", "barrier 4 passed", "P5 operand built", "P5 epilogue done", "barrier 5 passed"]
    print(f"persistent decode kernel, batch {batch}, {grid} CTAs: us after the first CTA began the layer (min / median / max)")
    for k, n in enumerate(names):
        col = sorted((r[k] - t0) / 1e3 for r in rows)
        print(f"  {n:18s} {col[0]:8.2f} {col[len(col) // 2]:8.2f} {col[-1]:8.2f}")
    for s in slots:
        eng.free_slot(s)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "plain-cpu"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="layer sizes (default: the contract's Llama 3.2 1B)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all)")
    ap.add_argument("--prompt-len", type=int, default=0, help="fixed prompt length instead of uniform[128,1024]")
    ap.add_argument("--prompt-range", default="", help="LO,HI: prompt lengths uniform in [LO, HI] (default 128,1024)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="longest sequence the cache is sized for")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="--only prefill: tokens of the prompt")
    ap.add_argument("--prefill-batch", type=int, default=0,
                    help="--only prefill: a packed batch of that many prompts with lengths from --prompt-range")
    ap.add_argument("--only", choices=["decode", "prefill", "phases", "sampled"],
                    help="run one small workload (for profiling) and stop; phases: see phase_stamps()")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode kernels one by one (for profiling)")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "computerex/dlgo is a Go module (no setup.py/pyproject.toml: pip cannot install it), no Go "
                          "toolchain is in the image, and its GPU path is Vulkan, which is unavailable on this box"}))
        return 0
    if a.impl == "plain-cpu":
        print(json.dumps(plain_cpu_baseline()))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    import torch
    import dlgo_b200
    warmup = max(a.warmup, 3)
    pk = peaks()
    global PROMPT_LEN, PROMPT_RANGE
    PROMPT_LEN = a.prompt_len
    if a.prompt_range:
        lo, hi = (int(v) for v in a.prompt_range.split(","))
        PROMPT_RANGE = (lo, hi)
    MODEL.update(SHAPES[a.shape])
    layers_of_config = MODEL["num_hidden_layers"]
    if a.layers > 0:
        MODEL["num_hidden_layers"] = a.layers
    a.layers = MODEL["num_hidden_layers"]
    tmp = tempfile.mkdtemp(prefix="dlgo_b200_bench_")
    try:
        make_model_dir(tmp)
        llm = dlgo_b200.load_llm(tmp, a.context, dtype="bfloat16", max_batch=max(64, a.batch),
                                 cuda_graphs=not a.no_graphs)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    eng = llm.engine
    if a.only == "phases":
        return phase_stamps(llm, a.batch)
    if a.only == "decode":
        r = decode_run(llm, a.batch, a.steps, warmup)
        kv = sum(2 * n.num_kv_heads * n.head_dim for n in eng.model.cache_needs()[0] if n is not None) * 2
        gbs = (eng.weight_bytes() + a.batch * r["mean_context"] * kv) / (r["ms_per_step"] / 1e3) / 1e9
        print(json.dumps({"only": "decode", "shape": a.shape, "layers": a.layers, "batch": a.batch,
                          "mean_context": round(r["mean_context"], 1), "ms_per_step": round(r["ms_per_step"], 4),
                          "tok_s": round(r["tok_s"], 1), "launches": r["launches"], "hbm_gbs": round(gbs, 1),
                          "hbm_frac": round(gbs / pk["hbm_gbs"], 4), "peaks": pk["source"]}))
        return 0
    if a.only == "sampled":
        print(json.dumps(sampled_run(llm, a.batch, a.steps)))
        return 0
    if a.only == "prefill":
        lens = [len(p) for p in prompts_for(a.prefill_batch)] if a.prefill_batch > 0 else [a.prefill_tokens]
        ms = prefill_run(llm, a.prefill_tokens, reps=max(1, a.steps), lens=lens)
        fl = prefill_flops(a.prefill_tokens, lens)
        print(json.dumps({"only": "prefill", "shape": a.shape, "layers": a.layers, "prompts": len(lens),
                          "tokens": sum(lens), "ms": round(ms, 3), "tok_s": round(sum(lens) / (ms / 1e3), 1),
                          "tflops": round(fl / (ms / 1e3) / 1e12, 1),
                          "frac_of_burst": round(fl / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4), "peaks": pk["source"]}))
        return 0
    main_run = decode_run(llm, a.batch, a.steps, warmup, sample_clocks=True)
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = round(decode_run(llm, b, min(a.steps, 64), warmup)["tok_s"], 1)
    e2e = e2e_run(llm, a.batch, a.steps)
    pre_ms = prefill_run(llm, PREFILL_TOKENS)
    weight_bytes = eng.weight_bytes()
    kv_per_pos = sum(2 * n.num_kv_heads * n.head_dim for n in eng.model.cache_needs()[0] if n is not None) * 2
    step_bytes = weight_bytes + a.batch * main_run["mean_context"] * kv_per_pos
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
    flops = prefill_flops(PREFILL_TOKENS)
    out = {
        "metric": "decode tok/s @ batch %d (%s shape, bf16); points: batch 1/64; prefill tok/s @ 2,048" % (
            a.batch, {"1b": "Llama-3.2-1B", "3b": "Llama-3.2-3B", "8b": "Llama-3.1-8B"}[a.shape]),
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights seed 2)",
        "impl": "ours",
        "config": {
            "model": {"1b": "llama-3.2-1b-shape", "3b": "llama-3.2-3b-shape", "8b": "llama-3.1-8b-shape"}[a.shape],
            "layers": a.layers, "layers_of_config": layers_of_config, "hidden": MODEL["hidden_size"],
            "heads": MODEL["num_attention_heads"], "kv_heads": MODEL["num_key_value_heads"],
            "head_dim": MODEL["head_dim"], "ffn": MODEL["intermediate_size"], "vocab": MODEL["vocab_size"],
            "tied": MODEL["tie_word_embeddings"], "global_batch": a.batch,
            "seq_len": a.context, "prompt_len": ("uniform[%d,%d] seed 3" % PROMPT_RANGE if a.prompt_len <= 0 else a.prompt_len), "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "none (1 GPU)", "l2": "inputs larger than L2 (weights read per step: %.2f GB)" % (weight_bytes / 1e9),
            "cuda_graph": True, "peaks": pk["source"]},
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": 3 * 4 * a.batch,
                "d2h_bytes_per_step": 4 * a.batch},
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "prefill": {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
