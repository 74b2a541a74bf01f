#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.1-8B shape with random bf16 weights on
one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Prints ONE JSON line.  ``value``: decoded tokens a second at a batch of 8 (K single-token
steps timed on the device with CUDA events after W warm-up steps).  ``e2e``: the same
through ``Runner.generate`` (host token ids in, host token ids out; every step uploads
its inputs from pinned memory and reads the sampled ids back), K steps on the host's clock
after at least 24 single-token steps of the same generation (``e2e.window`` says which; the
figure from the first decoded token on stands beside it).  ``prefill``: one step
over a 2,048-token prompt.  ``roofline``: bytes a decode step must read (every weight
it uses once, and the cache of the live sequences) over its time, against the measured
copy bandwidth.  ``points``: decode at batch 1 and 64.

Weights (15 GB) are far larger than the L2 cache, so every timed step reads them from
HBM; no extra flush is needed.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the Llama-3.1-8B shape the headline numbers are quoted on
LLAMA_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 128256, "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "torch_dtype": "bfloat16",
}
CONTEXT = 4096
PROMPT_RANGE = (128, 2048)
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=FALLBACK_PEAKS["bf16_tflops"]), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", "0", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0])); mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def matmul_params(cfg, layers):
    d, I = cfg["hidden_size"], cfg["intermediate_size"]
    H, G, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = d * (H + 2 * G) * hd + H * hd * d + 2 * I * d + I * d
    return layers * per_layer, cfg["vocab_size"] * d


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=24)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="only the batch given (no batch 1 / 64 points)")
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="do not time the CPU baseline (vs_baseline stays null)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate; no cargo/rustc in this image and no network, "
                          "so it cannot be installed"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch
    from rustyllm_b200 import GenerationOptions, Runner, SamplerConfig, kernels

    peaks, peak_src = load_peaks()
    cfg = dict(LLAMA_8B)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    dev = torch.device("cuda:0")
    max_b = max(64, args.batch)
    runner = Runner.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", num_layers=layers,
                                max_cache_tokens=max_b * CONTEXT, max_batch=max_b, max_context=CONTEXT)
    eng = runner.engine
    rng = np.random.default_rng(0)
    layer_params, head_params = matmul_params(cfg, layers)
    weight_bytes = 2 * (layer_params + head_params)
    kv_bytes_per_token = layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2

    def draw_prompts(batch):
        lens = rng.integers(PROMPT_RANGE[0], PROMPT_RANGE[1], size=batch).tolist()
        return [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lens]

    def time_decode(batch, steps, warmup, prompts=None):
        """Prefill `batch` prompts of U[128, 2048) tokens, then time `steps` single-token steps."""
        prompts = prompts or draw_prompts(batch)
        slots = [eng.alloc_slot() for _ in range(batch)]
        for b in range(batch):            # one prompt a step keeps the prefill's scratch small
            eng.step([slots[b]], [prompts[b]], None)
        toks = [[int(t)] for t in rng.integers(0, cfg["vocab_size"], size=batch)]
        for _ in range(warmup):
            eng.step(slots, toks, "last")
        torch.cuda.synchronize()
        ctx_tokens = sum(eng.cache.length(s) for s in slots)
        l0 = kernels.launch_count
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            eng.step(slots, toks, "last")
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = kernels.launch_count - l0
        mean_ctx = ctx_tokens + batch * steps / 2
        for s in slots:
            eng.free_slot(s)
        return ms, launches, mean_ctx

    def point(batch, ms, ctx_tokens):
        """One decode measurement as a record: tokens a second, the step's time, the mean context of
        its sequences and the fraction of the copy bandwidth its bytes (weights + live cache) reach."""
        gbs = (weight_bytes + ctx_tokens * kv_bytes_per_token) / (ms * 1e-3) / 1e9
        return {"value": batch * 1000.0 / ms, "ms_per_step": round(ms, 4), "mean_context": round(ctx_tokens / batch, 1),
                "gb_s": round(gbs, 1), "frac": round(gbs / peaks["hbm_gbs"], 4)}

    clocks = ClockSampler()
    clocks.start()
    headline_prompts = draw_prompts(args.batch)      # the device-timed and the end-to-end arm decode the same batch
    ms, launches, ctx_tokens = time_decode(args.batch, args.steps, args.warmup, headline_prompts)
    clock_info = clocks.stop()
    value = args.batch * 1000.0 / ms
    step_bytes = weight_bytes + ctx_tokens * kv_bytes_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    # ---- prefill of 2,048 tokens ----
    s = eng.alloc_slot()
    prompt = rng.integers(0, cfg["vocab_size"], size=PREFILL_TOKENS).tolist()
    eng.step([s], [prompt], "last")
    eng.free_slot(s)
    torch.cuda.synchronize()
    pre_ms = []
    for _ in range(3):
        s = eng.alloc_slot()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([s], [prompt], "last")
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
        eng.free_slot(s)
    pms = sorted(pre_ms)[1]
    T = PREFILL_TOKENS
    H, hd = cfg["num_attention_heads"], cfg["head_dim"]
    attn_flops = layers * 2 * 2 * H * hd * (T * (T + 1) // 2)     # QK^T and PV over the causal half
    pre_flops = 2 * T * layer_params + 2 * head_params + attn_flops
    prefill = {"value": T * 1000.0 / pms, "tokens": T, "ms": round(pms, 3),
               "frac": pre_flops / (pms * 1e-3) / (peaks["bf16_tflops"] * 1e12)}

    # ---- batch 1 and 64 ----
    points, point_details = {}, {}
    if not args.skip_points:
        for b in (1, 64):
            # behind their prompt steps (a second of work at full power for 64 prompts) the clocks need some
            # twenty steps to come back, so these points never take fewer warm-up steps than the end-to-end arm
            pm, _, pctx = time_decode(b, max(32, args.steps // 2), max(args.warmup, 24))
            points[f"decode_b{b}"] = b * 1000.0 / pm
            point_details[f"decode_b{b}"] = point(b, pm, pctx)

    # ---- end to end through the entry point ----
    # One generation; the host's clock is read in the token callback, when the ids of a step are in
    # the host's hands.
    prompts = headline_prompts
    mk = lambda n: GenerationOptions(max_tokens=n, sampler=SamplerConfig(temperature=0.8), seed=1, ignore_eos=True)
    runner.generate(prompts, mk(4))                   # captures the step for this batch size
    # The ~20 steps right behind a prompt step of thousands of tokens run 15 to 20 % slower (3.8 ms
    # instead of 3.2: the clocks the prompt step's power draw left behind; with 16-token prompts the
    # first step is as fast as the hundredth).  The timed window therefore starts after at least 24
    # single-token steps, whatever --warmup says; the figure from the first decoded token on is
    # reported beside it.
    lead = max(args.warmup, 24)
    stamps = []
    def on_token(i, _tok):
        if i == args.batch - 1:                       # the last sequence of a step's tokens
            stamps.append(time.perf_counter())
    t_gen = time.perf_counter()
    runner.generate(prompts, mk(lead + args.steps + 1), on_token=on_token)
    assert len(stamps) == lead + args.steps + 1
    e2e_value = args.batch * args.steps / (stamps[lead + args.steps] - stamps[lead])
    # the same generation from its first decoded token on (the steps right behind the prompt step
    # run at the clocks that step's power draw left behind), and with the prompt step included
    e2e_from_first = args.batch * (lead + args.steps) / (stamps[-1] - stamps[0])
    e2e_with_prompt = args.batch * (lead + args.steps + 1) / (stamps[-1] - t_gen)
    # the reference's default sampler (top-k 40, top-p 0.9, repeat penalty 1.1; src/sampling.rs:30-52)
    # instead of plain temperature sampling: the path a user of the reference's defaults gets
    ref_s = SamplerConfig.reference_defaults()
    stamps_ref = []
    runner.generate(prompts, GenerationOptions(max_tokens=lead + args.steps + 1, sampler=ref_s, seed=1, ignore_eos=True),
                    on_token=lambda i, _t: stamps_ref.append(time.perf_counter()) if i == args.batch - 1 else None)
    e2e_ref_sampler = args.batch * args.steps / (stamps_ref[lead + args.steps] - stamps_ref[lead])
    # per single-token step: 7B+1 int32 (tokens, positions, slots, offsets, lengths, wanted rows)
    # and 3B float32 for the sampler (temperature, uniform, min_p), all from pinned memory
    h2d_per_step = (7 * args.batch + 1) * 4 + 3 * args.batch * 4
    kernels.check_device_errors()

    # ---- the CPU baseline: this library's plain C++ float32 decoder at the same widths and depth ----
    # The reference cannot be built here (no Rust toolchain) and publishes no number for this
    # configuration, so the baseline is our own CPU restatement of its formulas, timed on this
    # machine's host cores.  Like the reference it has no batching: its tokens a second are the same
    # for one request or for eight one after another.
    cpu = None
    if not args.skip_cpu_baseline:
        del runner, eng
        torch.cuda.empty_cache()
        try:
            from rustyllm_b200 import baseline
            cpu = baseline.time_decode(dict(cfg, num_hidden_layers=layers), distinct_layers=min(2, layers), context=4, tokens=4)
        except Exception as e:      # a host without g++ or OpenMP: the GPU numbers stand without it
            cpu = {"unavailable": f"{type(e).__name__}: {e}"[:200]}

    out = {
        "metric": "Llama-3.1-8B decode tok/s at batch 8 (bf16, random weights, context 4096)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / cpu["tokens_per_s"]) if cpu and "tokens_per_s" in cpu else None,
        "dtype": "bf16", "data": "synthetic (seeded random token ids, random-init weights N(0, 0.02))",
        "impl": "ours",
        "config": {"model": "Llama-3.1-8B shape", "layers": layers, "layers_of_config": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": "U[128,2048)",
                   "mean_context": round(ctx_tokens / args.batch, 1), "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (15 GB of weights a step)", "peaks": peak_src,
                   "decode": "CUDA graph per batch size and class of lengths",
                   "points": "batch 1 and 64: at least 24 warm-up and 32 timed single-token steps each",
                   "e2e_loop": "each step copies its integers from pinned memory and its sampled ids back; "
                               "a step is queued before the host has read the previous step's ids"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": int(h2d_per_step),
                "d2h_bytes_per_step": 4 * args.batch,
                "window": f"single-token steps {lead + 1} to {lead + args.steps} of one generation (the first {lead} run at the clocks the prompt step left behind)",
                "from_first_decoded_token": e2e_from_first, "with_prompt_step": e2e_with_prompt,
                "reference_default_sampler": e2e_ref_sampler},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"]},
        "points": points,
        "point_details": dict(point_details, **{f"decode_b{args.batch}": point(args.batch, ms, ctx_tokens)}),
        "cpu_baseline": cpu,
        "clocks": clock_info,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
