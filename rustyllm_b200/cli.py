"""Command line in the manner of the reference's ``rusty-llm`` (SimonWaldherr/RustyLLM src/main.rs:39-127
for the options, 359-611 for their parsing, 1064-1094 for the statistics block,
1479-1628 for the benchmark JSON).  Options keep the reference's names and meanings
where this library has the thing they control:

  [model-dir] / --model, --prompt / -p, --max-tokens / -n, --temp / -t, --top-p, --top-k,
  --min-p, --repeat-penalty, --seed, --stop, --max-context, --kv-cache-dtype,
  --bench, --bench-json, --bench-runs, --bench-output, --kernel-bench,
  --kernel-bench-json, --kernel-bench-runs, --verbose / -v, --inspect, --list-tensors.

Differences, all from the missing tokenizer: ``--prompt`` takes token ids (separated by
spaces or commas) and ``--stop`` takes a token id or a sequence of ids; generated ids
are printed instead of text.  Added: ``--dtype`` (bfloat16 | float32), ``--random``
(random weights from the model folder's config.json alone, or from a config.json path),
``--prompt-file`` (one prompt of ids per line: a batch), and for the benchmark with
synthetic prompts ``--batch``, ``--prompt-len`` or ``--prompt-len-range lo,hi`` (lengths
drawn uniformly from [lo, hi) with the seed).  ``--decode-tokens``, ``--context``, ``--runs``
and ``--json`` are other spellings of ``--max-tokens``, ``--max-context``, ``--bench-runs``
and ``--bench-json``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional, Sequence


def _ids(text: str) -> List[int]:
    out = []
    for tok in text.replace(",", " ").split():
        try:
            out.append(int(tok))
        except ValueError:
            raise SystemExit(f"'{tok}' is not a token id; this library has no tokenizer, prompts are ids")
    return out


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="rustyllm", description="Generate with a Llama model folder on one B200.",
                                formatter_class=argparse.RawDescriptionHelpFormatter, epilog=__doc__)
    p.add_argument("model_pos", nargs="?", metavar="model-dir", help="folder with config.json and model.safetensors")
    p.add_argument("--model", help="same as the positional model folder")
    p.add_argument("--random", action="store_true", help="random weights from the folder's config.json (no safetensors needed)")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="compute dtype (default: bfloat16)")
    p.add_argument("--prompt", "--prompt-ids", "-p", dest="prompt", help="input prompt as token ids, e.g. '1 15043 3186' or 1,15043,3186")
    p.add_argument("--prompt-file", help="file with one prompt of token ids per line (a batch)")
    p.add_argument("--max-tokens", "--decode-tokens", "-n", dest="max_tokens", type=int, default=256, help="Max tokens to generate (default: 256)")
    p.add_argument("--temp", "-t", type=float, default=0.7, help="Temperature (default: 0.7, 0=greedy)")
    p.add_argument("--top-p", type=float, default=1.0, help="Nucleus sampling threshold (default: 1 = off; reference: 0.9)")
    p.add_argument("--top-k", type=int, default=0, help="Top-K filtering (default: 0 = off; reference: 40)")
    p.add_argument("--min-p", type=float, default=0.0, help="Min-P cutoff, relative to top token; 0 disables (default: 0)")
    p.add_argument("--repeat-penalty", type=float, default=1.0, help="Repetition penalty (default: 1 = off; reference: 1.1)")
    p.add_argument("--reference-sampler", action="store_true", help="the reference's sampler defaults: top-p 0.9, top-k 40, repeat penalty 1.1")
    p.add_argument("--seed", type=int, default=0, help="RNG seed (default: time-based)")
    p.add_argument("--stop", action="append", default=[], help="stop when this token id (or sequence of ids) is generated; repeatable")
    p.add_argument("--ignore-eos", action="store_true", help="do not stop at the model's end-of-sequence ids")
    p.add_argument("--max-context", "--context", dest="max_context", type=int, help="Cap runtime context/KV-cache length")
    p.add_argument("--kv-cache-dtype", default="auto", choices=["auto", "f32", "bf16", "q8"], help="KV cache dtype (auto = the compute dtype)")
    p.add_argument("--batch", type=int, default=1, help="benchmark: sequences per batch with synthetic prompts")
    p.add_argument("--prompt-len", type=int, default=128, help="benchmark: synthetic prompt length")
    p.add_argument("--prompt-len-range", metavar="LO,HI", help="benchmark: synthetic prompt lengths drawn uniformly from [LO, HI)")
    p.add_argument("--bench", action="store_true", help="Run a non-streaming generation benchmark")
    p.add_argument("--bench-json", "--json", dest="bench_json", action="store_true", help="Run benchmark and emit machine-readable JSON")
    p.add_argument("--bench-output", action="store_true", help="Include generated ids for each benchmark run")
    p.add_argument("--bench-runs", "--runs", dest="bench_runs", type=int, default=3, help="Number of benchmark runs (default: 3)")
    p.add_argument("--kernel-bench", action="store_true", help="Run isolated kernel benchmark")
    p.add_argument("--kernel-bench-json", action="store_true", help="Emit isolated kernel benchmark JSON")
    p.add_argument("--kernel-bench-runs", type=int, default=25, help="Number of kernel benchmark runs (default: 25)")
    p.add_argument("--kernel-bench-layer", type=int, default=0, help="Transformer layer to benchmark (default: 0)")
    p.add_argument("--ubatch", type=int, default=None, help="Logical prefill microbatch/chunk size: most prompt tokens one step runs (default: 16384)")
    p.add_argument("--verbose", "-v", action="store_true", help="Print startup timing details")
    p.add_argument("--inspect", action="store_true", help="Inspect config and checkpoint compatibility without loading weights")
    p.add_argument("--list-tensors", action="store_true", help="Print the checkpoint's tensor inventory and exit")
    return p


def _options(args):
    from . import GenerationOptions, SamplerConfig
    if args.reference_sampler:
        ref = SamplerConfig.reference_defaults()
        sampler = SamplerConfig(temperature=args.temp, top_p=ref.top_p, top_k=ref.top_k, min_p=args.min_p,
                                repeat_penalty=ref.repeat_penalty)
    else:
        sampler = SamplerConfig(temperature=args.temp, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                                repeat_penalty=args.repeat_penalty)
    stop_ids, stop_seqs = [], []
    for s in args.stop:
        ids = _ids(s)
        (stop_ids if len(ids) == 1 else stop_seqs).append(ids[0] if len(ids) == 1 else ids)
    opts = GenerationOptions(max_tokens=args.max_tokens, sampler=sampler, seed=args.seed, stop_token_ids=tuple(stop_ids),
                             stop_sequences=tuple(tuple(s) for s in stop_seqs), ignore_eos=args.ignore_eos,
                             max_context=args.max_context)
    if args.ubatch is not None:
        opts.prefill_step_tokens = args.ubatch
    opts.validate()
    return opts


def inspect(model_dir: str, list_tensors: bool) -> int:
    """Configuration, architecture and checkpoint compatibility, without loading weights
    (the reference's --inspect / --list-tensors over GGUF metadata)."""
    import torch
    from .config.files import read_config_json
    from .config.registry import resolve_architecture
    from .models.decoder import DecoderModel
    from .parts import Runtime
    from .weights.loader import WeightsError, check_checkpoint
    from .weights.safetensors_io import Checkpoint
    cfg = read_config_json(model_dir)
    arch = resolve_architecture(cfg)
    typed = arch.parse_config(cfg)
    spec = arch.build_spec(typed)
    print(f"architecture: {arch.name}")
    for k, v in (typed.to_dict() if hasattr(typed, "to_dict") else dict(typed)).items():
        print(f"  {k}: {v}")
    ck = Checkpoint(model_dir)
    print(f"checkpoint: {len(ck.entries)} tensors in {len(ck.files)} file(s), {ck.total_bytes} bytes")
    if list_tensors:
        for name, e in sorted(ck.entries.items()):
            print(f"  {name:60s} {str(e.dtype).replace('torch.', ''):9s} {list(e.shape)}")
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    try:
        check_checkpoint(model.param_specs(), ck.entries, spec.ignored_tensors, model_dir)
        print("compatibility: supported")
        return 0
    except WeightsError as e:
        print(f"compatibility: NOT loadable\n{e}")
        return 1


def synthetic_prompt_lengths(args, rnd) -> List[int]:
    """Lengths of the benchmark's synthetic prompts: ``--batch`` times ``--prompt-len``, or drawn
    uniformly from ``--prompt-len-range lo,hi`` (hi excluded) with the seeded generator."""
    if not args.prompt_len_range:
        if args.prompt_len <= 0:
            raise SystemExit("--prompt-len must be greater than 0")
        return [args.prompt_len] * args.batch
    try:
        lo, hi = (int(x) for x in args.prompt_len_range.replace(":", ",").split(","))
    except ValueError:
        raise SystemExit(f"--prompt-len-range wants two integers 'lo,hi', got {args.prompt_len_range!r}")
    if not (0 < lo < hi):
        raise SystemExit(f"--prompt-len-range needs 0 < lo < hi, got {lo},{hi}")
    return [rnd.randrange(lo, hi) for _ in range(args.batch)]


def _load(args, model_dir: str, max_batch: int):
    import torch
    from . import Runner
    kv = {"auto": None, "f32": torch.float32, "bf16": torch.bfloat16}.get(args.kv_cache_dtype, "q8")
    if kv == "q8":
        raise SystemExit("--kv-cache-dtype q8 is not implemented (the reference parses it and reports it as pending, too)")
    if kv is not None and kv != {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]:
        raise SystemExit("--kv-cache-dtype must match --dtype in this library (the attention kernels read the cache in the compute dtype)")
    t0 = time.perf_counter()
    if args.random:
        cfg_path = model_dir if model_dir.endswith(".json") else os.path.join(model_dir, "config.json")
        with open(cfg_path) as f:
            cfg = json.load(f)
        runner = Runner.from_config(cfg, seed=args.seed or 1, dtype=args.dtype, max_batch=max_batch, max_context=args.max_context)
        info = None
    else:
        runner, info = Runner.from_path(model_dir, dtype=args.dtype, max_batch=max_batch, max_context=args.max_context)
    if args.verbose:
        print(f"Loaded {runner.architecture()} '{runner.model_name()}' in {time.perf_counter() - t0:.2f}s", file=sys.stderr)
        if info is not None:
            print(f"  file size {info.file_size_bytes / 1e6:.1f} MB; parse {info.parse_time * 1e3:.0f} ms; "
                  f"compatibility {info.compatibility_time * 1e3:.0f} ms; weights {info.weights_time * 1e3:.0f} ms; "
                  f"runner {info.runner_time * 1e3:.0f} ms", file=sys.stderr)
        print(f"  parameters {runner.model.parameter_bytes() / 1e9:.2f} GB, cache {runner.cache.memory_bytes() / 1e9:.2f} GB "
              f"({runner.cache.num_pages} pages of {runner.cache.page_size} tokens), dtype {args.dtype}", file=sys.stderr)
    return runner, info


def _print_stats(results) -> None:
    """The reference's statistics block (src/main.rs:1064-1094)."""
    prompt = sum(r.stats.prompt_tokens for r in results)
    gen = sum(r.stats.generated_tokens for r in results)
    st = results[0].stats
    print("\n\n─── Stats ───────────────────────────────", file=sys.stderr)
    print(f"Prompt: {prompt} tokens", file=sys.stderr)
    print(f"Generated: {gen} tokens", file=sys.stderr)
    print(f"Prefill: {st.prefill_time:.2f}s ({prompt / max(st.prefill_time, 0.001):.1f} tok/s)", file=sys.stderr)
    print(f"Decode: {st.decode_time:.2f}s ({gen / max(st.decode_time, 0.001):.2f} tok/s)", file=sys.stderr)
    print(f"Total: {st.total_time:.2f}s", file=sys.stderr)


def run_benchmark(runner, info, prompts, opts, runs: int, as_json: bool, with_output: bool) -> int:
    """``--bench`` / ``--bench-json``: the reference's fields (src/main.rs:1521-1623) per run
    and in the summary; seeds go seed, seed+1, ... over the runs as there."""
    import dataclasses
    results, tp, tg, tpre, tdec, ttot, twall = [], 0, 0, 0.0, 0.0, 0.0, 0.0
    for run in range(runs):
        o = dataclasses.replace(opts, seed=(opts.seed + run) if opts.seed else 0)
        t0 = time.perf_counter()
        res = runner.generate(prompts, o)
        wall = time.perf_counter() - t0
        p = sum(r.stats.prompt_tokens for r in res); g = sum(r.stats.generated_tokens for r in res)
        st = res[0].stats
        row = {"run": run + 1, "prompt_tokens": p, "generated_tokens": g, "prefill_ms": round(st.prefill_time * 1e3),
               "decode_ms": round(st.decode_time * 1e3), "total_ms": round(st.total_time * 1e3),
               "wall_ms": round(wall * 1e3), "prefill_tok_s": p / max(st.prefill_time, 0.001),
               "decode_tok_s": g / max(st.decode_time, 0.001)}
        if with_output:
            row["token_ids"] = [r.token_ids for r in res]
        results.append(row)
        tp += p; tg += g; tpre += st.prefill_time; tdec += st.decode_time; ttot += st.total_time; twall += wall
        if not as_json:
            print(f"run {run + 1}: prompt {p} tok, generated {g} tok, prefill {row['prefill_tok_s']:.1f} tok/s, "
                  f"decode {row['decode_tok_s']:.2f} tok/s")
    # what a decode step has to read: every matrix once (the embedding table only where it is also the
    # head) and the cache of the live sequences at their mean length over the run
    m = runner.model
    weights = m.parameter_bytes()
    if m.head.weight.data_ptr() != m.embedding.weight.data_ptr():
        weights -= m.embedding.weight.numel() * m.embedding.weight.element_size()
    per_token = sum(g.bytes_per_token() for g in runner.cache.groups)
    mean_live = tp / runs + tg / runs / 2.0
    step_bytes = weights + per_token * mean_live
    steps_s = (tg / len(prompts)) / max(tdec, 0.001)            # every sequence decodes one token a step
    summary = {"decode_step_bytes": step_bytes, "decode_gb_s": step_bytes * steps_s / 1e9,
               "avg_prompt_tokens": tp / runs, "avg_generated_tokens": tg / runs, "avg_prefill_ms": tpre * 1e3 / runs,
               "avg_decode_ms": tdec * 1e3 / runs, "avg_total_ms": ttot * 1e3 / runs, "avg_wall_ms": twall * 1e3 / runs,
               "aggregate_prefill_tok_s": tp / max(tpre, 0.001), "aggregate_decode_tok_s": tg / max(tdec, 0.001)}
    if as_json:
        s = opts.sampler
        print(json.dumps({
            "type": "rusty-llm.benchmark", "model": runner.model_name() or "unknown", "architecture": runner.architecture(),
            "load_ms": round(info.load_time * 1e3) if info else 0, "file_size_bytes": info.file_size_bytes if info else 0,
            "runs": runs, "prompt": [len(p) for p in prompts],
            "options": {"max_tokens": opts.max_tokens, "temperature": s.temperature, "top_p": s.top_p, "top_k": s.top_k,
                        "min_p": s.min_p, "repeat_penalty": s.repeat_penalty, "seed": opts.seed,
                        "stop_sequences": [list(x) for x in opts.stop_sequences],
                        "runtime": {"max_context": opts.max_context, "batch": len(prompts)}},
            "results": results, "summary": summary}, indent=2))
    else:
        print(f"aggregate: prefill {summary['aggregate_prefill_tok_s']:.1f} tok/s, decode {summary['aggregate_decode_tok_s']:.2f} tok/s")
    return 0


def run_kernel_benchmark(runner, runs: int, as_json: bool, layer_index: int = 0) -> int:
    """``--kernel-bench``: per-operation time of one layer at one token, in the spirit of the
    reference's rows (attn_qkv.fused, attn_rope.qk, attn_scan.ctx*, ffn_gate_up.fused,
    ffn_activation.silu_mul, output; src/runtime.rs:2639-2815), with bytes and GB/s."""
    import torch
    from . import kernels as K
    if not 0 <= layer_index < len(runner.model.blocks):
        raise SystemExit(f"--kernel-bench-layer {layer_index}: the model has layers 0 to {len(runner.model.blocks) - 1}")
    blk = runner.model.blocks[layer_index]
    att, ff = blk.mixer, blk.feed_forward
    dev, dt = runner.runtime.device, runner.runtime.compute_dtype
    esz = 2 if dt == torch.bfloat16 else 4
    d = runner.model.spec.hidden_size

    def timed(fn):
        """Microseconds a call on the device: the runs are captured in one CUDA graph and replayed,
        so that the host's time to launch does not stand in for kernels of a few microseconds."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(runs):
                    fn()
            graph.replay()
            stream.synchronize()
            e0.record(stream)
            graph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / runs

    from .parts.linear import OUT_ADD_F32, OUT_F32, OUT_SAME, linear
    x = torch.randn(1, d, device=dev)
    xn = torch.empty(1, d, device=dev, dtype=dt)
    rows = []
    rows.append(("attn_norm.rms", timed(lambda: K.rmsnorm(x, blk.mixer_norm.weight, xn, blk.mixer_norm.eps)), d * 4))
    qkv = torch.empty(1, att.wqkv.shape[0], device=dev, dtype=att.wqkv.dtype)
    xq = xn.to(att.wqkv.dtype)
    rows.append(("attn_qkv.fused", timed(lambda: linear(xq, att.wqkv, qkv, OUT_SAME, att.bqkv)), att.wqkv.numel() * att.wqkv.element_size()))
    a = torch.randn(1, att.wo.shape[1], device=dev).to(att.wo.dtype)
    rows.append(("attn_output", timed(lambda: linear(a, att.wo, x, OUT_ADD_F32, att.bo)), att.wo.numel() * att.wo.element_size()))
    gu = torch.empty(1, ff.wgu.shape[0], device=dev, dtype=ff.wgu.dtype)
    xf = xn.to(ff.wgu.dtype)
    rows.append(("ffn_gate_up.fused", timed(lambda: linear(xf, ff.wgu, gu, OUT_SAME, ff.bgu)), ff.wgu.numel() * ff.wgu.element_size()))
    h = torch.empty(1, ff.I, device=dev, dtype=gu.dtype)
    rows.append(("ffn_activation.silu_mul", timed(lambda: K.swiglu(gu, h)), 3 * ff.I * esz))
    rows.append(("ffn_down", timed(lambda: linear(h, ff.wdown, x, OUT_ADD_F32, ff.bdown)), ff.wdown.numel() * ff.wdown.element_size()))
    head = runner.model.head
    logits = torch.empty(1, head.V, device=dev)
    xh = xn.to(head.weight.dtype)
    rows.append(("output", timed(lambda: linear(xh, head.weight, logits, OUT_F32)), head.weight.numel() * head.weight.element_size()))
    # attention over a cached context of several lengths
    eng = runner.engine
    max_ctx = min(runner.cache.max_seq_len, runner.cache.free_pages * runner.cache.page_size)
    for ctx in (32, 128, 512, 2048, 8192):
        if ctx + 1 > max_ctx:
            break
        s = eng.alloc_slot()
        eng.step([s], [[1] * ctx], None)
        group, layer = runner.cache.kv_entry(layer_index)
        st = eng.step_state(torch.tensor([1, ctx, s, 0, 1, s, ctx + 1, 0], dtype=torch.int32, device=dev), (1, 1, 1), [1], [ctx + 1])
        runner.cache.prepare([s], [1])
        q = torch.randn(1, qkv.shape[1], device=dev).to(dt)
        o = torch.empty(1, att.H * att.hd, device=dev, dtype=dt)
        t = timed(lambda: K.attention(q, group.k_pool(layer), group.v_pool(layer), group.page_table, st, o, att.H, att.G, att.hd, att.scale))
        rows.append((f"attn_scan.ctx{ctx}", t, 2 * (ctx + 1) * att.G * att.hd * esz))
        eng.free_slot(s)
    if as_json:
        # the reference's envelope (src/main.rs:1672-1676): "type" names the record, "format" its layout
        print(json.dumps({"type": "rusty-llm.kernel_benchmark", "format": "llm-kernel-bench.v1", "runtime": "rustyllm_b200",
                          "model": runner.model_name(), "runs": runs, "layer": layer_index,
                          "rows": [{"name": n, "avg_us": t, "bytes": b, "gb_s": b / t / 1e3} for n, t, b in rows]}, indent=2))
    else:
        for n, t, b in rows:
            print(f"{n:28s} {t:10.2f} us   {b / 1e6:10.2f} MB   {b / t / 1e3:9.1f} GB/s")
    return 0


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    model_dir = args.model or args.model_pos
    if not model_dir:
        build_parser().print_usage(sys.stderr)
        print("error: no model folder given", file=sys.stderr)
        return 2
    if args.inspect or args.list_tensors:
        return inspect(model_dir, args.list_tensors)
    try:
        opts = _options(args)
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    bench = args.bench or args.bench_json
    kbench = args.kernel_bench or args.kernel_bench_json
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts = [_ids(line) for line in f if line.strip()]
    elif args.prompt:
        prompts = [_ids(args.prompt)]
    elif bench:
        import random
        rnd = random.Random(args.seed or 1)
        prompts = None   # filled once the vocabulary is known
    elif kbench:
        prompts = []
    else:
        print("error: no prompt; give --prompt 'id id ...' or --prompt-file (this library has no tokenizer and no REPL)", file=sys.stderr)
        return 2
    runner, info = _load(args, model_dir, max_batch=max(args.batch, len(prompts) if prompts else 1))
    if kbench:
        return run_kernel_benchmark(runner, args.kernel_bench_runs, args.kernel_bench_json, args.kernel_bench_layer)
    if prompts is None:
        V = runner.model.spec.vocab_size
        prompts = [[rnd.randrange(V) for _ in range(n)] for n in synthetic_prompt_lengths(args, rnd)]
    if bench:
        return run_benchmark(runner, info, prompts, opts, args.bench_runs, args.bench_json, args.bench_output)
    single = len(prompts) == 1
    if single:
        res = [runner.generate_stream(prompts[0], opts, lambda t: (sys.stdout.write(f"{t} "), sys.stdout.flush()))]
        sys.stdout.write("\n")
    else:
        res = runner.generate(prompts, opts)
        for r in res:
            print(" ".join(str(t) for t in r.token_ids))
    _print_stats(res)
    return 0


if __name__ == "__main__":
    sys.exit(main())
