"""Times one kernel of the library alone, at a chosen shape, on random data.

    python -m rustyllm_b200.bench_kernels gemm --m 8 --n 28672 --k 4096 [--mode same|f32|add|swiglu] [--parts 0]
    python -m rustyllm_b200.bench_kernels attention-decode --batch 8 --context 800 [--splits 0] [--contexts 1761,1350,159 | --context-range 128,2048]
    python -m rustyllm_b200.bench_kernels attention-prefill --tokens 2048
    python -m rustyllm_b200.bench_kernels rmsnorm | swiglu | rope --m 8
    python -m rustyllm_b200.bench_kernels sample --m 8 --n 128256 [--greedy | --top-k 40 --top-p 0.9 | --top-p 0.9]

Each run launches the kernel ``--reps`` times after ``--warmup`` launches, rotating over
several copies of the big operand so that the 126 MB L2 cannot serve it, times the
launches with CUDA events and prints one line with microseconds a launch and the
achieved bandwidth or arithmetic rate (``--graph``: the timed launches run from one
CUDA graph, for kernels shorter than a launch takes the host).  It is the program the ncu captures under
``profiles/`` were taken from (few launches, small operands).
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import kernels as K

DEV = torch.device("cuda:0")
BF = torch.bfloat16


GRAPH = False      # --graph: the timed launches are captured in one CUDA graph (no host time between them)


def _time(fn, warmup: int, reps: int) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if GRAPH:
        stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for i in range(reps):
                    fn(warmup + i)
            graph.replay()
            stream.synchronize()
            e0.record(stream)
            graph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps
    e0.record()
    for i in range(reps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def gemm(a) -> None:
    mode = {"same": K.OUT_SAME, "f32": K.OUT_F32, "add": K.OUT_ADD_F32, "swiglu": K.OUT_SWIGLU}[a.mode]
    copies = max(2, min(8, int(300e6 // (a.n * a.k * 2)) + 1))
    ws = [torch.randn(a.n, a.k, device=DEV).to(BF) * 0.02 for _ in range(copies)]
    x = torch.randn(a.m, a.k, device=DEV).to(BF)
    if mode == K.OUT_SWIGLU:      # weight rows interleaved (gate, up): the epilogue writes silu(gate) * up, [M, N/2]
        out = torch.zeros(a.m, a.n // 2, device=DEV, dtype=BF)
    else:
        out = torch.zeros(a.m, a.n, device=DEV, dtype=BF if mode == K.OUT_SAME else torch.float32)
    us = _time(lambda i: K.gemm_tc(x, ws[i % copies], out, mode, force_splits=a.parts), a.warmup, a.reps)
    K.check_device_errors()
    flops, wbytes = 2.0 * a.m * a.n * a.k, a.n * a.k * 2.0
    print(f"gemm_tc M={a.m} N={a.n} K={a.k} parts={a.parts or K.gemm_tc_splits(a.m, a.n, a.k)}: {us:.2f} us, "
          f"{wbytes / us / 1e6:.2f} TB/s of weights, {flops / us / 1e6:.1f} TFLOP/s")


def _cache(batch: int, context: int, G: int, hd: int, layers: int):
    pages_per = -(-(context + 64) // 64)
    pools = [torch.randn(2, batch * pages_per, G, 64, hd, device=DEV).to(BF) for _ in range(layers)]
    pt = torch.arange(batch * pages_per, dtype=torch.int32, device=DEV).view(batch, pages_per)
    return pools, pt


def attention_decode(a) -> None:
    H, G, hd = a.heads, a.kv_heads, a.head_dim
    lens = [int(x) for x in a.contexts.split(",")] if a.contexts else [a.context] * a.batch
    if a.context_range:                      # seeded uniform draw, as the benchmarks' prompts
        lo, hi = (int(x) for x in a.context_range.split(","))
        g = torch.Generator().manual_seed(0)
        lens = torch.randint(lo, hi, (a.batch,), generator=g).tolist()
    a.batch, a.context = len(lens), max(lens)
    kv_bytes = sum(lens) * G * hd * 2 * 2
    layers = max(2, min(8, int(300e6 // kv_bytes) + 1))
    pools, pt = _cache(a.batch, a.context, G, hd, layers)
    slots = torch.arange(a.batch, dtype=torch.int32, device=DEV)
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    q = torch.randn(a.batch, (H + 2 * G) * hd, device=DEV).to(BF)
    out = torch.empty(a.batch, H * hd, device=DEV, dtype=BF)
    sp = a.splits or K.decode_splits(a.batch, G)
    plan = K.decode_plan(slots, kv, 0, sp) if a.batch > 1 and not a.cluster else None    # once a step, as the engine makes it
    if a.ordered:                            # every sequence whole, the longest first
        sp, plan = 1, K.decode_order(slots, kv, 0)
    us = _time(lambda i: K.attention_decode(q, pools[i % layers][0], pools[i % layers][1], pt, slots, kv, out, H, G, hd,
                                            1 / math.sqrt(hd), num_splits=sp, plan=plan, cluster=a.cluster), a.warmup, a.reps)
    print(f"attention_decode B={a.batch} context={a.contexts or a.context_range or a.context} (mean {sum(lens) / len(lens):.0f}) H={H} G={G} hd={hd} splits={sp}{' in order' if a.ordered else ''}: "
          f"{us:.2f} us, {kv_bytes / us / 1e6:.2f} TB/s of cache")


def attention_prefill(a) -> None:
    H, G, hd, T = a.heads, a.kv_heads, a.head_dim, a.tokens
    pools, pt = _cache(1, T, G, hd, 2)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    q = torch.randn(T, (H + 2 * G) * hd, device=DEV).to(BF)
    out = torch.empty(T, H * hd, device=DEV, dtype=BF)
    tc = not a.mma and K.attention_prefill_tc_supported(BF, H, G, hd)
    fn = K.attention_prefill_tc if tc else K.attention_prefill
    cu, sl, kl = i32([0, T]), i32([0]), i32([T])
    us = _time(lambda i: fn(q, pools[i % 2][0], pools[i % 2][1], pt, cu, sl, kl, [T], out, H, G, hd, 1 / math.sqrt(hd)),
               a.warmup, a.reps)
    K.check_device_errors()
    flops = 2 * 2 * H * hd * (T * (T + 1) / 2)
    print(f"attention_prefill ({'tcgen05' if tc else 'mma.sync'}) T={T} H={H} G={G} hd={hd}: {us:.2f} us, "
          f"{flops / us / 1e6:.1f} TFLOP/s (causal half counted)")


def sample(a) -> None:
    rows, V = a.m, a.n
    copies = max(2, int(300e6 // (rows * V * 4)) + 1)
    logits = [torch.randn(rows, V, device=DEV) * 3 for _ in range(copies)]
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    temps = torch.full((rows,), 0.8, device=DEV); u = torch.rand(rows, device=DEV)
    if a.top_k > 0 or a.top_p < 1.0:          # the candidate kernels: top-k (with top-p inside it) or top-p alone
        idx = torch.arange(rows, dtype=torch.int32, device=DEV)
        pp = torch.full((rows,), a.top_p, device=DEV); zero = torch.zeros(rows, device=DEV)
        if a.top_k > 0:
            kk = torch.full((rows,), a.top_k, dtype=torch.int32, device=DEV)
            us = _time(lambda i: K.sample_candidates(logits[i % copies], temps, u, zero, out, idx, kk, pp, None, None), a.warmup, a.reps)
        else:
            us = _time(lambda i: K.sample_candidates(logits[i % copies], temps, u, zero, out, None, None, None, idx, pp), a.warmup, a.reps)
        print(f"sample_candidates rows={rows} vocab={V} top_k={a.top_k} top_p={a.top_p}: {us:.2f} us")
        return
    if a.greedy:
        us = _time(lambda i: K.argmax(logits[i % copies], out), a.warmup, a.reps)
    else:
        us = _time(lambda i: K.sample_temperature(logits[i % copies], temps, u, out), a.warmup, a.reps)
    print(f"{'argmax' if a.greedy else 'sample_temperature'} rows={rows} vocab={V}: {us:.2f} us, "
          f"{rows * V * 4 * (1 if a.greedy else 2) / us / 1e3:.1f} GB/s of logits read")


def small(a) -> None:
    d, I, H, G, hd, M = a.hidden, a.intermediate, a.heads, a.kv_heads, a.head_dim, a.m
    if a.kernel == "rmsnorm":
        x = torch.randn(M, d, device=DEV); w = torch.ones(d, device=DEV); o = torch.empty(M, d, device=DEV, dtype=BF)
        us = _time(lambda i: K.rmsnorm(x, w, o, 1e-5), a.warmup, a.reps)
        nbytes = M * d * 6
    elif a.kernel == "swiglu":
        gu = torch.randn(M, 2 * I, device=DEV).to(BF); o = torch.empty(M, I, device=DEV, dtype=BF)
        us = _time(lambda i: K.swiglu(gu, o), a.warmup, a.reps)
        nbytes = M * I * 6
    else:
        pools, pt = _cache(M, 128, G, hd, 1)
        qkv = torch.randn(M, (H + 2 * G) * hd, device=DEV).to(BF)
        pos = torch.full((M,), 100, dtype=torch.int32, device=DEV); slots = torch.arange(M, dtype=torch.int32, device=DEV)
        inv = torch.rand(hd // 2, device=DEV)
        us = _time(lambda i: K.rope_kv_write(qkv, pos, slots, pt, inv, H, G, hd, hd, False, pools[0][0], pools[0][1]), a.warmup, a.reps)
        nbytes = M * (H + 2 * G) * hd * 2 * 2
    print(f"{a.kernel} M={M}: {us:.2f} us, {nbytes / us / 1e3:.1f} GB/s")


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m rustyllm_b200.bench_kernels", description=__doc__,
                                formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("kernel", choices=["gemm", "attention-decode", "attention-prefill", "rmsnorm", "swiglu", "rope", "sample"])
    p.add_argument("--m", type=int, default=8); p.add_argument("--n", type=int, default=4096); p.add_argument("--k", type=int, default=4096)
    p.add_argument("--mode", default="same", choices=["same", "f32", "add", "swiglu"]); p.add_argument("--parts", type=int, default=0)
    p.add_argument("--batch", type=int, default=8); p.add_argument("--context", type=int, default=800)
    p.add_argument("--contexts", default="", help="attention-decode: comma-separated lengths, one per sequence (instead of --batch/--context)")
    p.add_argument("--context-range", default="", help="attention-decode: LO,HI - lengths drawn uniformly from [LO, HI) with a fixed seed")
    p.add_argument("--splits", type=int, default=0); p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--heads", type=int, default=32); p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128); p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--intermediate", type=int, default=14336)
    p.add_argument("--greedy", action="store_true", help="sample: the argmax kernel")
    p.add_argument("--top-k", type=int, default=0, help="sample: the top-k kernel with this k (and --top-p inside it)")
    p.add_argument("--top-p", type=float, default=1.0, help="sample: nucleus threshold; without --top-k the top-p kernel over the whole vocabulary")
    p.add_argument("--cluster", action="store_true", help="attention-decode: the chunks of a sequence as one thread-block cluster (--splits 2, 4 or 8)")
    p.add_argument("--ordered", action="store_true", help="attention-decode: every sequence whole, the longest first (a plan made once)")
    p.add_argument("--mma", action="store_true", help="attention-prefill: the mma.sync kernel also where tcgen05 applies")
    p.add_argument("--warmup", type=int, default=3); p.add_argument("--reps", type=int, default=20)
    p.add_argument("--graph", action="store_true", help="capture the timed launches in one CUDA graph: kernels that take "
                   "less time than a launch costs the host are then timed back to back")
    a = p.parse_args(argv)
    global GRAPH
    GRAPH = a.graph
    {"gemm": gemm, "attention-decode": attention_decode, "attention-prefill": attention_prefill, "sample": sample}.get(a.kernel, small)(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
