"""bin/trace_run as a user runs it: a subprocess fed steps on standard input; the same
requests whole, with the last 32 tokens one by one, and in batches of unequal
lengths, in 32-bit and in bfloat16, against the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from gpu_helpers import assert_close_logits, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_trace(model_dir, dtype, steps, out_dir, max_tokens):
    """Feeds the steps one at a time, waiting for 'done <step>' after each."""
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
                          "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens)],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for st in steps:
        p.stdin.write(json.dumps(st) + "\n")
        p.stdin.flush()
        line = p.stdout.readline().strip()
        assert line == f"done {st['step']}", f"got {line!r}"
    p.stdin.close()
    assert p.wait(timeout=120) == 0


def read_step(out_dir, step, vocab):
    a = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
    return torch.from_numpy(a.reshape(-1, vocab))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_three_cuts(model_dirs, tmp_path, name, dtype):
    d, cfg = model_dirs[name]
    V = cfg["vocab_size"]
    reqs = {f"r{i}": random_tokens(V, n, 500 + i) for i, n in enumerate([40, 97, 33, 70])}
    steps, expect = [], {}     # expect[step] = list of (request, positions)
    sn = 0
    # cut 1: each request alone and whole
    for rid, toks in reqs.items():
        steps.append({"step": sn, "entries": [{"id": rid + "w", "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid + "w"]})
        expect[sn] = [(rid, list(range(len(toks))))]; sn += 1
    # cut 2: all but the last 32 in one step, then one by one
    for rid, toks in reqs.items():
        n = len(toks)
        steps.append({"step": sn, "entries": [{"id": rid + "d", "tokens": toks[:n - 32], "want": [n - 33]}], "end": []})
        expect[sn] = [(rid, [n - 33])]; sn += 1
        for t in range(n - 32, n):
            steps.append({"step": sn, "entries": [{"id": rid + "d", "tokens": [toks[t]], "want": [0]}],
                          "end": [rid + "d"] if t == n - 1 else []})
            expect[sn] = [(rid, [t])]; sn += 1
    # cut 3: a batch of unequal lengths; prompts of 8/60/1/33 tokens, then one token each;
    # shorter requests end earlier; a step in which nothing is wanted lies in between
    starts = {"r0": 8, "r1": 60, "r2": 1, "r3": 33}
    steps.append({"step": sn, "entries": [{"id": rid + "b", "tokens": reqs[rid][:starts[rid]], "want": [starts[rid] - 1]}
                                          for rid in reqs], "end": []})
    expect[sn] = [(rid, [starts[rid] - 1]) for rid in reqs]; sn += 1
    fed = dict(starts)
    live = list(reqs)
    k = 0
    while live:
        entries, exp, end = [], [], []
        for rid in live:
            want = [] if k == 1 else [0]
            entries.append({"id": rid + "b", "tokens": [reqs[rid][fed[rid]]], "want": want})
            if want:
                exp.append((rid, [fed[rid]]))
            fed[rid] += 1
            if fed[rid] == len(reqs[rid]):
                end.append(rid + "b")
        steps.append({"step": sn, "entries": entries, "end": end})
        if exp:
            expect[sn] = exp
        sn += 1; k += 1
        live = [rid for rid in live if fed[rid] < len(reqs[rid])]
    out_dir = str(tmp_path / "out")
    # live at most: the batch of cut 3 -> 1 + 2 + 1 + 2 pages
    run_trace(d, dtype, steps, out_dir, max_tokens=64 * 6)
    assert not os.path.exists(os.path.join(out_dir, f"{[s['step'] for s in steps if not any(e['want'] for e in s['entries'])][0]}.f32"))
    for step, exp in expect.items():
        got = read_step(out_dir, step, V)
        ref = torch.cat([plain_logits(d, reqs[rid])[pos] for rid, pos in exp])
        assert_close_logits(got, ref, dtype, f"{name} step {step}")


@pytest.mark.parametrize("name", ["C", "E"])
def test_replay_of_a_random_trace(model_dirs, tmp_path, name):
    """Batches drawn at random, one after another: 1 to 8 requests of 1 to 300 prompt tokens and 0 to
    39 further tokens each, logits wanted at random places of the prompts and at four decoded tokens
    in five, requests that end with their prompt, steps in which nothing is wanted; the cache sized
    to the token exactly (the most that live requests hold, each rounded up to 64).  Both dtypes."""
    import random
    d, cfg = model_dirs[name]
    V, maxpos = cfg["vocab_size"], cfg["max_position_embeddings"]
    rng = random.Random(len(name) + V)
    steps, expect, reqs, sn, peak = [], {}, {}, 0, 0
    for batch in range(3):
        ids = [f"b{batch}r{i}" for i in range(rng.randrange(1, 9))]
        lens = {r: rng.randrange(1, min(300, maxpos - 45)) for r in ids}
        decs = {r: rng.randrange(0, 40) for r in ids}
        for r in ids:
            reqs[r] = random_tokens(V, lens[r] + decs[r], rng.randrange(1 << 30))
        peak = max(peak, sum(-(-(lens[r] + decs[r]) // 64) * 64 for r in ids))
        entries, exp = [], []
        for r in ids:
            want = sorted(rng.sample(range(lens[r]), rng.randrange(0, min(4, lens[r]) + 1)))
            entries.append({"id": r, "tokens": reqs[r][:lens[r]], "want": want})
            if want:
                exp.append((r, want))
        steps.append({"step": sn, "entries": entries, "end": [r for r in ids if decs[r] == 0]})
        if exp:
            expect[sn] = exp
        sn += 1
        fed, live = dict(lens), [r for r in ids if decs[r] > 0]
        while live:
            entries, exp, end = [], [], []
            for r in live:
                want = [0] if rng.random() < 0.8 else []
                entries.append({"id": r, "tokens": [reqs[r][fed[r]]], "want": want})
                if want:
                    exp.append((r, [fed[r]]))
                fed[r] += 1
                if fed[r] == len(reqs[r]):
                    end.append(r)
            steps.append({"step": sn, "entries": entries, "end": end})
            if exp:
                expect[sn] = exp
            sn += 1
            live = [r for r in live if fed[r] < len(reqs[r])]
    for dtype in ("float32", "bfloat16"):
        out_dir = str(tmp_path / dtype)
        run_trace(d, dtype, steps, out_dir, max_tokens=peak)
        for step, exp in expect.items():
            got = read_step(out_dir, step, V)
            ref = torch.cat([plain_logits(d, reqs[r])[pos] for r, pos in exp])
            assert_close_logits(got, ref, dtype, f"{name} step {step}")
