"""Trace replay: feeds given token ids through the model step by step and writes
logits.  It samples nothing and has no model code of its own: it drives the same
registry, loader, cache, step function and kernels that generation uses.

Input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
``entries``: for each request its next tokens and the places among them whose
logits are wanted; ``end``: requests that are finished after this step (their slot
and pages go back).  For a step in which something is wanted, ``<out>/<step>.f32``
holds the logits at the wanted places in the order of the entries and of ``want``,
little-endian float32 ``[wanted, vocab]``.  After every step a line ``done <step>``
is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import numpy as np
import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from ..kernels import PAGE_SIZE
    from .runner import Runner   # late: building the kernels prints progress lines
    os.makedirs(args.out, exist_ok=True)
    pages = -(-args.max_tokens // PAGE_SIZE)     # the cache's own unit is the 64 tokens the option counts in
    runner, _ = Runner.from_path(args.model, dtype=args.dtype, device=args.device,
                                 max_cache_tokens=pages * PAGE_SIZE, max_batch=min(max(pages, 1), 1024))
    engine = runner.engine
    slot_of: Dict[str, int] = {}
    dev = torch.device(args.device)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = rec.get("entries", [])
        if entries:
            slots, tokens, want = [], [], []
            for e in entries:
                rid = str(e["id"])
                if rid not in slot_of:
                    slot_of[rid] = engine.alloc_slot()
                slots.append(slot_of[rid])
                tokens.append(list(e["tokens"]))
                want.append(list(e.get("want", [])))
            logits = engine.step(slots, tokens, want)
            if logits is not None:
                arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.synchronize(dev)
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slot_of:
                engine.free_slot(slot_of.pop(rid))
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()
    from .. import kernels
    kernels.check_device_errors()
    if int(runner.model.embedding.bad_token.item()) != 0:
        print("trace_run: a token id outside the vocabulary reached the device", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
