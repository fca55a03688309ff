"""Trace replay: feed given token ids through a model step by step and write the logits of chosen places.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps arrive on standard input, one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}

Every entry appends tokens to its request (admitted at its first entry); all entries of a step run as ONE
batch through the engine's own step builder, paged cache, recurrent-state slots and kernels
(`b200q_engine_step_replay`) — portions of prompts beside single tokens.  Nothing is sampled.  For a step
with wanted places `<out>/<step>.f32` receives their logits, little-endian fp32 [wanted, vocab], in the
order of the entries; after every step the line `done <step>` is printed.  Requests listed in "end" give
their pages and state slot back.  The cache pool holds --max-tokens tokens (rounded up to whole pages)
and there are state slots for MAX_LIVE requests.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

MAX_LIVE = 4


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to whole pages)")
    ap.add_argument("--max-live", type=int, default=MAX_LIVE, help="requests that may be live at once")
    a = ap.parse_args(argv)

    from . import lib as L

    L.ensure_built()
    import numpy as np
    import torch

    from .model import BLOCK_SIZE, Engine, NativeModel, checkpoint_engine_weights, resolve_model

    spec, model_dir = resolve_model(a.model)
    dtype = torch.float32 if a.dtype == "float32" else torch.bfloat16
    if dtype == torch.float32 and not getattr(spec, "layered", False):
        print(f"{spec.arch}: no float32 path for this architecture", file=sys.stderr)
        return 3
    L.require_device()
    torch.cuda.set_device(0)
    # a request's pages are whole: every live request may waste up to one page
    num_blocks = (a.max_tokens + BLOCK_SIZE - 1) // BLOCK_SIZE + a.max_live
    budget = max(a.max_tokens, 16)
    model = NativeModel(spec, checkpoint_engine_weights(spec, model_dir), max_tokens=budget, max_seqs=a.max_live,
                        max_model_len=max(a.max_tokens, 2), num_blocks=num_blocks, dtype=dtype,
                        max_logit_rows=budget)
    eng = Engine(model, max_num_seqs=a.max_live, max_num_batched_tokens=budget, max_model_len=model.max_model_len)
    ids, next_id = {}, 0   # request name -> engine id; ids are never used twice
    out = sys.stdout
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        entries = []
        for e in st["entries"]:
            if e["id"] not in ids:
                next_id += 1
                ids[e["id"]] = next_id
            entries.append((ids[e["id"]], e["tokens"], e.get("want") or []))
        if entries:
            logits = eng.step_replay(entries)
            if logits.shape[0]:
                tmp = os.path.join(a.out, f".{st['step']}.f32.tmp")
                logits.astype("<f4", copy=False).tofile(tmp)
                os.replace(tmp, os.path.join(a.out, f"{st['step']}.f32"))
        for name in st.get("end") or []:
            if name in ids:
                eng.abort(ids.pop(name))
        out.write(f"done {st['step']}\n")
        out.flush()
    eng.close()
    model.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
