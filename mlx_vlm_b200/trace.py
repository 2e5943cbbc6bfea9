"""Replay a trace of token ids through a model, step by step, and write the logits that the trace asks for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input: one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries`: for each request its next tokens and the places among them whose logits are wanted; all entries of a
step are ONE batch of the model's step function.  `end`: requests that are finished after the step (their cache
slot is released and used again).  Output: DIR/<step>.f32 = little-endian fp32 [wanted, vocab] for every step
that wants something, and a line `done <step>` on standard output after every step.

Nothing is sampled.  The model class is chosen by config.json (utils.load_model); the cache is the model's own
pool with one slot per live request; the step is `language_model.step`, the function under `__call__`,
`prefill_rows` and the batch scheduler.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, default=0, help="most tokens that live requests hold at any time")
    a = ap.parse_args(argv)

    import numpy as np
    import torch
    from .models.cache import SlotTable
    from .utils import load_model

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device (there is no CPU path)", file=sys.stderr)
        return 2
    model = load_model(a.model, dtype=a.dtype, strict=False)     # tensors the configuration does not name are ignored
    lm = model.language_model
    if not hasattr(lm, "step"):
        print(f"trace_run: {type(model).__module__} has no token-level step function", file=sys.stderr)
        return 3
    eng = model.engine
    os.makedirs(a.out, exist_ok=True)
    n_slots = 4
    pool = lm.make_pool(rows=n_slots, capacity=min(max(a.max_tokens, 1), 4096))
    slots = SlotTable(n_slots)
    caches = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        entries = st.get("entries", [])
        for e in entries:
            if e["id"] not in caches:
                if not slots.free:
                    eng.stream.synchronize()
                    with torch.cuda.stream(eng.stream):
                        pool.add_slots(2 * slots.n_slots, live_tokens=pool.capacity)
                    slots.grow(pool.batch)
                caches[e["id"]] = lm.make_cache_row(pool, slots.acquire(e["id"]))
        if entries:
            logits = lm.step([e["tokens"] for e in entries], [caches[e["id"]] for e in entries],
                             want=[e.get("want", []) for e in entries])
            if logits.shape[0]:
                with torch.cuda.stream(eng.stream):
                    host = logits.to("cpu", non_blocking=False)
                eng.stream.synchronize()
                tmp = os.path.join(a.out, f".{st['step']}.part")
                host.numpy().astype("<f4").tofile(tmp)
                os.replace(tmp, os.path.join(a.out, f"{st['step']}.f32"))
        for rid in st.get("end", []):
            if rid in caches:
                del caches[rid]
                slots.release(rid)
        sys.stdout.write(f"done {st['step']}\n")
        sys.stdout.flush()
    eng.stream.synchronize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
