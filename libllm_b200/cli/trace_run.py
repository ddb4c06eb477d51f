"""Trace replay: feeds given token ids through a model step by step and writes logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps are read from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at the
wanted places, in the order of the entries and of ``want``, as little-endian 32-bit
floats [wanted, vocab].  After every step ``done <step>`` is printed and flushed.

It samples nothing and has no forward pass, cache or loader of its own: it drives the
host library's model, step function and cache (C++), the ones generation uses.  The reference's
nearest thing is the test that feeds stored token ids and compares stored logits
(src/libllm/llama_test.cc:143-190) and its token-by-token loop (:211-216)."""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--no-graphs", action="store_true", help="do not capture single-token steps as CUDA graphs")
    args = ap.parse_args(argv)

    from libllm_b200.engine import Engine, StepItem

    os.makedirs(args.out, exist_ok=True)
    engine = Engine.from_folder(args.model, dtype=args.dtype, max_tokens=args.max_tokens, use_graphs=not args.no_graphs,
                                max_seq_len=max(64, (args.max_tokens + 63) // 64 * 64))
    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        items = []
        for e in rec["entries"]:
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.open_sequence()
            items.append(StepItem(slots[rid], e["tokens"], e.get("want", [])))
        if items:
            logits = engine.step(items)          # float32 [wanted, vocab] in host memory, the step complete
            if logits is not None and logits.shape[0] > 0:
                with open(os.path.join(args.out, f"{rec['step']}.f32"), "wb") as f:
                    f.write(logits.astype("<f4", copy=False).tobytes())
        for rid in rec.get("end", []):
            if rid in slots:
                engine.close_sequence(slots.pop(rid))
        print(f"done {rec['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
