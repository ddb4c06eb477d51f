"""Drives the engine the way a trace does: batches of requests that start together with
their prompts and go on by one token each; shorter requests end earlier."""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

from libllm_b200.engine import Engine, StepItem


def replay_batch(engine: Engine, requests: Sequence[Tuple[str, List[int], int]]) -> Dict[str, torch.Tensor]:
    """``requests``: (id, all tokens, prompt length).  The prompt goes in one step, the rest
    one token a step.  Returns id -> logits [len(tokens), vocab] (CPU, float32)."""
    slots = {rid: engine.open_sequence() for rid, _, _ in requests}
    rows: Dict[str, List[torch.Tensor]] = {rid: [] for rid, _, _ in requests}
    fed = {rid: 0 for rid, _, _ in requests}
    live = list(requests)
    first = True
    while live:
        items, ids = [], []
        for rid, toks, n_prompt in live:
            n = n_prompt if first else 1
            piece = toks[fed[rid]:fed[rid] + n]
            items.append(StepItem(slots[rid], piece, list(range(len(piece)))))
            ids.append((rid, len(piece)))
        logits = torch.from_numpy(engine.step(items))
        o = 0
        for rid, n in ids:
            rows[rid].append(logits[o:o + n])
            fed[rid] += n
            o += n
        nxt = []
        for r in live:
            if fed[r[0]] >= len(r[1]):
                engine.close_sequence(slots.pop(r[0]))
            else:
                nxt.append(r)
        live = nxt
        first = False
    engine.cache_check()
    return {rid: torch.cat(v, 0) for rid, v in rows.items()}
