"""The generation loop above the step function.

The reference's loop serves one sequence: stop if the current token is a stop token,
prefill or decode, pick the next token, stop if that is a stop token; the stop token is
never handed out (src/libllm/generator.cc:140-156).  This loop does the same for many
requests: it forms batches of unequal prompts, runs each batch's prompts in one step
and then one token per live sequence per step, drops sequences as they end (their
slots and pages go back at once) and starts the next batch when a batch is done."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional, Sequence, Tuple


from ..errors import CacheError, InvalidArgError
from ..sampling.rng import uniform
from .step import Engine, SamplingParams, StepItem


@dataclass
class Request:
    prompt: Sequence[int]
    max_new_tokens: int
    index: int = 0                      # position in the caller's list; also the RNG stream


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: Sequence[int], capacity_tokens: int,
                 max_batch: int, page_size: int = 64, max_seq_len: Optional[int] = None) -> List[List[int]]:
    """Splits requests, in order, into batches that fit the cache when every sequence
    grows to its full length (prompt + new tokens, rounded up to whole pages).  A
    request that cannot fit alone is an error."""
    batches: List[List[int]] = [[]]
    used = 0
    for i, (n, m) in enumerate(zip(prompt_lengths, max_new_tokens)):
        if n < 1:
            raise InvalidArgError(f"request {i}: a prompt needs at least one token")
        if m < 0:
            raise InvalidArgError(f"request {i}: max_new_tokens must not be negative")
        total = n + m
        if max_seq_len is not None and total > max_seq_len:
            raise InvalidArgError(f"request {i}: {n} prompt + {m} new tokens exceed the longest "
                                  f"sequence ({max_seq_len})")
        need = (total + page_size - 1) // page_size * page_size
        if need > capacity_tokens:
            raise CacheError(f"request {i} needs room for {need} tokens, the cache holds {capacity_tokens}")
        if batches[-1] and (used + need > capacity_tokens or len(batches[-1]) >= max_batch):
            batches.append([])
            used = 0
        batches[-1].append(i)
        used += need
    return [b for b in batches if b]


def should_stop(token: int, n_generated: int, max_new_tokens: int, stop_tokens) -> Tuple[bool, bool]:
    """(ends, emit): a stop token ends the sequence and is not emitted; reaching the
    limit ends it after emitting."""
    if token in stop_tokens:
        return True, False
    return n_generated + 1 >= max_new_tokens, True


def generate(engine: Engine, prompts: Sequence[Sequence[int]], max_new_tokens,
             sampling: SamplingParams = SamplingParams(), seed: int = 0,
             stop_tokens: Optional[Iterable[int]] = None, max_batch: int = 64,
             on_token: Optional[Callable[[int, int], None]] = None) -> List[List[int]]:
    """Generated tokens per prompt.  ``max_new_tokens`` is one number or one per prompt;
    ``stop_tokens`` defaults to the model's own (config.json's eos_token_id);
    ``on_token(request index, token)`` is called as tokens arrive."""
    n = len(prompts)
    limits = [max_new_tokens] * n if isinstance(max_new_tokens, int) else list(max_new_tokens)
    if len(limits) != n:
        raise InvalidArgError("max_new_tokens: one number, or one per prompt")
    stops_set = frozenset(engine.model.spec.stop_tokens if stop_tokens is None else stop_tokens)
    sampling.validate()
    out: List[List[int]] = [[] for _ in range(n)]
    capacity = engine.cache.n_pages * engine.page_size
    batches = plan_batches([len(p) for p in prompts], limits, capacity, max_batch, engine.page_size,
                           engine.max_seq_len)
    for batch in batches:
        live = [i for i in batch if limits[i] > 0]
        if not live:
            continue
        slots = {i: engine.open_sequence() for i in live}
        try:
            # The step that is running on the device: (request ids in row order, pending tokens).
            # While the host waits for its tokens, the next step is already queued behind it with
            # every sequence that can still go on; it takes its tokens from the device.  A
            # sequence that turns out to have ended (a stop token) has then run one step too
            # many: its result is dropped and its slot is given back, nothing else sees it.
            produced = {i: 0 for i in live}
            items = [StepItem(slots[i], list(prompts[i]), [len(prompts[i]) - 1]) for i in live]
            running = (live, engine.step_tokens(items, sampling, [uniform(seed, i, 0) for i in live]))
            ended = set()
            while running is not None:
                ids, pending = running
                # queue the next step: the sequences of this one that have not reached their count
                ahead = [(row, i) for row, i in enumerate(ids) if i not in ended and produced[i] + 1 < limits[i]]
                nxt = None
                if ahead:
                    items = [StepItem(slots[i], [0], [0], fed_row=row) for row, i in ahead]
                    uni = [uniform(seed, i, produced[i] + 1) for _, i in ahead]
                    nxt = ([i for _, i in ahead], engine.step_tokens(items, sampling, uni))
                # now this step's tokens (the one device-to-host read of the step)
                for i, tok in zip(ids, pending.result()):
                    if i in ended:
                        continue                    # it ran one step beyond its end
                    stops, emit = should_stop(tok, produced[i], limits[i], stops_set)
                    if emit:
                        out[i].append(tok)
                        produced[i] += 1
                        if on_token is not None:
                            on_token(i, tok)
                    if stops:
                        ended.add(i)
                        engine.close_sequence(slots.pop(i))
                running = nxt
        finally:
            for s in slots.values():
                engine.close_sequence(s)
    return out
