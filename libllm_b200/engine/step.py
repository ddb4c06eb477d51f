"""The step function: a batch of sequences, each bringing its next tokens (a whole
prompt, a piece of one, or a single token), run as one batch from the cache.

The reference has two entry points for one sequence, ``prefill`` and ``decode``
(src/libllm/model_for_generation.h:62-69, src/libllm/llama.cc:349-368), and a
rectangular batch inside the model.  Here one function takes ragged batches: the
tokens of all sequences lie one after another, per-token arrays say which sequence and
position each belongs to, and the kernels index the paged cache with them.  Only the
tokens given are computed; padding does not exist.

Steps in which every sequence brings one token are captured once per batch shape as a
CUDA graph and replayed; the graph's first kernel brings the step's descriptor (tokens,
positions, page tables) from pinned host memory into the graph's fixed buffer, its last
one takes the sampled tokens out.  Prompt steps whose shape comes back are captured too."""
from __future__ import annotations

import gc
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import KVCache
from ..csrc import ops
from ..errors import InvalidArgError
from ..parts.base import StepContext
from .model import Model


@dataclass
class StepItem:
    """One sequence's share of a step: its slot, its next tokens, and the places among
    these tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()
    fed_row: Optional[int] = None      # its one token is the one the previous step sampled for this row


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 is greedy; top_k 0 draws from the whole vocabulary.  The defaults
    are the reference's (src/libllm/llm.cc:125-132)."""
    temperature: float = 1.0
    top_k: int = 50
    top_p: float = 0.8

    def validate(self) -> None:
        if self.temperature < 0:
            raise InvalidArgError("temperature must not be negative")
        if not 0 <= self.top_k <= 1024:
            raise InvalidArgError("top_k must lie in 0..1024 (0: the whole vocabulary)")
        if not self.top_p > 0:
            raise InvalidArgError("top_p must be positive")
        if self.top_k == 0 and self.top_p < 1.0 and self.temperature > 0:
            raise InvalidArgError("top_p below 1 needs a top_k")


GREEDY = SamplingParams(temperature=0.0, top_k=1, top_p=1.0)


@dataclass
class _Piece:
    """Part of one item that runs in one launch sequence."""
    index: int          # index of the item in the step
    slot: int
    start: int          # offset into the item's tokens
    count: int
    past: int           # tokens cached before this piece


class _Descriptor:
    """Host staging and device copy of one step's integer arrays."""

    def __init__(self, device, n_tokens: int, n_seqs: int, n_want: int, widths: List[int]):
        self.n_tokens, self.n_seqs, self.n_want, self.widths = n_tokens, n_seqs, n_want, widths
        T, B, W = n_tokens, n_seqs, n_want
        sizes = [T, T, T, B + 1, B, B, W, B, T] + [B * w for w in widths]
        self.offsets = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])]).astype(int)
        total = int(self.offsets[-1])
        self.host = torch.empty(total, dtype=torch.int32, pin_memory=True)
        self.host.zero_()
        self.np = self.host.numpy()
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        self.copied = torch.cuda.Event()
        self._pending = False
        self._sizes = sizes

    def field(self, i: int, dev: bool = False):
        a, n = int(self.offsets[i]), self._sizes[i]
        return (self.dev if dev else self.np)[a:a + n]

    def wait_host_free(self) -> None:
        if self._pending:
            self.copied.synchronize()
            self._pending = False

    def upload(self) -> None:
        self.dev.copy_(self.host, non_blocking=True)
        self.in_flight()

    def in_flight(self) -> None:
        """What was launched up to here reads the host staging (a copy, or a graph that copies
        by itself): the staging is free again when that has run."""
        self.copied.record()
        self._pending = True


class Engine:
    def __init__(self, model: Model, max_tokens: int, max_seq_len: Optional[int] = None,
                 max_slots: Optional[int] = None, max_step_tokens: int = 8192, page_size: int = 64,
                 use_graphs: bool = True):
        """``max_tokens``: tokens all live sequences may hold together (each sequence's
        count rounded up to a multiple of ``page_size``); it sizes the cache."""
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        self.page_size = page_size
        n_pages = (max_tokens + page_size - 1) // page_size
        self.max_seq_len = min(max_seq_len or model.max_positions, model.max_positions, n_pages * page_size)
        self.max_step_tokens = max(1, max_step_tokens)
        self.use_graphs = use_graphs
        self.cache = KVCache(model.run_cache_needs(), model.run_state_needs(), max_tokens, self.dtype,
                             self.device, page_size, max_slots)
        self.vocab = model.spec.vocab_size
        # The tokens the last sampling step drew, kept on the device: the next step can take them
        # from here (StepItem.fed_row) while the host is still reading them back.
        self.last_tokens = torch.zeros(max(self.max_step_tokens, 1024), dtype=torch.int32, device=self.device)
        self._token_buffers = [torch.empty(self.last_tokens.numel(), dtype=torch.int32, pin_memory=True)
                               for _ in range(4)]
        self._token_turn = 0
        self._graphs: Dict[tuple, "_DecodeGraph"] = {}
        # A single-token step's graph holds its own copies (descriptor in, tokens out), so a step is one
        # launch.  Each shape has two graphs taken in turn: while one step runs, the next one's
        # descriptor is written into the other graph's staging, and a step's tokens are read
        # while the other graph's step runs.
        self._graphs_alt: Dict[tuple, "_DecodeGraph"] = {}
        self._graph_turn: Dict[tuple, int] = {}
        self._last_decode_graph: Optional["_DecodeGraph"] = None
        # Prompt steps whose shape comes back (batches of equal prompts, a benchmark's repetitions)
        # are captured too, from their second occurrence on; a few are kept, the oldest goes.
        self._prompt_graphs: "OrderedDict[tuple, _StepGraph]" = OrderedDict()
        self._prompt_seen: Dict[tuple, int] = {}
        self.max_prompt_graphs = 4
        self.prompt_graph_max_tokens = 2048      # longer steps gain nothing that pays for the capture
        self._eager_desc: Dict[tuple, _Descriptor] = {}
        self.launch_log: Optional[List[str]] = None
        self.steps_run = 0

    # ---------------------------------------------------------------- sequences
    def open_sequence(self) -> int:
        return self.cache.open()

    def close_sequence(self, slot: int) -> None:
        self.cache.close(slot)

    def sequence_length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---------------------------------------------------------------- the step
    def step(self, items: Sequence[StepItem], sampling: Optional[SamplingParams] = None,
             uniforms: Optional[Sequence[float]] = None, return_logits: bool = True):
        """Runs the items' tokens and returns the logits at the wanted places, a 32-bit
        device tensor [wanted, vocab] in the order of the items and of their ``want``.
        With ``sampling`` it returns (logits or None, tokens): a token drawn at each
        wanted place (int32 on the device); ``uniforms`` then holds one number in [0, 1)
        per wanted place.  What a step of single tokens returns lies in its graph's buffers,
        which the step after next of the same shape writes again: copy what is to be kept."""
        items = list(items)
        if not items:
            raise InvalidArgError("a step needs at least one sequence")
        self._validate(items)
        n_want = sum(len(it.want) for it in items)
        if sampling is not None:
            sampling.validate()
            if uniforms is None:
                uniforms = [0.0] * n_want
            if len(uniforms) != n_want:
                raise InvalidArgError("one uniform number per wanted place is needed")
        # Pages first: either the whole step fits the cache or nothing changes.
        self.cache.reserve({it.slot: self.cache.length(it.slot) + len(it.tokens) for it in items})

        decode_only = all(len(it.tokens) == 1 for it in items)
        out = None
        if decode_only and self.use_graphs and len(items) <= self.max_step_tokens:
            out = self._run_decode_graph(items, sampling, uniforms, return_logits)
        elif self.use_graphs:
            out = self._run_prompt_graph(items, sampling, uniforms, return_logits)     # None: not this time
        if out is None:
            out = self._run_eager(items, sampling, uniforms, return_logits)
        self.steps_run += 1
        return out

    def step_tokens(self, items: Sequence[StepItem], sampling: SamplingParams,
                    uniforms: Optional[Sequence[float]] = None) -> "PendingTokens":
        """Runs a step that samples one token per item (each wants exactly one place) and returns
        at once: the tokens stay on the device in ``last_tokens`` (row i = item i), where the next
        step's items may take them from (``StepItem.fed_row``), and are on their way to pinned
        host memory; ``PendingTokens.result()`` waits for that copy."""
        items = list(items)
        if any(len(it.want) != 1 for it in items):
            raise InvalidArgError("step_tokens: every item wants exactly one place")
        n = len(items)
        if n > self.last_tokens.numel():
            raise InvalidArgError(f"step_tokens: {n} sequences, at most {self.last_tokens.numel()} are taken")
        self._last_decode_graph = None
        _, tokens = self.step(items, sampling, uniforms, return_logits=False)
        g = self._last_decode_graph
        if g is not None and g.host_tokens is not None and tokens.data_ptr() == self.last_tokens.data_ptr():
            # the graph has copied them out itself; its buffer is read before the graph runs again
            return PendingTokens(n, g.host_tokens, g.desc.copied)
        if tokens.data_ptr() != self.last_tokens.data_ptr():
            self.last_tokens[:n].copy_(tokens)
        host = self._token_buffers[self._token_turn]
        self._token_turn = (self._token_turn + 1) % len(self._token_buffers)
        host[:n].copy_(self.last_tokens[:n], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return PendingTokens(n, host, done)

    def _validate(self, items: Sequence[StepItem]) -> None:
        seen = set()
        for it in items:
            if it.slot in seen:
                raise InvalidArgError(f"slot {it.slot} appears twice in one step")
            seen.add(it.slot)
            n = len(it.tokens)
            if n == 0:
                raise InvalidArgError(f"slot {it.slot}: a sequence in a step brings at least one token")
            past = self.cache.length(it.slot)       # raises if the slot is not open
            if past + n > self.max_seq_len:
                raise InvalidArgError(f"slot {it.slot}: {past} + {n} tokens exceed the longest sequence "
                                      f"this engine holds ({self.max_seq_len})")
            if it.fed_row is not None:
                if n != 1 or not 0 <= it.fed_row < self.last_tokens.numel():
                    raise InvalidArgError(f"slot {it.slot}: a fed token is one token from a row of the last step")
            else:
                for t in it.tokens:
                    if not 0 <= int(t) < self.vocab:
                        raise InvalidArgError(f"slot {it.slot}: token id {t} outside the vocabulary ({self.vocab})")
            for w in it.want:
                if not 0 <= int(w) < n:
                    raise InvalidArgError(f"slot {it.slot}: wanted place {w} outside the {n} tokens given")

    # ---------------------------------------------------------------- descriptor
    def _fill(self, desc: _Descriptor, pieces: List[_Piece], items: Sequence[StepItem],
              want_rows: List[int], uniforms: Optional[Sequence[float]], upload: bool = True) -> None:
        desc.wait_host_free()
        tokens, tok_seq, tok_pos = desc.field(0), desc.field(1), desc.field(2)
        seq_start, seq_past, seq_slot = desc.field(3), desc.field(4), desc.field(5)
        want, uni, fed = desc.field(6), desc.field(7), desc.field(8)
        o = 0
        for b, p in enumerate(pieces):
            it = items[p.index]
            if it.fed_row is not None:
                tokens[o] = 0
                fed[o] = it.fed_row
            else:
                tokens[o:o + p.count] = it.tokens[p.start:p.start + p.count]
                fed[o:o + p.count] = -1
            tok_seq[o:o + p.count] = b
            tok_pos[o:o + p.count] = np.arange(p.past + p.start, p.past + p.start + p.count)
            seq_start[b] = o
            seq_past[b] = p.past + p.start
            seq_slot[b] = p.slot
            o += p.count
        seq_start[len(pieces)] = o
        want[:len(want_rows)] = want_rows
        if uniforms is not None:
            uni.view(np.float32)[:len(uniforms)] = np.asarray(uniforms, dtype=np.float32)
        slots = [p.slot for p in pieces]
        for g, w in enumerate(desc.widths):
            desc.field(9 + g).reshape(len(pieces), w)[:] = self.cache.page_table(g, slots, w)
        if upload:
            desc.upload()

    def _context(self, desc: _Descriptor, pieces: List[_Piece], n_want: int, decode_only: bool,
                 max_kv_len: int) -> Tuple[StepContext, List[torch.Tensor]]:
        B = len(pieces)
        ctx = StepContext(
            dtype=self.dtype, device=self.device, n_tokens=desc.n_tokens, n_seqs=B,
            tokens=desc.field(0, True), tok_seq=desc.field(1, True), tok_pos=desc.field(2, True),
            seq_start=desc.field(3, True), seq_past=desc.field(4, True), seq_slot=desc.field(5, True),
            want_rows=desc.field(6, True)[:n_want], q_lens=[p.count for p in pieces],
            past_lens=[p.past + p.start for p in pieces], slots=[p.slot for p in pieces],
            max_q_len=max(p.count for p in pieces), max_kv_len=max_kv_len, decode_only=decode_only)
        ctx.extras["uniforms"] = desc.field(7, True).view(torch.float32)
        ctx.extras["fed"] = (self.last_tokens, desc.field(8, True))
        tables = [desc.field(9 + g, True).view(B, w) for g, w in enumerate(desc.widths)]
        return ctx, tables

    def _sample(self, logits: torch.Tensor, sampling: SamplingParams, uniforms: torch.Tensor,
                into_last: bool = False) -> torch.Tensor:
        if into_last and logits.shape[0] <= self.last_tokens.numel():
            out = self.last_tokens[:logits.shape[0]]
        else:
            out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        if sampling.temperature == 0:
            return ops.argmax(logits, out)
        return ops.sample(logits, sampling.temperature, sampling.top_k, sampling.top_p, uniforms, out)

    # ---------------------------------------------------------------- eager path (prompts, mixed steps)
    def _run_eager(self, items, sampling, uniforms, return_logits):
        pieces_all: List[List[_Piece]] = [[]]
        room = self.max_step_tokens
        for i, it in enumerate(items):
            past = self.cache.length(it.slot)
            start, n = 0, len(it.tokens)
            while start < n:
                if room == 0:
                    pieces_all.append([])
                    room = self.max_step_tokens
                c = min(room, n - start)
                pieces_all[-1].append(_Piece(i, it.slot, start, c, past))
                start += c
                room -= c
        logits_parts, token_parts = [], []
        want_base = np.cumsum([0] + [len(it.want) for it in items])
        order: List[int] = []          # index into the flat wanted list, in the order computed
        for pieces in pieces_all:
            T = sum(p.count for p in pieces)
            want_rows, uni = [], []
            o = 0
            for p in pieces:
                for j, w in enumerate(items[p.index].want):
                    if p.start <= w < p.start + p.count:
                        want_rows.append(o + w - p.start)
                        order.append(int(want_base[p.index]) + j)
                        if uniforms is not None:
                            uni.append(uniforms[int(want_base[p.index]) + j])
                o += p.count
            widths = [self._table_width(pieces)] * len(self.cache.groups)
            desc = self._eager_descriptor(T, len(pieces), len(want_rows), widths)
            self._fill(desc, pieces, items, want_rows, uni if uniforms is not None else None)
            max_kv = max(p.past + p.start + p.count for p in pieces)
            ctx, tables = self._context(desc, pieces, len(want_rows), all(p.count == 1 for p in pieces), max_kv)
            logits = self.model.forward(ctx, self.cache, tables)
            if sampling is not None and len(want_rows):
                token_parts.append(self._sample(logits, sampling, ctx.extras["uniforms"]))
            if return_logits or sampling is None:
                logits_parts.append(logits)
            for p in pieces:
                self.cache.commit(p.slot, p.past + p.start + p.count)
            desc.wait_host_free()
        perm = None
        if order != sorted(order):
            perm = torch.tensor(np.argsort(order), device=self.device)
        logits = None
        if logits_parts:
            logits = logits_parts[0] if len(logits_parts) == 1 else torch.cat(logits_parts, 0)
            if perm is not None:
                logits = logits[perm]
        if sampling is None:
            return logits
        if token_parts:
            tokens = token_parts[0] if len(token_parts) == 1 else torch.cat(token_parts, 0)
        else:
            tokens = torch.empty(0, dtype=torch.int32, device=self.device)
        if perm is not None:
            tokens = tokens[perm]
        return (logits if return_logits else None), tokens

    def _eager_descriptor(self, T: int, B: int, W: int, widths: List[int]) -> _Descriptor:
        """Staging buffers are kept per shape: pinned allocations are slow to make."""
        key = (T, B, W, tuple(widths))
        desc = self._eager_desc.get(key)
        if desc is None:
            if len(self._eager_desc) >= 64:
                self._eager_desc.pop(next(iter(self._eager_desc)))
            desc = self._eager_desc[key] = _Descriptor(self.device, T, B, W, widths)
        return desc

    def _table_width(self, pieces: List[_Piece]) -> int:
        need = max((p.past + p.start + p.count + self.page_size - 1) // self.page_size for p in pieces)
        return max(8, (need + 7) // 8 * 8)

    # ---------------------------------------------------------------- graph path (one token each)
    def _run_decode_graph(self, items, sampling, uniforms, return_logits):
        B = len(items)
        pieces = [_Piece(i, it.slot, 0, 1, self.cache.length(it.slot)) for i, it in enumerate(items)]
        need_pages = max((p.past + 1 + self.page_size - 1) // self.page_size for p in pieces)
        width = 8
        while width < need_pages:
            width *= 2
        key = (B, width, sampling)
        turn = self._graph_turn.get(key, 0)
        self._graph_turn[key] = turn ^ 1
        table = self._graphs if turn == 0 else self._graphs_alt
        graph = table.get(key)
        if graph is None:
            graph = table[key] = _DecodeGraph(self, B, width, sampling)
        # Logits are computed for every sequence; the wanted ones are picked afterwards.
        rows = [i for i, it in enumerate(items) if len(it.want)]
        uni_full = None
        if sampling is not None:
            uni_full = [0.0] * B
            for r, u in zip(rows, uniforms):
                uni_full[r] = u
        self._fill(graph.desc, pieces, items, list(range(B)), uni_full, upload=False)
        graph.run()
        graph.desc.in_flight()                 # the staging is free, and the tokens are out, when this launch is done
        self._last_decode_graph = graph
        for p in pieces:
            self.cache.commit(p.slot, p.past + 1)
        pick = None if len(rows) == B else torch.tensor(rows, device=self.device, dtype=torch.long)
        logits = graph.logits if pick is None else graph.logits[pick]
        if sampling is None:
            return logits
        tokens = graph.tokens if pick is None else graph.tokens[pick]
        return (logits if return_logits else None), tokens

    # ---------------------------------------------------------------- graph path (prompts whose shape repeats)
    def _run_prompt_graph(self, items, sampling, uniforms, return_logits):
        """A prompt step as a graph replay, or None when it is to run eagerly: the step must be short
        (the host issues a step's 130-odd launches in 2 to 4 ms, which is what a graph saves; a
        capture costs 30 to 50 ms, and hundreds where its buffers are gigabytes), want few places,
        and have a shape that was seen before.  The shape is
        what the launches depend on: tokens and sequences in the step, places wanted, the page
        tables' width and the longest prompt rounded up to the attention kernel's tile of rows.
        Which sequence has how many tokens, and where they stand, is in the descriptor."""
        T = sum(len(it.tokens) for it in items)
        n_want = sum(len(it.want) for it in items)
        if T > min(self.max_step_tokens, self.prompt_graph_max_tokens) or n_want == 0 or n_want > 64 or len(items) > 1024:
            return None
        pieces = [_Piece(i, it.slot, 0, len(it.tokens), self.cache.length(it.slot)) for i, it in enumerate(items)]
        need_pages = max((p.past + p.count + self.page_size - 1) // self.page_size for p in pieces)
        width = 8
        while width < need_pages:
            width *= 2
        max_q = (max(p.count for p in pieces) + 127) // 128 * 128
        key = (T, len(items), n_want, width, max_q, sampling)
        graph = self._prompt_graphs.get(key)
        if graph is None:
            seen = self._prompt_seen.get(key, 0) + 1
            if len(self._prompt_seen) > 4096:
                self._prompt_seen.clear()
            self._prompt_seen[key] = seen
            if seen < 2:
                return None
            while len(self._prompt_graphs) >= self.max_prompt_graphs:
                torch.cuda.synchronize()
                self._prompt_graphs.popitem(last=False)
            graph = self._prompt_graphs[key] = _StepGraph(self, T, len(items), n_want, width, max_q, sampling)
        else:
            self._prompt_graphs.move_to_end(key)
        want_rows, o = [], 0
        for p in pieces:
            want_rows.extend(o + w for w in items[p.index].want)
            o += p.count
        self._fill(graph.desc, pieces, items, want_rows, list(uniforms) if sampling is not None else None)
        graph.run()
        for p in pieces:
            self.cache.commit(p.slot, p.past + p.count)
        # a prompt step's results are the caller's own (as the eager path's are): not the graph's buffers
        logits = graph.logits.clone() if (return_logits or sampling is None) else None
        if sampling is None:
            return logits
        return logits, graph.tokens.clone()


class PendingTokens:
    """Tokens of a step on their way from the device to the host."""

    def __init__(self, n: int, host: torch.Tensor, done: "torch.cuda.Event"):
        self.n, self._host, self._done = n, host, done

    def result(self) -> List[int]:
        self._done.synchronize()
        return self._host[:self.n].tolist()


class _StepGraph:
    """A captured step of T tokens of B sequences with ``n_want`` wanted places, page tables
    ``width`` wide and no sequence bringing more than ``max_q`` tokens."""

    def __init__(self, engine: Engine, T: int, B: int, n_want: int, width: int, max_q: int,
                 sampling: Optional[SamplingParams], decode_only: bool = False):
        self.engine, self.T, self.B, self.n_want, self.width, self.max_q = engine, T, B, n_want, width, max_q
        self.sampling, self.decode_only = sampling, decode_only
        self.desc = _Descriptor(engine.device, T, B, n_want, [width] * len(engine.cache.groups))
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.tokens: Optional[torch.Tensor] = None
        # single-token steps carry their copies inside the graph
        self.host_tokens = (torch.empty(B, dtype=torch.int32, pin_memory=True)
                            if decode_only and sampling is not None else None)

    def _body(self):
        eng = self.engine
        if self.decode_only:
            ops.copy_words(self.desc.host, self.desc.dev, self.desc.host.numel())
        # stand-in pieces: the launches depend on the step's shape alone
        pieces = [_Piece(i, 0, 0, 1, 0) for i in range(self.B)]
        ctx, tables = eng._context(self.desc, pieces, self.n_want, self.decode_only, self.width * eng.page_size)
        ctx.max_q_len = self.max_q
        logits = eng.model.forward(ctx, eng.cache, tables)
        tokens = None
        if self.sampling is not None:
            tokens = eng._sample(logits, self.sampling, ctx.extras["uniforms"], into_last=self.decode_only)
            if self.host_tokens is not None:
                ops.copy_words(tokens, self.host_tokens, self.B)
        return logits, tokens

    def run(self) -> None:
        if self.graph is None:
            # First use: the step runs once outside capture (which also loads kernels and
            # sizes library workspaces) and its results are this call's results; then the
            # same launches are captured, which executes nothing.  The step must not run
            # twice: a mixer with state of its own would advance twice.
            side = torch.cuda.Stream(device=self.engine.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                logits, tokens = self._body()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            # Nothing but the step's own launches may happen while it is captured.  Python's
            # garbage collector could otherwise pick this moment to destroy CUDA objects of an
            # engine dropped earlier (graphs, events, pinned buffers), and a call such as a free
            # from a destructor invalidates the capture.
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
                    self._static = self._body()
            finally:
                if gc_was_on:
                    gc.enable()
            self.logits, self.tokens = logits, tokens
            return
        self.graph.replay()
        self.logits, self.tokens = self._static


class _DecodeGraph(_StepGraph):
    """A captured step of B sequences bringing one token each, page tables ``width`` wide."""

    def __init__(self, engine: Engine, B: int, width: int, sampling: Optional[SamplingParams]):
        super().__init__(engine, B, B, B, width, 1, sampling, decode_only=True)
