"""The ``llm`` command line, in the manner of the reference's (go/bin/main.go:37-53):

    llm chat -m FOLDER [-device auto|cuda] [-dtype bfloat16|float32]
    llm generate -m FOLDER --prompt-ids 1,2,3 [--prompt-ids ...] [--max-new-tokens N]
                 [--temperature T] [--top-k K] [--top-p P] [--seed S] [--no-stop]

``chat`` is the reference's loop (go/bin/chat.go:67-131): a prompt per line, ``:new`` starts a
new session, ``:sys TEXT`` sets what every session starts with, and after each reply a line
with the number of tokens, the time and the milliseconds per token.  Text is not part of
this library, so a line is a list of token ids (separated by spaces or commas) and the
reply is printed as ids; a session keeps its history and every turn runs the whole
history again, as the reference's chat does (go/bin/chat.go:107-112).  The sampler's
defaults are the reference's: temperature 1.0, top_k 50, top_p 0.8 (src/libllm/llm.cc:125-132).
``generate`` does not exist in the reference: it is the batched entry point on the
command line, one prompt per ``--prompt-ids``; each reply is one line of ids on standard
output.  ``download`` is not built (no network; model folders are local)."""
from __future__ import annotations

import argparse
import sys
import time
from typing import List


def parse_ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def usage() -> None:
    e = sys.stderr
    print("Usage: llm COMMAND", file=e)
    print("", file=e)
    print("Commands:", file=e)
    print("    chat           Chat with LLM (token ids in, token ids out)", file=e)
    print("    generate       Generate continuations of one or more prompts", file=e)
    print("", file=e)
    print("Run 'llm COMMAND -h' for more information on a command.", file=e)


def add_common(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("-m", "--model", dest="model", required=True,
                    help="the model folder (config.json and model.safetensors)")
    ap.add_argument("-device", "--device", dest="device", default="auto", choices=["auto", "cuda", "cpu"],
                    help="inference device, either cuda or auto (there is no cpu path)")
    ap.add_argument("-dtype", "--dtype", dest="dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-tokens", type=int, default=65536, help="tokens the cache holds")
    ap.add_argument("--max-seq-len", type=int, default=None, help="longest sequence (default: the model's)")


def load(args):
    from .. import Device, Model
    device = {"auto": Device.AUTO, "cuda": Device.CUDA, "cpu": Device.CPU}[args.device]
    return Model(args.model, device=device, dtype=args.dtype, max_tokens=args.max_tokens,
                 max_seq_len=args.max_seq_len)


def chat_main(argv) -> int:
    ap = argparse.ArgumentParser(prog="llm chat")
    add_common(ap)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.8)
    ap.add_argument("--max-new-tokens", type=int, default=256)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    model = load(args)
    print("Please input your question (token ids).")
    print("    Type ':new' to start a new session (clean history).")
    print("    Type ':sys <ids>' to set the system prompt and start a new session .")
    history: List[int] = []
    system: List[int] = []
    turn = 0
    while True:
        print("> ", end="", flush=True)
        line = sys.stdin.readline()
        if not line:
            print()
            break
        q = line.strip()
        if len(q) > 5 and q[:5].lower() == ":sys ":
            system, history = parse_ids(q[5:]), []
            continue
        if q.lower() == ":new":
            print("===== new session =====")
            history = []
            continue
        if not q:
            continue
        try:
            ids = parse_ids(q)
        except ValueError:
            print("a line is a list of token ids, ':new' or ':sys <ids>'", file=sys.stderr)
            continue
        if not history and system:
            history = list(system)
        history += ids
        t0 = time.time()
        answer = []
        for chunk in model.complete(history, top_k=args.top_k, top_p=args.top_p, temperature=args.temperature,
                                    max_new_tokens=args.max_new_tokens, seed=args.seed + turn):
            print(chunk.token, end=" ", flush=True)
            answer.append(chunk.token)
        print()
        history += answer
        turn += 1
        dur = time.time() - t0
        n = max(1, len(answer))
        print(f"({len(answer)} tokens, time={dur:.2f}s, {dur * 1000 / n:.2f}ms per token)")
    return 0


def generate_main(argv) -> int:
    ap = argparse.ArgumentParser(prog="llm generate")
    add_common(ap)
    ap.add_argument("--prompt-ids", action="append", required=True, help="a prompt as token ids; may be repeated")
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=1.0, help="0 is greedy")
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.8)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-stop", action="store_true", help="ignore the model's stop tokens")
    ap.add_argument("--stop-ids", default=None, help="stop tokens instead of the model's own")
    args = ap.parse_args(argv)
    prompts = [parse_ids(p) for p in args.prompt_ids]
    model = load(args)
    stops = [] if args.no_stop else (parse_ids(args.stop_ids) if args.stop_ids else None)
    t0 = time.time()
    out = model.generate(prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                         top_k=args.top_k, top_p=args.top_p, seed=args.seed, stop_token_ids=stops)
    dur = time.time() - t0
    n = sum(len(o) for o in out)
    print(f"({n} tokens, time={dur:.2f}s, {dur * 1000 / max(1, n):.2f}ms per token)", file=sys.stderr)
    for o in out:
        print(",".join(map(str, o)))
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        usage()
        return 1
    command, rest = argv[0], argv[1:]
    from ..errors import LlmError
    try:
        if command == "chat":
            return chat_main(rest)
        if command == "generate":
            return generate_main(rest)
    except LlmError as e:
        print(f"llm: {e}", file=sys.stderr)
        return 1
    print(f'Invalid command "{command}"\n', file=sys.stderr)
    usage()
    return 1


if __name__ == "__main__":
    sys.exit(main())
