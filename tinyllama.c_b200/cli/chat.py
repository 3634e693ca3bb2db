"""chat: a multi-turn loop over one sequence (chat.c:201-355).

    bin/chat -m DIR [-n 393216] [-t 0.8 ...]

Every input line is a turn given as token ids; it is appended to the sequence at its current
position (history is never recomputed, chat.c:296), then tokens are generated until a stop
token, the token budget or a full context (chat.c:315-339).  `/clear` starts a new sequence
(chat.c:265-270), `/quit` ends the program.  The reference wraps turns in a chat template
(tokenizer.c:321-373); with token ids in and out, templates are the caller's business.
"""
from __future__ import annotations

import argparse
import sys

from .options import add_common, parse_ids, sampling_params


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="chat", description=__doc__.split("\n\n")[0])
    add_common(ap, default_tokens=393216)
    ap.add_argument("-s", "--system", default=None, help="token ids that open every new sequence")
    ap.add_argument("-nt", "--no-thinking", action="store_true", help="ignored (a template switch of the reference)")
    args = ap.parse_args(argv)
    import tinyllama_c_b200 as tlc
    ctx = args.ctx if args.ctx > 0 else 0
    llm = tlc.LLM(args.model, dtype=args.dtype, max_tokens=ctx or 4096, max_seqs=1)
    llm.max_context = ctx = min(ctx or llm.max_context, llm.max_context)
    params = sampling_params(args)
    system = parse_ids(args.system) if args.system else []
    # cached: the tokens the slot's cache holds; pending: tokens the next turn opens with (the system prompt
    # of a new sequence, or the last emitted token of a turn that ended at its budget before the model ran it)
    slot, cached, pending, n_draw = llm.cache.acquire(), [], list(system), 0
    print("token ids per line; /clear starts over, /quit ends", file=sys.stderr)
    for line in sys.stdin:
        line = line.strip()
        if line == "/quit":
            break
        if line == "/clear":
            llm.cache.release(slot)
            slot, cached, pending = llm.cache.acquire(), [], list(system)
            continue
        turn = pending + parse_ids(line)
        if not turn:
            continue
        room = ctx - len(cached) - 1
        if room <= 0:
            print("context is full; /clear to start over", file=sys.stderr)
            continue
        turn = turn[:room]                                        # chat.c:289-294
        pending = []
        # the turn goes on in the held slot through the same loop as every other generation: prompt in
        # pieces of at most ubatch tokens, captured decode steps, stop tokens, budget, full context
        r = llm.generate([turn], params, max_new_tokens=args.tokens, ignore_eos=args.ignore_eos,
                         max_step_tokens=max(1, args.ubatch),
                         continuations=[tlc.Continuation(slot, cached, n_draw)],
                         on_token=lambda i, tok: print(tok, end=" ", flush=True))[0]
        print(flush=True)
        n_draw += len(r.tokens) + (1 if r.finish_reason == "stop" else 0)
        run = len(r.tokens) - r.uncached
        cached = cached + turn + r.tokens[:run]
        pending = r.tokens[run:]
    llm.cache.release(slot)
    return 0


if __name__ == "__main__":
    sys.exit(main())
