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
    from tinyllama_c_b200.engine import StepEntry
    from tinyllama_c_b200.sampling import Sampler
    ctx = args.ctx if args.ctx > 0 else 0
    llm = tlc.LLM(args.model, dtype=args.dtype, max_tokens=ctx or 4096, max_seqs=1)
    ctx = min(ctx or llm.max_context, llm.max_context)
    params = sampling_params(args)
    sampler = Sampler(params, llm.model.device)
    stop = set() if args.ignore_eos else set(llm.config.stop_token_ids)
    system = parse_ids(args.system) if args.system else []
    slot, history, n_draw = llm.cache.acquire(), [], 0
    pending = list(system)
    print("token ids per line; /clear starts over, /quit ends", file=sys.stderr)
    for line in sys.stdin:
        line = line.strip()
        if line == "/quit":
            break
        if line == "/clear":
            llm.cache.release(slot)
            slot, history, pending = llm.cache.acquire(), [], list(system)
            continue
        turn = pending + parse_ids(line)
        pending = []
        if not turn:
            continue
        room = ctx - len(history) - 1
        if room <= 0:
            print("context is full; /clear to start over", file=sys.stderr)
            continue
        turn = turn[:room]                                        # chat.c:289-294
        out = []
        for i in range(0, len(turn), max(1, args.ubatch)):        # prompt in pieces of at most ubatch tokens
            chunk = turn[i:i + max(1, args.ubatch)]
            last = i + len(chunk) >= len(turn)
            logits = llm.step([StepEntry(slot, chunk, [len(chunk) - 1] if last else [])])
        history += turn
        while len(out) < args.tokens and len(history) < ctx:
            tok = int(sampler.sample(logits, [history], [0], [n_draw]).cpu()[0])
            n_draw += 1
            if tok in stop:
                break
            out.append(tok)
            history.append(tok)
            print(tok, end=" ", flush=True)
            if len(history) >= ctx:
                break
            logits = llm.step([StepEntry(slot, [tok], [0])])
        print(flush=True)
    llm.cache.release(slot)
    return 0


if __name__ == "__main__":
    sys.exit(main())
