"""bench: run one prompt, generate, report prefill and decode speed (bench.c:139-322).

    bin/bench -m DIR -i "5 17 3 200" [-n 128] [-t 0.8 -tk 40 -tp 0.9 -P 0.05] [-r 1] [-o FILE]

The prompt is a list of token ids (the reference takes text and tokenises it, bench.c:171).
Like the reference it times the prompt pass and the token loop separately and repeats the
whole run -r times, resetting the sequence in between (bench.c:196-250).
"""
from __future__ import annotations

import argparse
import sys
import time

from .options import add_common, parse_ids, sampling_params


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="bench", description=__doc__.split("\n\n")[0])
    add_common(ap, default_tokens=128)
    ap.add_argument("-i", "--input", required=True, help="prompt as token ids separated by spaces")
    ap.add_argument("-o", "--output", default=None, help="save the generated token ids to this file")
    ap.add_argument("-r", "--repeat", type=int, default=1)
    ap.add_argument("-b", "--batch", type=int, default=1, help="copies of the prompt generated together")
    args = ap.parse_args(argv)
    import tinyllama_c_b200 as tlc
    prompt = parse_ids(args.input)
    if not prompt:
        raise SystemExit("Input is required (-i / --input)")
    n_tokens = max(1, args.tokens)
    ctx = args.ctx if args.ctx > 0 else None
    need = (len(prompt) + n_tokens + 63) // 64 * 64 * max(1, args.batch)
    llm = tlc.LLM(args.model, dtype=args.dtype, max_tokens=max(need, 64), max_seqs=max(1, args.batch))
    if ctx:
        llm.max_context = min(llm.max_context, ctx)
    params = sampling_params(args)
    result = None
    for r in range(max(1, args.repeat)):
        t0 = time.perf_counter()
        result = llm.generate([prompt] * max(1, args.batch), params, max_new_tokens=n_tokens,
                              ignore_eos=args.ignore_eos, max_batch=max(1, args.batch), max_step_tokens=max(1, args.ubatch))
        wall = time.perf_counter() - t0
        st = llm.last_stats
        pre = st["prefill_tokens"] / st["prefill_s"] if st["prefill_s"] > 0 else float("nan")
        dec = st["decode_tokens"] / st["decode_s"] if st["decode_s"] > 0 else float("nan")
        print(f"run {r + 1}: prompt {len(prompt)} tokens x {max(1, args.batch)}, generated "
              f"{sum(len(x.tokens) for x in result)} tokens in {wall:.3f} s | prefill {pre:.1f} tok/s | "
              f"decode {dec:.1f} tok/s | finish: {result[0].finish_reason}")
    print(" ".join(str(t) for t in result[0].tokens))
    if args.output:
        with open(args.output, "w") as f:
            f.write(" ".join(str(t) for t in result[0].tokens) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
