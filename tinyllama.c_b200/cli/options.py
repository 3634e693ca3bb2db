"""Command-line options in the manner of CodeClaper/tinyllama.c's bench and chat programs.

Names, meanings and defaults follow bench.c:64-127 and chat.c:88-153 where the reference has
the option.  Options that do not apply to a single-GPU library for token ids are accepted
and ignored (-T/--threads, -ngl/--n-gpu-layers) so that command lines carry over; there is
no tokenizer here, so -i/--input and the chat loop take token ids separated by spaces.
"""
from __future__ import annotations

import argparse

from ..sampling.params import SamplingParams


def add_common(ap: argparse.ArgumentParser, default_tokens: int) -> None:
    ap.add_argument("-m", "--model", required=True, help="model folder (config.json + model.safetensors)")
    ap.add_argument("-c", "--ctx", type=int, default=0, help="context size (default: the model's max_position_embeddings)")
    ap.add_argument("-ub", "--ubatch", type=int, default=512, help="max tokens per forward pass of a prompt")
    ap.add_argument("-n", "--tokens", type=int, default=default_tokens, help="tokens to generate")
    ap.add_argument("-T", "--threads", type=int, default=-1, help="ignored (CPU threads of the reference)")
    ap.add_argument("-ngl", "--n-gpu-layers", type=int, default=-1, help="ignored (the whole model runs on the GPU)")
    ap.add_argument("-t", "--temp", type=float, default=0.8, help="temperature (0 = greedy)")
    ap.add_argument("-tp", "--topp", type=float, default=0.9)
    ap.add_argument("-tk", "--topk", type=int, default=40)
    ap.add_argument("-P", "--minp", type=float, default=0.05)
    ap.add_argument("-rp", "--repeat-penalty", type=float, default=1.1)
    ap.add_argument("-rl", "--repeat-last-n", type=int, default=64)
    ap.add_argument("-fp", "--frequency-penalty", type=float, default=0.0)
    ap.add_argument("-pp", "--presence-penalty", type=float, default=0.0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--seed", type=int, default=0, help="seed of the sampler's draws")
    ap.add_argument("--ignore-eos", action="store_true", help="do not stop at the stop tokens")


def sampling_params(args) -> SamplingParams:
    return SamplingParams(temperature=args.temp, top_k=args.topk, top_p=args.topp, min_p=args.minp,
                          repeat_penalty=args.repeat_penalty, repeat_last_n=args.repeat_last_n,
                          frequency_penalty=args.frequency_penalty, presence_penalty=args.presence_penalty,
                          seed=args.seed)


def parse_ids(text: str):
    try:
        return [int(x) for x in text.replace(",", " ").split()]
    except ValueError as e:
        raise SystemExit(f"token ids must be integers separated by spaces: {e}")
