"""probe: small workloads for a profiler, and kernel timings.

The reference times one kernel with CUDA events in gpu_bench_matvec (gpu.cu:2092-2130) and
accumulates wall time per op class around its graph walk (graph.c:1288-1301).  This program
plays both roles for this library:

    bin/probe decode  --batch 8 --layers 2 --prompt 512     three eager one-token steps (for ncu)
    bin/probe prefill --layers 2 --prompt 2048              one prompt, twice (for ncu)
    bin/probe prefill --batch 16 --unequal --prompt 2048    16 prompts of 64..2048 tokens together, twice
    bin/probe linear  --rows 2048 --n 6704 --k 2048 [--accumulate] [--swiglu] [--bf16-out] [--tile 64|128|256] [--split n]
    bin/probe kernels --batch 8                             every decode-step kernel, warm, in a CUDA graph

Models are random, with the layer sizes of bench.py (--sizes 1.5B, 3B or 7B) and --layers layers.
"""
from __future__ import annotations

import argparse
import os
import sys


def _model(layers: int, sizes: str = "1.5B", room: int = 64 * 1024):
    import tinyllama_c_b200 as tlc
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
    import bench
    cfg = dict(bench.CONFIGS[sizes], num_hidden_layers=layers)
    return tlc.LLM(tlc.random_model(cfg, seed=0), max_tokens=max(room, 64 * 1024), max_seqs=64), cfg


def run_steps(args) -> None:
    import torch
    from tinyllama_c_b200.engine import StepEntry
    B = args.batch if args.what == "decode" or args.unequal else 1
    llm, cfg = _model(args.layers, args.sizes, B * (args.prompt + 128))
    g = torch.Generator().manual_seed(0)
    slots = [llm.cache.acquire() for _ in range(B)]
    prompts = torch.randint(0, cfg["vocab_size"], (B, args.prompt), generator=g).tolist()
    if args.what == "decode":
        for i in range(0, B, 8):
            llm.step([StepEntry(s, p, ()) for s, p in zip(slots[i:i + 8], prompts[i:i + 8])])
        torch.cuda.synchronize()
        for _ in range(3):
            llm.step([StepEntry(s, [5], (0,)) for s in slots])
    elif args.unequal:
        # prompts of 64..--prompt tokens together, in steps of at most 8192 tokens as generation runs them
        from tinyllama_c_b200.engine.generate import EngineBackend
        import tinyllama_c_b200 as tlc
        lens = torch.randint(64, args.prompt + 1, (B,), generator=g).tolist()
        backend = EngineBackend(llm.model, llm.cache, tlc.GREEDY)
        for it in range(2):
            if it:
                for s in slots:
                    llm.cache.release(s)
                slots = [llm.cache.acquire() for _ in range(B)]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            backend.step_and_sample([(s, p[:n]) for s, p, n in zip(slots, prompts, lens)], [[]] * B, list(range(B)), [0] * B)
            e1.record()
            torch.cuda.synchronize()
            print(f"{sum(lens)} tokens of {B} prompts: {e0.elapsed_time(e1):.2f} ms", flush=True)
    else:
        for it in range(2):
            s = slots[0] if it == 0 else llm.cache.acquire()
            llm.step([StepEntry(s, prompts[0], (args.prompt - 1,))])
    torch.cuda.synchronize()
    print("ok")


def timeit(name, fn, nbytes=None, flops=None, reps=50):
    """Mean time of `reps` back-to-back launches replayed from a CUDA graph."""
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(reps):
                fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph.replay()
    torch.cuda.synchronize()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000 / reps
    extra = f"  {nbytes / us / 1e3:8.1f} GB/s" if nbytes else ""
    extra += f"  {flops / us / 1e6:8.1f} TFLOP/s" if flops else ""
    print(f"{name:36s} {us:9.2f} us{extra}", flush=True)


def run_linear(args) -> None:
    import torch
    from tinyllama_c_b200 import ops
    lib = ops.library()
    lib.tlc_linear_tile_override(args.tile)
    lib.tlc_linear_split_override(args.split)
    M, N, K = args.rows, args.n, args.k
    a = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * K ** -0.5).bfloat16()      # outputs of order one, as in a model
    if args.swiglu:
        act = torch.zeros(M, N // 2, dtype=torch.bfloat16, device="cuda")
        timeit(f"linear+swiglu {M}x{N}x{K} tile={args.tile or 'auto'}", lambda: ops.linear_swiglu(a, w, act, None, None),
               flops=2.0 * M * N * K, reps=20)
        ops.check_errors()
        return
    out = torch.zeros(M, N, dtype=torch.bfloat16 if args.bf16_out else torch.float32, device="cuda")
    # few rows: the time is that of streaming the weights, so rotate over copies that together exceed the L2
    ncopy = max(1, int(400e6 // (N * K * 2)) + 1) if M <= 128 else 1
    ws = [w] + [w.clone() for _ in range(ncopy - 1)]
    st = {"i": 0}

    def fn():
        ops.linear(a, ws[st["i"] % ncopy], out, None, None, args.accumulate)
        st["i"] += 1
    timeit(f"linear {M}x{N}x{K} tile={args.tile or 'auto'}", fn, nbytes=N * K * 2 if ncopy > 1 else None,
           flops=2.0 * M * N * K, reps=max(20, ncopy * 2))
    ops.check_errors()


def run_kernels(args) -> None:
    import torch
    from tinyllama_c_b200 import ops
    ops.library()
    dev, bf, f32 = "cuda", torch.bfloat16, torch.float32
    B, CTX = args.batch, args.prompt
    D, F, V, H, KV, hd = 2048, 4096, 65536, 8, 2, 128
    Di, Hs, P, N, G, K = 3072, 48, 64, 256, 1, 4
    Cd = Di + 2 * G * N
    Pd = Di + Cd + Hs
    x32 = torch.randn(B, D, device=dev)
    w = torch.ones(D, device=dev)
    xn = torch.empty(B, D, dtype=bf, device=dev)
    timeit("rmsnorm", lambda: ops.rmsnorm(x32, w, 1e-5, xn))

    def lin(name, Nn, Kk, accumulate):
        # rotate over copies of the weights that together exceed L2, so that every call streams from HBM
        ncopy = max(2, int(400e6 // (Nn * Kk * 2)) + 1)
        Ws = [torch.randn(Nn, Kk, device=dev).to(bf) for _ in range(ncopy)]
        a = torch.randn(B, Kk, device=dev).to(bf)
        out = torch.zeros(B, Nn, dtype=f32, device=dev)
        st = {"i": 0}

        def fn():
            ops.linear(a, Ws[st["i"] % ncopy], out, None, None, accumulate)
            st["i"] += 1
        timeit(name, fn, Nn * Kk * 2, reps=ncopy * 3)
    lin("linear qkv 1536x2048", 1536, 2048, False)
    lin("linear in_proj 6704x2048", Pd, 2048, False)
    lin("linear o 2048x1024 (+=)", 2048, 1024, True)
    lin("linear out 2048x3072 (+=)", 2048, 3072, True)
    lin("linear gate_up 8192x2048", 8192, 2048, False)
    lin("linear down 2048x4096 (+=)", 2048, 4096, True)
    lin("linear head 65536x2048", 65536, 2048, False)
    n_pages = B * ((CTX + 64) // 64 + 1)
    kp = torch.randn(n_pages, KV, 64, hd, device=dev).to(bf)
    vp = torch.randn_like(kp)
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).reshape(B, -1).contiguous()
    pos = torch.full((B,), CTX, dtype=torch.int32, device=dev)
    rs = torch.arange(B, dtype=torch.int32, device=dev)
    slots = rs.clone()
    q = torch.randn(B, H * hd, device=dev).to(bf)
    o = torch.empty_like(q)
    timeit(f"attention, one token, context {CTX}",
           lambda: ops.attention(q, kp, vp, table, pos, rs, slots, o, H, KV, hd, 0.088, 0, 2 * CTX),
           B * KV * CTX * hd * 2 * 2)
    qkv = torch.randn(B, (H + 2 * KV) * hd, device=dev)
    inv = torch.rand(hd // 2, device=dev)
    timeit("rope_kv_store", lambda: ops.rope_kv_store(qkv, 0, H * hd, (H + KV) * hd, q, kp, vp, inv, pos, rs, slots, table,
                                                      H, KV, hd, True))
    proj = torch.randn(B, Pd, device=dev)
    cw, cb = torch.randn(Cd, K, device=dev), torch.randn(Cd, device=dev)
    dtb, A = torch.randn(Hs, device=dev), -torch.rand(Hs, device=dev)
    cstate = torch.zeros(B, K - 1, Cd, device=dev)
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
    xbc, dt, dA = torch.empty(B, Cd, device=dev), torch.empty(B, Hs, device=dev), torch.empty(B, Hs, device=dev)
    timeit("mamba_conv, one token", lambda: ops.mamba_conv(proj, Di, Di + Cd, cw, cb, dtb, A, cstate, cu, rs, slots, pos,
                                                           xbc, dt, dA, True))
    state = torch.zeros(B, Hs, P, N, device=dev)
    y = torch.empty(B, Di, device=dev)
    Dk = torch.ones(Hs, device=dev)
    timeit("ssm_scan, one token", lambda: ops.ssm_scan(xbc, dt, dA, Dk, state, cu, slots, pos, y, Hs, P, N, G),
           B * Hs * P * N * 4 * 2)
    gated = torch.empty(B, Di, dtype=bf, device=dev)
    nw = torch.ones(Di, device=dev)
    timeit("gated_rmsnorm", lambda: ops.gated_rmsnorm(y, proj[:, :Di], nw, 1e-5, G, False, gated))
    gu = torch.randn(B, 2 * F, device=dev)
    act = torch.empty(B, F, dtype=bf, device=dev)
    timeit("swiglu", lambda: ops.swiglu(gu, act))
    lg = torch.randn(B, V, device=dev)
    tok = torch.empty(B, dtype=torch.int32, device=dev)
    timeit("argmax", lambda: ops.argmax(lg, tok))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="probe", description=__doc__.split("\n\n")[0])
    ap.add_argument("what", choices=["decode", "prefill", "linear", "kernels"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--sizes", default="1.5B", choices=["1.5B", "3B", "7B"], help="decode, prefill: layer sizes of the model")
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--n", type=int, default=6704)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--accumulate", action="store_true")
    ap.add_argument("--unequal", action="store_true", help="prefill: --batch prompts of 64..--prompt tokens in one batch")
    ap.add_argument("--tile", type=int, default=0, choices=[0, 64, 128, 256])
    ap.add_argument("--split", type=int, default=0, help="linear: blocks that share a tile's K-steps (0: chosen, 1: none)")
    ap.add_argument("--swiglu", action="store_true", help="linear: gate|up rows interleaved by 8, SwiGLU in the epilogue")
    ap.add_argument("--bf16-out", action="store_true", help="linear: bfloat16 output instead of float32")
    args = ap.parse_args(argv)
    if args.what in ("decode", "prefill"):
        run_steps(args)
    elif args.what == "linear":
        run_linear(args)
    else:
        run_kernels(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
