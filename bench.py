#!/usr/bin/env python3
"""Decode and prefill throughput of Falcon-H1 (1.5B layer sizes, random weights) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A step is one decode step of the whole batch (8 sequences by default, each continuing a
512-token prompt; the cache is sized for the 4096-token benchmark context).  The line
printed is one JSON object:
  value      decoded tokens per second, timed on the device (CUDA events around K replayed steps
             of the engine's captured decode step, sampling included)
  e2e        the same through the Python entry point LLM.generate(): host token ids in, host
             token ids out, every step copying its inputs from pinned memory and reading its
             result back
  prefill    one 2,048-token prompt: tokens per second, milliseconds, fraction of the bf16 peak
  roofline   bytes a decode step has to read (every weight once + the live cache) / its time,
             against the measured HBM bandwidth
  points     decode at batch 1, 16, 32 and 64, at batch 8 with 3,800-token prompts, and the workloads of the
             3B and 7B layer sizes (16 unequal prompts with 256 sampled tokens each; batch-64 decode from
             1,024-token prompts and one 8,192-token prompt)
The reference publishes no Falcon-H1 number (vs_baseline is null) and runs the model on the CPU only
(falcon_h1.c:78-83); --impl reference builds the unmodified reference and measures that CPU engine on the
same layer sizes at batch 1, the only batch it has (baseline/reference_arm.py).
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Falcon-H1-1.5B layer sizes (context 4096, tied embeddings, muP multipliers set)
CONFIG_1P5B = dict(
    architectures=["FalconH1ForCausalLM"], model_type="falcon_h1", vocab_size=65536, hidden_size=2048,
    num_hidden_layers=24, num_attention_heads=8, num_key_value_heads=2, head_dim=128, intermediate_size=4096,
    rope_theta=1e11, max_position_embeddings=4096, rms_norm_eps=1e-5, tie_word_embeddings=True,
    mamba_d_ssm=3072, mamba_n_heads=48, mamba_d_head=64, mamba_n_groups=1, mamba_d_state=256, mamba_d_conv=4,
    mamba_chunk_size=128, mamba_conv_bias=True, mamba_proj_bias=False, mamba_rms_norm=True,
    mamba_norm_before_gate=False, embedding_multiplier=5.66, lm_head_multiplier=0.039, key_multiplier=0.39,
    attention_in_multiplier=1.0, attention_out_multiplier=0.94, ssm_in_multiplier=1.25, ssm_out_multiplier=0.24,
    mlp_multipliers=[0.88, 0.3], ssm_multipliers=[0.35, 0.25, 0.7, 0.5, 0.35])
# the 3B and 7B layer sizes (their other options as above): --sizes 3B / 7B
CONFIG_3B = dict(CONFIG_1P5B, hidden_size=2560, num_hidden_layers=32, num_attention_heads=10, intermediate_size=8192,
                 mamba_d_ssm=4096, mamba_n_heads=32, mamba_d_head=128)
CONFIG_7B = dict(CONFIG_1P5B, hidden_size=3072, num_hidden_layers=44, num_attention_heads=12, intermediate_size=12288,
                 vocab_size=130048, max_position_embeddings=8192, tie_word_embeddings=False,
                 mamba_d_ssm=3072, mamba_n_heads=24, mamba_d_head=128)
CONFIGS = {"1.5B": CONFIG_1P5B, "3B": CONFIG_3B, "7B": CONFIG_7B}


def peaks():
    p = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            m = json.load(open(path))
            p = dict(hbm_gbs=float(m.get("hbm_gbs", p["hbm_gbs"])), bf16_tflops=float(m.get("bf16_tflops", p["bf16_tflops"])),
                     source="measured")
        except Exception:
            pass
    return p


def sizes(cfg):
    D, F, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    H, KV, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    Di, Hs, N, G, K = cfg["mamba_d_ssm"], cfg["mamba_n_heads"], cfg["mamba_d_state"], cfg["mamba_n_groups"], cfg["mamba_d_conv"]
    Cd = Di + 2 * G * N
    Pd = Di + Cd + Hs
    layer_w = D * (H * hd + 2 * KV * hd) + H * hd * D + D * Pd + Di * D + 2 * D * F + F * D
    return dict(D=D, F=F, V=V, L=L, H=H, KV=KV, hd=hd, Di=Di, Hs=Hs, N=N, G=G, K=K, Cd=Cd, Pd=Pd, layer_w=layer_w,
                P=Di // Hs)


def decode_bytes(cfg, batch, context):
    """Bytes one decode step has to read: every weight it uses once (bf16 matrices, head
    included), and the cache of the live sequences (bf16 keys and values up to `context`,
    the 32-bit conv window and SSM state)."""
    s = sizes(cfg)
    weights = (s["L"] * s["layer_w"] + s["V"] * s["D"]) * 2          # the head's matrix; a token's embedding row is 4 KB
    kv = 2 * s["L"] * s["KV"] * s["hd"] * 2 * context
    state = s["L"] * (s["Hs"] * s["P"] * s["N"] + (s["K"] - 1) * s["Cd"]) * 4
    return weights + batch * (kv + state)


def prefill_flops(cfg, T):
    s = sizes(cfg)
    gemm = 2 * T * s["L"] * s["layer_w"] + 2 * s["V"] * s["D"]          # head on one row
    attn = s["L"] * 2 * 2 * s["H"] * s["hd"] * T * (T + 1) / 2           # QK^T and PV, causal
    ssd = s["L"] * T * s["Hs"] * s["P"] * s["N"] * 6                       # state update + readout
    return gemm + attn + ssd


class Clocks:
    """Samples nvidia-smi while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.p = None
        return self

    def __exit__(self, *a):
        self.result = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
        if self.p is None:
            return
        time.sleep(0.15)
        self.p.terminate()
        out, _ = self.p.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6 or not f[0].isdigit():
                continue
            sm.append(int(f[0]))
            mx.append(int(f[1]))
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            sm.sort()
            self.result = dict(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), reasons=sorted(reasons))


def time_decode(llm, tlc, batch, prompt_len, steps, warmup, seed):
    """Device time of `steps` decode steps of `batch` sequences through the engine's own decode step
    (EngineBackend.decode_step: reserve, upload, replay of the captured step, read-back, commit)."""
    import torch
    from tinyllama_c_b200 import ops
    from tinyllama_c_b200.engine import EngineBackend, StepEntry
    g = torch.Generator().manual_seed(seed)
    V = llm.config.vocab_size
    slots = [llm.cache.acquire() for _ in range(batch)]
    prompts = torch.randint(0, V, (batch, prompt_len), generator=g).tolist()
    # prompts in groups that bound activation memory
    group = max(1, 8192 // prompt_len)
    for i in range(0, batch, group):
        llm.step([StepEntry(s, p, ()) for s, p in zip(slots[i:i + group], prompts[i:i + group])])
    backend = EngineBackend(llm.model, llm.cache, tlc.GREEDY, llm._graphs, True)
    toks = torch.randint(0, V, (batch,), generator=g).tolist()

    def one():
        nonlocal toks
        toks = backend.decode_step([(s, [t]) for s, t in zip(slots, toks)])

    for _ in range(max(3, warmup)):
        one()
    torch.cuda.synchronize()
    l0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with Clocks() as clk:
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = ops.launch_count() - l0
    ctx = prompt_len + max(3, warmup) + steps // 2
    for s in slots:
        llm.cache.release(s)
    ops.check_errors()
    return ms, launches, clk.result, ctx


def time_prefill(llm, T, seed, reps=3):
    import torch
    from tinyllama_c_b200 import ops
    from tinyllama_c_b200.engine import StepEntry
    g = torch.Generator().manual_seed(seed)
    best = None
    warm = 4                               # the first runs ramp the clocks and fill the tensor-map caches
    for r in range(reps + warm):
        toks = torch.randint(0, llm.config.vocab_size, (T,), generator=g).tolist()
        s = llm.cache.acquire()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        llm.step([StepEntry(s, toks, (T - 1,))])
        e1.record()
        torch.cuda.synchronize()
        llm.cache.release(s)
        if r >= warm:
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
    ops.check_errors()
    return best


def e2e_decode(llm, tlc, batch, prompt_len, steps, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, llm.config.vocab_size, (batch, prompt_len), generator=g).tolist()
    llm.generate(prompts, tlc.GREEDY, max_new_tokens=4, ignore_eos=True, max_batch=batch)      # warm-up, captures the graph
    llm.generate(prompts, tlc.GREEDY, max_new_tokens=steps + 1, ignore_eos=True, max_batch=batch)
    st = llm.last_stats
    return st["decode_tokens"] / st["decode_s"], st["h2d_bytes"] // max(1, st["decode_steps"]), \
        st["d2h_bytes"] // max(1, st["decode_steps"])


def time_generate(llm, tlc, n_prompts, lo, hi, new_tokens, temperature, seed):
    """Unequal prompts (lengths uniform in [lo, hi]) generated together through LLM.generate() with temperature
    sampling, every sequence to new_tokens: host token ids in and out, the second of two runs timed."""
    import torch
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (n_prompts,), generator=g).tolist()
    prompts = [torch.randint(0, llm.config.vocab_size, (n,), generator=g).tolist() for n in lens]
    sampling = tlc.SamplingParams(temperature=temperature, seed=seed)
    out = {}
    for run in range(2):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        llm.generate(prompts, sampling, max_new_tokens=new_tokens, ignore_eos=True, max_batch=n_prompts)
        torch.cuda.synchronize()
        out = dict(llm.last_stats, wall_s=time.perf_counter() - t0)
    return {"prompts": n_prompts, "prompt_tokens": sum(lens), "new_tokens": n_prompts * new_tokens,
            "temperature": temperature, "wall_s": round(out["wall_s"], 4),
            "prefill_tok_s": round(out["prefill_tokens"] / out["prefill_s"], 1),
            "decode_tok_s": round(out["decode_tokens"] / out["decode_s"], 1),
            "tok_s": round(n_prompts * new_tokens / out["wall_s"], 1)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (both numbers are reported)")
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--sizes", default="1.5B", choices=sorted(CONFIGS), help="layer sizes of this Falcon-H1 model")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--generate", type=int, default=0, metavar="N",
                    help="also generate 256 tokens for N prompts of 64..2048 tokens at temperature 0.7")
    ap.add_argument("--prefill-only", action="store_true", help="time the prompt of --prefill-tokens tokens only "
                    "(--steps repetitions when fewer than 8): what a profiler capture of the prompt kernels runs")
    ap.add_argument("--no-big", dest="big", action="store_false", help="skip the 3B and 7B workloads among the points")
    ap.add_argument("--no-pairs", action="store_true", help="run the linear layers on single blocks (128 x 256 tiles) instead "
                    "of pairs of blocks on 256 x 256 tiles: the comparison behind profiles/linear_tcgen05_prefill_2048.md")
    ap.add_argument("--ref-budget", type=float, default=600.0, help="seconds the reference arm may take (it runs fewer "
                    "layers, and says so, where all of them would take longer)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU library")
        return 2

    import torch
    import tinyllama_c_b200 as tlc
    if args.no_pairs:
        from tinyllama_c_b200 import ops
        ops.linear_pair_override(1)
    full_layers = CONFIGS[args.sizes]["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    cfg = dict(CONFIGS[args.sizes], num_hidden_layers=args.layers)
    s = sizes(cfg)
    pk = peaks()
    ctx_len = cfg["max_position_embeddings"]
    model = tlc.random_model(cfg, seed=0, dtype="bfloat16")
    # room for 64 sequences of prompt + decoded tokens, for the long prompt and for the unequal batch
    per_seq = -(-(args.prompt_len + 2 * args.steps + 80) // 64) * 64
    room = max(64 * 1024, max(64, args.batch) * per_seq, args.prefill_tokens + 64, args.generate * (2048 + 256 + 64),
               8 * 3968)
    llm = tlc.LLM(model, max_tokens=room, max_seqs=max(64, args.batch, args.generate))

    if args.prefill_only:
        T = args.prefill_tokens
        pms = time_prefill(llm, T, seed=3, reps=args.steps if args.steps < 8 else 3)
        print(json.dumps({"prefill": {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
                                      "frac": round(prefill_flops(cfg, T) / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
                          "layers": args.layers}))
        return 0

    ms, launches, clocks, ctx = time_decode(llm, tlc, args.batch, args.prompt_len, args.steps, args.warmup, seed=1)
    value = args.batch * 1000.0 / ms
    nbytes = decode_bytes(cfg, args.batch, ctx)
    achieved = nbytes / (ms * 1e-3) / 1e9
    e2e_v, h2d, d2h = e2e_decode(llm, tlc, args.batch, args.prompt_len, args.steps, seed=2)
    rec = {
        "metric": f"decode tok/s at batch {args.batch} (Falcon-H1-{args.sizes} sizes, {args.prompt_len}-token prompts, "
                  f"context {ctx_len})",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "config": {"model": f"Falcon-H1-{args.sizes} sizes", "global_batch": args.batch, "seq_len": ctx_len,
                   "prompt_len": args.prompt_len, "parallelism": "single GPU", "layers": args.layers,
                   "layers_full": full_layers, "hidden": cfg["hidden_size"],
                   "heads": f"{s['H']}q/{s['KV']}kv x{s['hd']}",
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "mamba": f"{s['Hs']} heads x{s['P']}, state {s['N']}, groups {s['G']}, conv {s['K']}",
                   "tied": cfg["tie_word_embeddings"],
                   "l2": f"inputs larger than L2 ({decode_bytes(cfg, 0, 0) / 1e9:.1f} GB of weights per step)"},
        "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": round(e2e_v, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"]},
    }
    if not args.no_points:
        T = args.prefill_tokens
        pms = time_prefill(llm, T, seed=3)
        fl = prefill_flops(cfg, T)
        rec["prefill"] = {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
                          "frac": round(fl / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        pts = {}
        for b in (1, 16, 32, 64):
            m, _, _, c = time_decode(llm, tlc, b, args.prompt_len, max(16, args.steps // 2), 3, seed=4 + b)
            pts[f"decode_b{b}"] = round(b * 1000.0 / m, 1)
            pts[f"decode_b{b}_hbm_frac"] = round(decode_bytes(cfg, b, c) / (m * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        m, _, _, c = time_decode(llm, tlc, 8, 3800, max(16, args.steps // 2), 3, seed=31)
        pts["decode_b8_ctx3800"] = round(8 * 1000.0 / m, 1)
        pts["decode_b8_ctx3800_hbm_frac"] = round(decode_bytes(cfg, 8, c) / (m * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        rec["points"] = pts
    if args.generate:
        rec["generate"] = time_generate(llm, tlc, args.generate, 64, 2048, 256, 0.7, seed=9)
    if args.big and not args.no_points and args.sizes == "1.5B":
        del llm, model
        torch.cuda.empty_cache()
        rec["points"].update(big_workloads(tlc, pk))
    print(json.dumps(rec))
    return 0


def big_workloads(tlc, pk):
    """The workloads of the 3B and 7B layer sizes: 16 unequal prompts of 64..2,048 tokens with 256 tokens sampled
    for each at temperature 0.7 (3B); decode at batch 64 from 1,024-token prompts and one 8,192-token prompt (7B)."""
    import torch
    out = {}
    cfg = CONFIGS["3B"]
    llm = tlc.LLM(tlc.random_model(cfg, seed=0, dtype="bfloat16"), max_tokens=16 * (2048 + 256 + 64), max_seqs=16)
    g = time_generate(llm, tlc, 16, 64, 2048, 256, 0.7, seed=9)
    out["3b_generate_16_tok_s"] = g["tok_s"]
    out["3b_generate_16_wall_s"] = g["wall_s"]
    m, _, _, c = time_decode(llm, tlc, 16, 512, 16, 3, seed=41)
    out["3b_decode_b16"] = round(16 * 1000.0 / m, 1)
    out["3b_decode_b16_hbm_frac"] = round(decode_bytes(cfg, 16, c) / (m * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    del llm
    torch.cuda.empty_cache()
    cfg = CONFIGS["7B"]
    llm = tlc.LLM(tlc.random_model(cfg, seed=0, dtype="bfloat16"), max_tokens=64 * 1152, max_seqs=64)
    m, _, _, c = time_decode(llm, tlc, 64, 1024, 16, 3, seed=42)
    out["7b_decode_b64"] = round(64 * 1000.0 / m, 1)
    out["7b_decode_b64_hbm_frac"] = round(decode_bytes(cfg, 64, c) / (m * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    pms = time_prefill(llm, 8192, seed=43, reps=2)
    out["7b_prefill_8192_tok_s"] = round(8192 * 1000.0 / pms, 1)
    out["7b_prefill_8192_bf16_frac"] = round(prefill_flops(cfg, 8192) / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
    del llm
    torch.cuda.empty_cache()
    return out


def reference_arm(args) -> int:
    """The unmodified reference (its CPU engine, the only path it has for Falcon-H1) on the same layer sizes:
    decode at batch 1 after a prompt of --prompt-len tokens, and one prompt of --prefill-tokens tokens."""
    try:
        from baseline import reference_arm as ra
        cfg = dict(CONFIGS[args.sizes])
        steps, warmup = max(1, min(args.steps, 32)), max(3, min(args.warmup, 4))
        r = ra.measure(cfg, steps, warmup, args.prompt_len, args.prefill_tokens, budget_s=args.ref_budget,
                       layers=args.layers)
    except Exception as e:                                  # noqa: BLE001 -- any failure is reported, never raised
        msg = " ".join(str(e).split())[:300]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference's CPU engine could not be built or run: {msg}"}))
        return 0
    s = sizes(cfg)
    tok_s = r["steps"] / r["decode_s"]
    rec = {
        "impl": "reference",
        "metric": f"decode tok/s at batch 1 (CodeClaper/tinyllama.c's CPU engine, {r['threads']} threads; Falcon-H1-"
                  f"{args.sizes} sizes, {args.prompt_len}-token prompt, context {cfg['max_position_embeddings']})",
        "value": round(tok_s, 3), "unit": "tok/s", "n_gpus": 0, "steps": r["steps"], "warmup": warmup,
        "ms_per_step": round(1000.0 * r["decode_s"] / r["steps"], 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 weights, fp32 arithmetic (the reference's CPU path)",
        "data": "synthetic (random weights in a GGUF file, pseudo-random token ids)",
        "config": {"model": f"Falcon-H1-{args.sizes} sizes", "global_batch": 1, "seq_len": cfg["max_position_embeddings"],
                   "prompt_len": args.prompt_len, "parallelism": f"CPU, {r['threads']} threads", "layers": r["layers"],
                   "layers_full": r["layers_full"], "hidden": cfg["hidden_size"], "heads": f"{s['H']}q/{s['KV']}kv x{s['hd']}",
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "mamba": f"{s['Hs']} heads x{s['P']}, state {s['N']}, groups {s['G']}, conv {s['K']}",
                   "tied": cfg["tie_word_embeddings"], "gguf_gb": round(r["gguf_bytes"] / 1e9, 2)},
        "e2e": {"value": round(tok_s, 3), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "host token ids in and out is the reference's only interface; no device is involved"},
        "gpu_launches": 0,
    }
    if r["prefill_s"] > 0:
        rec["prefill"] = {"value": round(args.prefill_tokens / r["prefill_s"], 1), "tokens": args.prefill_tokens,
                          "ms": round(1000.0 * r["prefill_s"], 1)}
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
