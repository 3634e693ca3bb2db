"""The reference arm of bench.py: CodeClaper/tinyllama.c itself, unmodified, on the benchmark's workload.

tinyllama.c is a C program without a Python package (`pip install` of it fails: neither setup.py nor
pyproject.toml), and its engine forces Falcon-H1 onto the CPU (src/model/falcon_h1.c:78-83: the Mamba2
ops have no CUDA twin).  Its stock Falcon-H1 path is therefore its CPU engine, and that is what runs
here:

  * `prepare()` copies the reference's `src/` tree, untouched, to baseline/_ref/src (git-ignored; it
    travels to the GPU box with the repository snapshot);
  * `build()` compiles those sources with the reference's own flags (src/Makefile:4: -O3 -march=native
    -ffast-math -pthread, -msse4.1 on x86) on the machine that runs the benchmark, together with a
    small driver that calls the reference's public API -- engine_open, session_create, graph_prepare,
    graph_execute, sample_token (core.h:28-35, graph.h:89-109, sampler.h:6) -- in the order of its own
    bench program (bench.c:196-250: reset, prompt pass timed, then single tokens timed);
  * `write_gguf()` writes a synthetic Falcon-H1 model in the only format the reference reads (GGUF v3,
    core.c:1349-1395) with bfloat16 matrices at the benchmark's layer sizes and random values.

Nothing of this repository's engine, kernels or models is on that path.  The reference serves one
sequence per session (def.h:533-542), so its figure is decode at batch 1; it is a CPU number.
"""
from __future__ import annotations

import json
import os
import shutil
import struct
import subprocess
import sys
import tempfile
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
SOURCES = ["core", "quants", "mm", "slog", "utils", "graph", "tokenizer", "sampler", "pthreads", "kvcache", "rax",
           "asctx", "tool", "model/llama", "model/qwen25", "model/qwen35", "model/deepseek", "model/falcon",
           "model/falcon_h1", "model/gemma3", "backend/cpu/cpu", "backend/cpu/cpu_op"]

DRIVER = r"""
/* Drives the reference through its public API in the order of its bench program (bench.c:196-250). */
#include <stdio.h>
#include <stdlib.h>
#include <time.h>
#include "core.h"
#include "graph.h"
#include "sampler.h"
static double now(void) { struct timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return t.tv_sec + 1e-9 * t.tv_nsec; }
int main(int argc, char **argv) {
    /* argv: model.gguf ctx nthreads prompt_len prefill_len warmup steps */
    if (argc < 8) return 2;
    u32 ctx = (u32)atoi(argv[2]); int nthreads = atoi(argv[3]);
    u32 prompt_len = (u32)atoi(argv[4]), prefill_len = (u32)atoi(argv[5]);
    int warmup = atoi(argv[6]), steps = atoi(argv[7]);
    EngineOptons eo = { .model_path = argv[1], .inspect = false };
    Engine *en = engine_open(&eo);
    if (!en) return 3;
    Session *s = session_create(en, ctx, DEFAULT_N_UBATCH, nthreads, 0, 1);
    if (!s) return 4;
    s->sample.temperature = 0.0f;                       /* greedy */
    u32 nv = s->cfg.n_vocab;
    u32 n_max = prefill_len > prompt_len ? prefill_len : prompt_len;
    u32 *ids = malloc(sizeof(u32) * (n_max + 1));
    unsigned long long x = 88172645463325252ULL;
    for (u32 i = 0; i < n_max; i++) { x ^= x << 13; x ^= x >> 7; x ^= x << 17; ids[i] = (u32)(x % nv); }
    if (!graph_prepare(s)) fprintf(stderr, "graph warm-up failed; timings include set-up\n");
    /* prompt pass */
    double prefill_s = -1.0;
    if (prefill_len > 0) {
        s->ops.reset(s);
        double t0 = now();
        if (!graph_execute(s, ids, prefill_len, s->logits)) return 5;
        prefill_s = now() - t0;
    }
    /* single tokens after a prompt */
    s->ops.reset(s);
    if (!graph_execute(s, ids, prompt_len, s->logits)) return 6;
    u32 tok = sample_token(s->logits, nv, &s->sample, s->tokens, s->n_tokens);
    for (int i = 0; i < warmup; i++) {
        if (!graph_execute(s, &tok, 1, s->logits)) return 7;
        tok = sample_token(s->logits, nv, &s->sample, s->tokens, s->n_tokens);
    }
    double t0 = now();
    for (int i = 0; i < steps; i++) {
        if (!graph_execute(s, &tok, 1, s->logits)) return 8;
        tok = sample_token(s->logits, nv, &s->sample, s->tokens, s->n_tokens);
    }
    double decode_s = now() - t0;
    printf("RESULT {\"prefill_s\": %.6f, \"decode_s\": %.6f, \"steps\": %d, \"last_token\": %u}\n", prefill_s, decode_s,
           steps, tok);
    return 0;
}
"""


def prepare(reference_root: str = "/root/reference") -> str:
    """Copies the reference's src/ tree, unmodified, to baseline/_ref/src (once)."""
    dst = os.path.join(REF_DIR, "src")
    if not os.path.isfile(os.path.join(dst, "core.c")):
        src = os.path.join(reference_root, "src")
        if not os.path.isfile(os.path.join(src, "core.c")):
            raise RuntimeError(f"the reference's sources are neither in {dst} nor in {src}")
        os.makedirs(REF_DIR, exist_ok=True)
        shutil.copytree(src, dst)
    return dst


def build(work: str) -> str:
    """Compiles the reference's CPU engine and the driver on this machine; returns the executable."""
    src = prepare()
    flags = ["-O3", "-march=native", "-ffast-math", "-pthread"]           # src/Makefile:4 (LTO left out: same code, faster build)
    if os.uname().machine in ("x86_64", "i386", "i686"):
        flags.append("-msse4.1")                                          # src/Makefile:16-18
    objs = []
    procs = []
    for s in SOURCES:
        o = os.path.join(work, s.replace("/", "_") + ".o")
        procs.append((s, subprocess.Popen(["gcc", *flags, "-I", src, "-c", os.path.join(src, s + ".c"), "-o", o],
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(o)
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"gcc failed on the reference's {s}.c:\n{out[-2000:]}")
    drv = os.path.join(work, "driver.c")
    with open(drv, "w") as f:
        f.write(DRIVER)
    exe = os.path.join(work, "ref_bench")
    p = subprocess.run(["gcc", *flags, "-I", src, drv, *objs, "-lm", "-o", exe], capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"gcc failed on the driver:\n{p.stdout[-1000:]}\n{p.stderr[-2000:]}")
    return exe


# ---- a synthetic Falcon-H1 GGUF (v3) with bfloat16 matrices -------------------------------------------
def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def _bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def tensor_table(cfg: dict):
    """(GGUF name, shape, kind) of every tensor the reference binds for Falcon-H1 (core.c:1092-1113);
    kind: matrix (bfloat16, N(0, 0.02)) | ones | a | d | dt | conv."""
    D, F, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    H, KV, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    Di, Hs, N, G, K = (cfg["mamba_d_ssm"], cfg["mamba_n_heads"], cfg["mamba_d_state"], cfg["mamba_n_groups"],
                       cfg["mamba_d_conv"])
    Cd = Di + 2 * G * N
    t = [("token_embd.weight", (V, D), "matrix"), ("output_norm.weight", (D,), "ones")]
    if not cfg.get("tie_word_embeddings", False):
        t.append(("output.weight", (V, D), "matrix"))
    for l in range(L):
        b = f"blk.{l}."
        t += [(b + "attn_norm.weight", (D,), "ones"), (b + "ffn_norm.weight", (D,), "ones"),
              (b + "attn_q.weight", (H * hd, D), "matrix"), (b + "attn_k.weight", (KV * hd, D), "matrix"),
              (b + "attn_v.weight", (KV * hd, D), "matrix"), (b + "attn_output.weight", (D, H * hd), "matrix"),
              (b + "ssm_in.weight", (Di + Cd + Hs, D), "matrix"), (b + "ssm_conv1d.weight", (Cd, K), "conv"),
              (b + "ssm_conv1d.bias", (Cd,), "conv"), (b + "ssm_a", (Hs,), "a"), (b + "ssm_d", (Hs,), "d"),
              (b + "ssm_dt.bias", (Hs,), "dt"), (b + "ssm_norm.weight", (Di,), "ones"),
              (b + "ssm_out.weight", (D, Di), "matrix"), (b + "ffn_gate.weight", (F, D), "matrix"),
              (b + "ffn_up.weight", (F, D), "matrix"), (b + "ffn_down.weight", (D, F), "matrix")]
    return t


def write_gguf(path: str, cfg: dict, seed: int = 0) -> int:
    """Writes the model; returns the file's size in bytes.  Tensors are drawn and written one at a time."""
    a = "falcon-h1"
    kv = []
    kv_u32 = lambda k, v: kv.append(_s(k.encode()) + struct.pack("<II", 4, int(v)))
    kv_f32 = lambda k, v: kv.append(_s(k.encode()) + struct.pack("<If", 6, float(v)))
    kv_str = lambda k, v: kv.append(_s(k.encode()) + struct.pack("<I", 8) + _s(v.encode()))
    kv_strs = lambda k, vs: kv.append(_s(k.encode()) + struct.pack("<IIQ", 9, 8, len(vs)) + b"".join(_s(v.encode()) for v in vs))
    kv_str("general.architecture", a)
    kv_str("tokenizer.ggml.model", "gpt2")
    kv_strs("tokenizer.ggml.tokens", [f"t{i}" for i in range(cfg["vocab_size"])])
    kv_strs("tokenizer.ggml.merges", [])
    kv_u32("tokenizer.ggml.bos_token_id", 0)
    kv_u32("tokenizer.ggml.eos_token_id", cfg["vocab_size"] - 1)
    kv_u32(a + ".context_length", cfg["max_position_embeddings"])
    kv_u32(a + ".attention.head_count", cfg["num_attention_heads"])
    kv_u32(a + ".attention.head_count_kv", cfg["num_key_value_heads"])
    kv_u32(a + ".attention.key_length", cfg["head_dim"])
    kv_u32(a + ".ssm.inner_size", cfg["mamba_d_ssm"])
    kv_u32(a + ".ssm.state_size", cfg["mamba_d_state"])
    kv_u32(a + ".ssm.group_count", cfg["mamba_n_groups"])
    kv_u32(a + ".ssm.time_step_rank", cfg["mamba_n_heads"])
    kv_u32(a + ".ssm.conv_kernel", cfg["mamba_d_conv"])
    kv_f32(a + ".rope.freq_base", cfg["rope_theta"])
    table = tensor_table(cfg)
    infos, off = [], 0
    for name, shape, kind in table:
        bf16 = kind == "matrix"
        nbytes = int(np.prod(shape)) * (2 if bf16 else 4)
        dims = list(shape)[::-1]                              # fastest-first (core.c:546-592)
        infos.append(_s(name.encode()) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", x) for x in dims)
                     + struct.pack("<IQ", 30 if bf16 else 0, off))
        off += nbytes + (-nbytes) % 32
    head = struct.pack("<IIQQ", 0x46554747, 3, len(table), len(kv)) + b"".join(kv) + b"".join(infos)
    head += b"\0" * ((-len(head)) % 32)
    rng = np.random.default_rng(seed)
    # matrices take their values from one pool of random bfloat16 numbers, read at a different offset for
    # every tensor (drawing 1.5e9 fresh values would take longer than the measurement; speed does not depend on them)
    pool = _bf16_bits(rng.standard_normal(1 << 24, dtype=np.float32) * 0.02)
    with open(path, "wb") as f:
        f.write(head)
        for name, shape, kind in table:
            if kind == "matrix":
                n = int(np.prod(shape))
                start = int(rng.integers(0, pool.size))
                reps = (start + n + pool.size - 1) // pool.size
                raw = np.tile(pool, reps)[start:start + n].tobytes() if reps > 1 else pool[start:start + n].tobytes()
            elif kind == "ones":
                raw = (1.0 + 0.1 * rng.standard_normal(shape)).astype(np.float32).tobytes()
            elif kind == "conv":
                raw = (0.2 * rng.standard_normal(shape)).astype(np.float32).tobytes()
            elif kind == "a":
                raw = (-rng.uniform(1.0, 16.0, shape)).astype(np.float32).tobytes()      # A = -exp(A_log), cpu_op.c:806-808
            elif kind == "d":
                raw = (1.0 + 0.1 * rng.standard_normal(shape)).astype(np.float32).tobytes()
            else:
                dt = np.exp(rng.uniform(np.log(1e-3), np.log(0.1), shape))
                raw = (dt + np.log(-np.expm1(-dt))).astype(np.float32).tobytes()
            f.write(raw + b"\0" * ((-len(raw)) % 32))
        return f.tell()


def run(exe: str, gguf: str, ctx: int, threads: int, prompt_len: int, prefill_len: int, warmup: int, steps: int,
        work: str, timeout: float) -> dict:
    env = dict(os.environ, TINY_LLAMA_LOCK=os.path.join(work, "lock"))
    p = subprocess.run([exe, gguf, str(ctx), str(threads), str(prompt_len), str(prefill_len), str(warmup), str(steps)],
                       env=env, capture_output=True, text=True, timeout=timeout)
    for line in p.stdout.splitlines():
        if line.startswith("RESULT "):
            return json.loads(line[len("RESULT "):])
    raise RuntimeError(f"the reference's driver ended with code {p.returncode}: {p.stderr[-1500:]} {p.stdout[-500:]}")


def measure(cfg: dict, steps: int, warmup: int, prompt_len: int, prefill_len: int, budget_s: float = 600.0,
            layers: int | None = None) -> dict:
    """Builds, calibrates on two layers, then runs as many layers as the time budget allows (all of them
    where it does).  Returns the figures and both layer counts."""
    threads = os.cpu_count() or 1
    full = cfg["num_hidden_layers"]
    with tempfile.TemporaryDirectory(prefix="tlc_ref_") as work:
        t0 = time.time()
        exe = build(work)
        build_s = time.time() - t0
        gguf = os.path.join(work, "model.gguf")
        ctx = cfg["max_position_embeddings"]
        if layers is None:
            small = dict(cfg, num_hidden_layers=min(2, full))
            write_gguf(gguf, small)
            t0 = time.time()
            run(exe, gguf, ctx, threads, prompt_len, prefill_len, 1, max(2, steps // 8), work, timeout=budget_s)
            t_cal = time.time() - t0
            # the calibration's time is dominated by the two prompt passes; scale it by layers
            layers = max(1, min(full, int(budget_s / max(t_cal / small["num_hidden_layers"], 1e-3))))
        use = dict(cfg, num_hidden_layers=layers)
        size = write_gguf(gguf, use)
        r = run(exe, gguf, ctx, threads, prompt_len, prefill_len, warmup, steps, work, timeout=4 * budget_s + 600)
    return dict(r, layers=layers, layers_full=full, threads=threads, gguf_bytes=size, build_s=round(build_s, 1))


if __name__ == "__main__":
    print(prepare(sys.argv[1] if len(sys.argv) > 1 else "/root/reference"))
