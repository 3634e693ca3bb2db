#!/usr/bin/env python3
"""Builds CodeClaper/tinyllama.c's own CPU engine and records its Falcon-H1 logits.

Run once, by hand, on a machine that has the reference checkout and gcc:

    python tests/golden/make_golden.py --reference /path/to/tinyllama.c --out tests/golden

It (1) draws tiny random Falcon-H1 weights under the tensor names the test-suite
uses, (2) writes them as a GGUF v3 file in the layout the reference binds
(core.c:998-1002, 1092-1113; 2-D dims fastest-first, core.c:546-592), folding into
the weights every multiplier the reference has no field for, (3) compiles the
reference's unmodified C sources with a small driver that calls
engine_open / session_create / graph_execute (core.h:28-35, graph.h:89) and
(4) stores tokens, weights and the reference's logits in ``<name>.npz``.

tests/test_plain_vs_reference.py then checks that tests/plain reproduces those
logits from the same weights.  Options the reference cannot express (projection
biases other than q/k/v, norm-before-gate, an eps other than 1e-6) are not in
these files; for them the plain implementation rests on the formulas alone.
"""
from __future__ import annotations

import argparse
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from plain import falcon_h1_plain as plain  # noqa: E402

CONFIGS = {
    # sizes of the first tiny test configuration, eps forced to the reference's constant
    "ref_a": dict(
        vocab_size=64, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=8, intermediate_size=48, rope_theta=10000.0,
        rms_norm_eps=1e-6, tie_word_embeddings=True, attention_bias=False, mlp_bias=False,
        mamba_d_ssm=32, mamba_n_heads=4, mamba_d_head=8, mamba_n_groups=1, mamba_d_state=16,
        mamba_d_conv=4, mamba_conv_bias=True, mamba_proj_bias=False, mamba_rms_norm=True,
        mamba_norm_before_gate=False, max_position_embeddings=256),
    # other sizes, grouped B/C, 3 taps, no conv bias, no ssm norm, q/k/v bias, multipliers
    "ref_b": dict(
        vocab_size=80, hidden_size=48, num_hidden_layers=3, num_attention_heads=6,
        num_key_value_heads=3, head_dim=12, intermediate_size=40, rope_theta=1000000.0,
        rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=True, mlp_bias=False,
        mamba_d_ssm=72, mamba_n_heads=6, mamba_d_head=12, mamba_n_groups=2, mamba_d_state=8,
        mamba_d_conv=3, mamba_conv_bias=False, mamba_proj_bias=False, mamba_rms_norm=False,
        mamba_norm_before_gate=False, max_position_embeddings=256,
        embedding_multiplier=5.0, lm_head_multiplier=0.5, key_multiplier=0.7,
        attention_in_multiplier=1.2, attention_out_multiplier=0.8, ssm_in_multiplier=1.1,
        ssm_out_multiplier=0.9, mlp_multipliers=[0.6, 1.3],
        ssm_multipliers=[0.5, 1.5, 0.8, 1.2, 0.7]),
}
N_TOKENS = 19


def random_weights(cfg: dict, seed: int) -> dict:
    d = plain.derived(cfg)
    rng = np.random.default_rng(seed)

    def mat(*shape, std=0.08):
        return (rng.standard_normal(shape) * std).astype(np.float32)

    W = {"model.embed_tokens.weight": mat(d["V"], d["D"], std=0.5),
         "model.final_layernorm.weight": (1 + mat(d["D"], std=0.1))}
    if not cfg["tie_word_embeddings"]:
        W["lm_head.weight"] = mat(d["V"], d["D"], std=0.3)
    for l in range(d["L"]):
        p = f"model.layers.{l}."
        W[p + "input_layernorm.weight"] = 1 + mat(d["D"], std=0.1)
        W[p + "pre_ff_layernorm.weight"] = 1 + mat(d["D"], std=0.1)
        W[p + "self_attn.q_proj.weight"] = mat(d["H"] * d["hd"], d["D"], std=0.3)
        W[p + "self_attn.k_proj.weight"] = mat(d["KV"] * d["hd"], d["D"], std=0.3)
        W[p + "self_attn.v_proj.weight"] = mat(d["KV"] * d["hd"], d["D"], std=0.2)
        W[p + "self_attn.o_proj.weight"] = mat(d["D"], d["H"] * d["hd"], std=0.2)
        if cfg["attention_bias"]:
            W[p + "self_attn.q_proj.bias"] = mat(d["H"] * d["hd"], std=0.2)
            W[p + "self_attn.k_proj.bias"] = mat(d["KV"] * d["hd"], std=0.2)
            W[p + "self_attn.v_proj.bias"] = mat(d["KV"] * d["hd"], std=0.2)
            W[p + "self_attn.o_proj.bias"] = np.zeros(d["D"], np.float32)   # no such tensor in the reference
        W[p + "mamba.in_proj.weight"] = mat(d["Pd"], d["D"], std=0.2)
        W[p + "mamba.conv1d.weight"] = mat(d["Cd"], 1, d["K"], std=0.4)
        if cfg["mamba_conv_bias"]:
            W[p + "mamba.conv1d.bias"] = mat(d["Cd"], std=0.2)
        W[p + "mamba.A_log"] = np.log(rng.uniform(1, 16, d["Hs"])).astype(np.float32)
        W[p + "mamba.D"] = (1 + mat(d["Hs"], std=0.2))
        dt = np.exp(rng.uniform(np.log(1e-3), np.log(0.1), d["Hs"]))
        W[p + "mamba.dt_bias"] = (dt + np.log(-np.expm1(-dt))).astype(np.float32)
        if cfg["mamba_rms_norm"]:
            W[p + "mamba.norm.weight"] = 1 + mat(d["Di"], std=0.1)
        W[p + "mamba.out_proj.weight"] = mat(d["D"], d["Di"], std=0.2)
        W[p + "feed_forward.gate_proj.weight"] = mat(d["F"], d["D"], std=0.2)
        W[p + "feed_forward.up_proj.weight"] = mat(d["F"], d["D"], std=0.2)
        W[p + "feed_forward.down_proj.weight"] = mat(d["D"], d["F"], std=0.2)
    return W


def fold_for_reference(cfg: dict, W: dict) -> dict:
    """GGUF tensors (reference names) with every multiplier folded into a weight."""
    d = plain.derived(cfg)
    g = lambda k, dflt: cfg.get(k, dflt)
    out = {"token_embd.weight": W["model.embed_tokens.weight"] * g("embedding_multiplier", 1.0),
           "output_norm.weight": W["model.final_layernorm.weight"]}
    if not cfg["tie_word_embeddings"]:
        out["output.weight"] = W["lm_head.weight"] * g("lm_head_multiplier", 1.0)
    else:
        assert g("embedding_multiplier", 1.0) == 1.0 and g("lm_head_multiplier", 1.0) == 1.0
    ain, aout = g("attention_in_multiplier", 1.0), g("attention_out_multiplier", 1.0)
    sin_, sout = g("ssm_in_multiplier", 1.0), g("ssm_out_multiplier", 1.0)
    km = g("key_multiplier", 1.0)
    mg, md = g("mlp_multipliers", [1.0, 1.0])
    m = g("ssm_multipliers", [1.0] * 5)
    mup = np.concatenate([np.full(d["Di"], m[0]), np.full(d["Di"], m[1]), np.full(d["G"] * d["N"], m[2]),
                          np.full(d["G"] * d["N"], m[3]), np.full(d["Hs"], m[4])]).astype(np.float32)
    for l in range(d["L"]):
        p, b = f"model.layers.{l}.", f"blk.{l}."
        out[b + "attn_norm.weight"] = W[p + "input_layernorm.weight"]
        out[b + "ffn_norm.weight"] = W[p + "pre_ff_layernorm.weight"]
        out[b + "attn_q.weight"] = W[p + "self_attn.q_proj.weight"] * ain
        out[b + "attn_k.weight"] = W[p + "self_attn.k_proj.weight"] * (ain * km)
        out[b + "attn_v.weight"] = W[p + "self_attn.v_proj.weight"] * ain
        if cfg["attention_bias"]:
            out[b + "attn_q.bias"] = W[p + "self_attn.q_proj.bias"]
            out[b + "attn_k.bias"] = W[p + "self_attn.k_proj.bias"] * km
            out[b + "attn_v.bias"] = W[p + "self_attn.v_proj.bias"]
        out[b + "attn_output.weight"] = W[p + "self_attn.o_proj.weight"] * aout
        out[b + "ssm_in.weight"] = W[p + "mamba.in_proj.weight"] * sin_ * mup[:, None]
        out[b + "ssm_conv1d.weight"] = W[p + "mamba.conv1d.weight"].reshape(d["Cd"], d["K"])
        if cfg["mamba_conv_bias"]:
            out[b + "ssm_conv1d.bias"] = W[p + "mamba.conv1d.bias"]
        out[b + "ssm_a"] = -np.exp(W[p + "mamba.A_log"])            # cpu_op.c:806-808
        out[b + "ssm_d"] = W[p + "mamba.D"]
        out[b + "ssm_dt.bias"] = W[p + "mamba.dt_bias"]
        if cfg["mamba_rms_norm"]:
            out[b + "ssm_norm.weight"] = W[p + "mamba.norm.weight"]
        out[b + "ssm_out.weight"] = W[p + "mamba.out_proj.weight"] * sout
        out[b + "ffn_gate.weight"] = W[p + "feed_forward.gate_proj.weight"] * mg
        out[b + "ffn_up.weight"] = W[p + "feed_forward.up_proj.weight"]
        out[b + "ffn_down.weight"] = W[p + "feed_forward.down_proj.weight"] * md
    return {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in out.items()}


# ---- GGUF v3 writer (core.c:1349-1395, 519-592) -----------------------------------
def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def write_gguf(path: str, cfg: dict, tensors: dict) -> None:
    d = plain.derived(cfg)
    kv = []

    def kv_u32(k, v): kv.append(_s(k.encode()) + struct.pack("<II", 4, v))
    def kv_f32(k, v): kv.append(_s(k.encode()) + struct.pack("<If", 6, v))
    def kv_str(k, v): kv.append(_s(k.encode()) + struct.pack("<I", 8) + _s(v.encode()))
    def kv_strs(k, vs): kv.append(_s(k.encode()) + struct.pack("<IIQ", 9, 8, len(vs))
                                  + b"".join(_s(v.encode()) for v in vs))

    a = "falcon-h1"
    kv_str("general.architecture", a)
    kv_str("tokenizer.ggml.model", "gpt2")
    kv_strs("tokenizer.ggml.tokens", [f"t{i}" for i in range(d["V"])])
    kv_strs("tokenizer.ggml.merges", [])
    kv_u32("tokenizer.ggml.bos_token_id", 0)
    kv_u32("tokenizer.ggml.eos_token_id", 1)
    kv_u32(a + ".context_length", cfg["max_position_embeddings"])
    kv_u32(a + ".attention.head_count", d["H"])
    kv_u32(a + ".attention.head_count_kv", d["KV"])
    kv_u32(a + ".attention.key_length", d["hd"])
    kv_u32(a + ".ssm.inner_size", d["Di"])
    kv_u32(a + ".ssm.state_size", d["N"])
    kv_u32(a + ".ssm.group_count", d["G"])
    kv_u32(a + ".ssm.time_step_rank", d["Hs"])
    kv_u32(a + ".ssm.conv_kernel", d["K"])
    kv_f32(a + ".rope.freq_base", cfg["rope_theta"])

    infos, blobs, off = [], [], 0
    for name, arr in tensors.items():
        dims = list(arr.shape)[::-1]                      # fastest-first
        infos.append(_s(name.encode()) + struct.pack("<I", len(dims))
                     + b"".join(struct.pack("<Q", x) for x in dims) + struct.pack("<IQ", 0, off))
        raw = arr.tobytes()
        pad = (-len(raw)) % 32
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kv)) + b"".join(kv) + b"".join(infos)
    head += b"\0" * ((-len(head)) % 32)
    with open(path, "wb") as f:
        f.write(head + b"".join(blobs))


DRIVER = r"""
#include <stdio.h>
#include <stdlib.h>
#include "core.h"
#include "graph.h"
int main(int argc, char **argv) {
    /* argv: model.gguf tokens.bin out.bin  -- token by token, then the whole prompt */
    EngineOptons eo = { .model_path = argv[1], .inspect = false };
    Engine *en = engine_open(&eo);
    FILE *f = fopen(argv[2], "rb"); u32 ids[4096]; u32 n = (u32)fread(ids, 4, 4096, f); fclose(f);
    FILE *o = fopen(argv[3], "wb");
    Session *s = session_create(en, 256, 512, 1, 0, 1);
    u32 nv = s->cfg.n_vocab;
    for (u32 i = 0; i < n; i++) {
        if (!graph_execute(s, &ids[i], 1, s->logits)) return 3;
        fwrite(s->logits, 4, nv, o);
    }
    session_free(s);
    s = session_create(en, 256, 512, 1, 0, 1);
    if (!graph_execute(s, ids, n, s->logits)) return 4;
    fwrite(s->logits, 4, nv, o);
    fclose(o);
    return 0;
}
"""

SOURCES = ["core", "quants", "mm", "slog", "utils", "graph", "tokenizer", "sampler", "pthreads",
           "kvcache", "rax", "asctx", "tool", "model/llama", "model/qwen25", "model/qwen35",
           "model/deepseek", "model/falcon", "model/falcon_h1", "model/gemma3",
           "backend/cpu/cpu", "backend/cpu/cpu_op"]


def build_reference(ref: str, work: str) -> str:
    src = os.path.join(ref, "src")
    objs = []
    for s in SOURCES:
        o = os.path.join(work, s.replace("/", "_") + ".o")
        subprocess.check_call(["gcc", "-O1", "-msse4.1", "-pthread", "-I", src, "-c",
                               os.path.join(src, s + ".c"), "-o", o])
        objs.append(o)
    drv = os.path.join(work, "driver.c")
    with open(drv, "w") as f:
        f.write(DRIVER)
    exe = os.path.join(work, "driver")
    subprocess.check_call(["gcc", "-O1", "-pthread", "-I", src, drv, *objs, "-lm", "-o", exe])
    return exe


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as work:
        exe = build_reference(args.reference, work)
        for seed, (name, cfg) in enumerate(CONFIGS.items()):
            W = random_weights(cfg, seed)
            tokens = np.random.default_rng(100 + seed).integers(0, cfg["vocab_size"], N_TOKENS).astype(np.uint32)
            gguf = os.path.join(work, name + ".gguf")
            write_gguf(gguf, cfg, fold_for_reference(cfg, W))
            tokens.tofile(os.path.join(work, "tok.bin"))
            env = dict(os.environ, TINY_LLAMA_LOCK=os.path.join(work, "lock"))
            subprocess.check_call([exe, gguf, os.path.join(work, "tok.bin"), os.path.join(work, "out.bin")],
                                  env=env, stdout=subprocess.DEVNULL)
            out = np.fromfile(os.path.join(work, "out.bin"), np.float32).reshape(N_TOKENS + 1, -1)
            mine = plain.forward(cfg, W, tokens.tolist())
            print(name, "max|reference - plain| token by token:", np.abs(out[:-1] - mine).max(),
                  " whole prompt, last row:", np.abs(out[-1] - mine[-1]).max(),
                  " logit scale:", np.abs(mine).max())
            np.savez_compressed(os.path.join(args.out, name + ".npz"), tokens=tokens,
                                logits_by_token=out[:-1], logits_whole_last=out[-1],
                                config=np.array(repr(cfg)),
                                **{"w:" + k: v for k, v in W.items()})


if __name__ == "__main__":
    main()
