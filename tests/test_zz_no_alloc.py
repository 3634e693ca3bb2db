"""The allocation-free attention entry point, called through its exported C symbol.

Some hosts of this library may not allocate device memory where they call it (a loop with a
no-allocation rule, a plugin in a process that owns all device memory).  For them
`tlc_attention_decode_no_alloc` keeps the split partials of single-token attention in a fixed
array inside the library.  This file checks that it gives what the regular entry point gives,
twice in a row (the second call finds the first call's leftovers in the array), and that it
refuses sizes beyond its built-in scratch.  It is collected last so that a run that stops at
the first failure has already run everything else.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 2 * 1024 * 1024


def _setup(seed, lens, H, KV, hd, dtype):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    pages_needed = [(n + 63) // 64 for n in lens]
    n_pages = sum(pages_needed) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros((B, max(pages_needed) + 1), dtype=torch.int32)
    for b in range(B):
        for i in range(pages_needed[b]):
            table[b, i] = perm.pop()
    dev = "cuda"
    return dict(
        q=torch.randn(B, H * hd, generator=g).to(dtype).to(dev),
        k=torch.randn(n_pages, KV, 64, hd, generator=g).to(dtype).to(dev),
        v=torch.randn(n_pages, KV, 64, hd, generator=g).to(dtype).to(dev),
        table=table.to(dev), pos=torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=dev),
        row_seq=torch.arange(B, dtype=torch.int32, device=dev), slots=torch.arange(B, dtype=torch.int32, device=dev))


def _call_no_alloc(lib, a, out, H, KV, hd, window, max_keys):
    fn = lib.tlc_attention_decode_no_alloc
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, i, vp, vp, vp, i, vp, vp, vp, vp, i, i, i, i, f, i, i, vp]
    fn.restype = ctypes.c_int
    code = 0 if out.dtype == torch.float32 else 1
    return fn(a["q"].data_ptr(), code, a["k"].data_ptr(), a["v"].data_ptr(), a["table"].data_ptr(), a["table"].shape[1],
              a["pos"].data_ptr(), a["row_seq"].data_ptr(), a["slots"].data_ptr(), out.data_ptr(), a["q"].shape[0], H, KV,
              hd, 1.0 / math.sqrt(hd), window, max_keys, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype,H,KV,hd,window", [(torch.bfloat16, 8, 2, 128, 0), (torch.float32, 6, 3, 24, 50)])
def test_no_alloc_entry_point_matches_the_regular_one_twice(dtype, H, KV, hd, window):
    from tinyllama_c_b200 import ops
    from tinyllama_c_b200.csrc import build
    ops.library()
    lib = build.load()                                   # the same shared library, reached through its C symbols
    tol = 2e-5 if dtype == torch.float32 else 6e-3       # the tolerances of tests/test_gpu_kernels.py
    for call, (seed, lens) in enumerate([(1, [700, 3, 129, 64]), (2, [65, 300])]):
        a = _setup(seed, lens, H, KV, hd, dtype)
        max_keys = 1024 if call == 0 else 512
        want = torch.empty_like(a["q"])
        ops.attention(a["q"], a["k"], a["v"], a["table"], a["pos"], a["row_seq"], a["slots"], want, H, KV, hd,
                      1.0 / math.sqrt(hd), window, max_keys)
        got = torch.full_like(a["q"], float("nan"))
        rc = _call_no_alloc(lib, a, got, H, KV, hd, window, max_keys)
        assert rc == 0, lib.tlc_last_error()
        torch.cuda.synchronize()
        err = (got.double() - want.double()).abs().max().item()
        assert err <= tol * want.double().abs().max().item(), f"call {call}: differs by {err:.3e}"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from tinyllama_c_b200 import ops
    from tinyllama_c_b200.csrc import build
    ops.library()
    lib = build.load()
    lib.tlc_last_error.restype = ctypes.c_char_p
    H, KV, hd = 8, 2, 128
    a = _setup(3, [5, 9], H, KV, hd, torch.bfloat16)
    out = torch.zeros_like(a["q"])
    # 2 rows x 8 heads x ceil(max_keys / 128) splits x 130 floats must stay within the scratch
    too_many_keys = (SCRATCH_FLOATS // (2 * 8 * 130) + 2) * 128
    rc = _call_no_alloc(lib, a, out, H, KV, hd, 0, too_many_keys)
    assert rc != 0 and b"exceed the built-in scratch" in lib.tlc_last_error()
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0                 # nothing was launched
