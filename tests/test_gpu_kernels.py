"""Each CUDA kernel alone against its plain PyTorch statement, at sizes other than the
models' (odd widths, head sizes that are no power of two, ragged batches)."""
import math

import pytest
import torch

from tinyllama_c_b200 import ops
from plain import ops_plain

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# output tolerance relative to the output's largest magnitude: float32 accumulation order /
# one bfloat16 rounding of the stored result
TOL = {torch.float32: 2e-5, torch.bfloat16: 6e-3}


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def rnd(g, *shape, dtype=torch.float32, scale=1.0):
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def cmp(name, args_cpu, outs, tol_of=None):
    """Calls ops.<name> on CUDA copies and ops_plain.<name> on the CPU tensors; compares the
    tensors at positions `outs`."""
    args_gpu = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args_cpu]
    getattr(ops, name)(*args_gpu)
    torch.cuda.synchronize()
    getattr(ops_plain, name)(*args_cpu)
    for i in outs:
        ref, got = args_cpu[i].double(), args_gpu[i].cpu().double()
        tol = (tol_of if tol_of is not None else TOL[args_cpu[i].dtype]) * max(1e-6, ref.abs().max().item())
        err = (ref - got).abs().max().item()
        assert err <= tol, f"{name}: output {i} differs by {err:.3e} (allowed {tol:.3e})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    g = gen(0)
    table = rnd(g, 301, 72, dtype=DT[dtype])
    tokens = torch.randint(0, 301, (19,), generator=g, dtype=torch.int32)
    cmp("embed", [tokens, table, 2.5, torch.empty(19, 72)], [3])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D", [72, 1000, 2049])
def test_rmsnorm(dtype, D):
    g = gen(1)
    x = rnd(g, 7, D, scale=3.0)
    w = 1 + rnd(g, D, scale=0.2)
    cmp("rmsnorm", [x, w, 1e-5, torch.empty(7, D, dtype=DT[dtype]), None], [3])
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    cmp("rmsnorm", [x, w, 1e-6, torch.empty(3, D, dtype=DT[dtype]), rows], [3])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D", [72, 1000, 2048, 3072, 4100, 8200])
def test_norms_of_many_rows(dtype, D):
    """From 512 rows on the vector kernels take fewer threads a row with several pieces each."""
    g = gen(3)
    T = 530
    x = rnd(g, T, D, scale=3.0)
    w = 1 + rnd(g, D, scale=0.2)
    cmp("rmsnorm", [x, w, 1e-5, torch.empty(T, D, dtype=DT[dtype]), None], [3])
    groups = 1 if D % 3 else 3
    z = rnd(g, T, D + 4)[:, 4:]
    for before in (False, True):
        args = [x, z, w, 1e-5, groups, before, torch.empty(T, D, dtype=DT[dtype])]
        gpu = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args]
        gpu[1] = torch.cat([torch.zeros(T, 4), z], dim=1).cuda()[:, 4:]      # a strided slice, as in the model
        ops.gated_rmsnorm(*gpu)
        ops_plain.gated_rmsnorm(*args)
        ref, got = args[6].double(), gpu[6].cpu().double()
        assert (ref - got).abs().max() <= TOL[DT[dtype]] * ref.abs().max() * 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("groups,before,with_w", [(1, False, True), (3, True, True), (2, False, False)])
def test_gated_rmsnorm(dtype, groups, before, with_w):
    g = gen(2)
    T, Di = 5, 6 * 26
    y = rnd(g, T, Di, scale=2.0)
    proj = rnd(g, T, Di + 11, dtype=DT[dtype])
    z = proj[:, 4:4 + Di]
    w = 1 + rnd(g, Di, scale=0.2) if with_w else None
    args = [y, z, w, 1e-5, groups, before, torch.empty(T, Di, dtype=DT[dtype])]
    gpu = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args]
    gpu[1] = proj.cuda()[:, 4:4 + Di]
    ops.gated_rmsnorm(*gpu)
    ops_plain.gated_rmsnorm(*args)
    ref, got = args[6].double(), gpu[6].cpu().double()
    assert (ref - got).abs().max() <= TOL[DT[dtype]] * ref.abs().max() * 2
    # the input as two summands (what the scan of prompts leaves), on the vector kernel (aligned) and the plain one
    for Dv, zoff in ((Di, 4), (6 * 24, 0)):
        y1, y2 = rnd(g, T, Dv, scale=2.0), rnd(g, T, Dv, scale=2.0)
        pr = rnd(g, T, Dv + 12, dtype=torch.float32 if zoff == 0 else DT[dtype])
        wv = None if w is None else w[:Dv].contiguous()
        out_cpu, out_gpu = torch.empty(T, Dv, dtype=DT[dtype]), torch.empty(T, Dv, dtype=DT[dtype], device="cuda")
        ops.gated_rmsnorm(y1.cuda(), pr.cuda()[:, zoff:zoff + Dv], None if wv is None else wv.cuda(), 1e-5, groups, before, out_gpu,
                          0.5, y2.cuda())
        ops_plain.gated_rmsnorm(y1, pr[:, zoff:zoff + Dv], wv, 1e-5, groups, before, out_cpu, 0.5, y2)
        assert (out_cpu.double() - out_gpu.cpu().double()).abs().max() <= TOL[DT[dtype]] * out_cpu.double().abs().max() * 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(dtype):
    g = gen(3)
    for in_dt in (torch.float32, DT[dtype]):
        gu = rnd(g, 9, 2 * 77, dtype=in_dt, scale=2.0)
        cmp("swiglu", [gu, torch.empty(9, 77, dtype=DT[dtype])], [1])
        gu = rnd(g, 9, 2 * 80, dtype=in_dt, scale=2.0)
        cmp("swiglu", [gu, torch.empty(9, 80, dtype=DT[dtype]), True], [1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,F,K", [(1, 24, 72), (8, 4096, 2048), (30, 160, 96), (33, 72, 200), (200, 328, 264), (2048, 512, 256)])
def test_linear_with_the_swiglu_epilogue(dtype, M, F, K):
    g = gen(17)
    a = rnd(g, M, K, dtype=DT[dtype])
    w = rnd(g, 2 * F, K, dtype=DT[dtype], scale=2 / math.sqrt(K))
    cs, cb = 1 + rnd(g, 2 * F, scale=0.3), rnd(g, 2 * F, scale=0.3)
    for scale, bias in ((None, None), (cs, cb)):
        cmp("linear_swiglu", [a, w, torch.empty(M, F, dtype=DT[dtype]), scale, bias], [2], tol_of=TOL[DT[dtype]] * 2)
    ops.check_errors()


@pytest.mark.parametrize("a_dt,w_dt,o_dt", [("float32", "float32", "float32"), ("bfloat16", "bfloat16", "bfloat16"),
                                            ("bfloat16", "bfloat16", "float32"), ("bfloat16", "float32", "bfloat16")])
@pytest.mark.parametrize("M,N,K", [(1, 130, 72), (5, 67, 200), (16, 64, 64), (17, 129, 100), (150, 70, 257),
                                   (8, 96, 1024), (17, 130, 72), (32, 40, 136), (33, 130, 72), (64, 200, 264), (65, 130, 72), (9, 2048, 2048), (129, 257, 200), (300, 128, 64), (64, 1000, 1096),
                                   (2048, 384, 512), (100, 1000, 520)])
def test_linear(a_dt, w_dt, o_dt, M, N, K):
    g = gen(4)
    a_full = rnd(g, M, K + 8, dtype=DT[a_dt])
    w = rnd(g, N, K, dtype=DT[w_dt], scale=1 / math.sqrt(K))
    cs, cb = 1 + rnd(g, N, scale=0.3), rnd(g, N)
    for accumulate in (False, True):
        for scale, bias in ((None, None), (cs, cb)):
            out_cpu = rnd(g, M, N + 3, dtype=DT[o_dt])
            out_gpu = out_cpu.cuda()
            a_gpu = a_full.cuda()
            ops.linear(a_gpu[:, :K], w.cuda(), out_gpu[:, :N], None if scale is None else scale.cuda(),
                       None if bias is None else bias.cuda(), accumulate)
            untouched = out_cpu[:, N:].clone()
            ops_plain.linear(a_full[:, :K], w, out_cpu[:, :N], scale, bias, accumulate)
            torch.cuda.synchronize()
            ops.check_errors()
            ref, got = out_cpu[:, :N].double(), out_gpu.cpu()[:, :N].double()
            tol = TOL[DT[o_dt]] * ref.abs().max().item() * (2 if a_dt == "float32" else 1)
            assert (ref - got).abs().max().item() <= tol
            assert torch.equal(out_gpu.cpu()[:, N:], untouched), "linear wrote outside its columns"


@pytest.mark.parametrize("splits", [0, 2, 3, 7])
def test_linear_with_the_k_steps_of_a_tile_shared_among_blocks(splits):
    """Batches of 33..128 rows times narrow matrices: several blocks share a tile's K-steps and the last to
    arrive adds the shares.  Each product runs three times (the arrival counters come back to zero), and two
    run at the same time on two streams (their scratch must not be shared)."""
    g = gen(21)
    try:
        ops.linear_split_override(splits)
        for M, N, K in ((64, 2048, 4096), (100, 200, 520), (40, 136, 264), (128, 1030, 1536)):
            a = rnd(g, M, K, dtype=torch.bfloat16)
            w = rnd(g, N, K, dtype=torch.bfloat16, scale=1 / math.sqrt(K))
            cs, cb = 1 + rnd(g, N, scale=0.3), rnd(g, N)
            for accumulate, scale, bias, o_dt in ((True, None, None, torch.float32), (False, cs, cb, torch.bfloat16),
                                                  (True, cs, None, torch.float32)):
                out_cpu = rnd(g, M, N, dtype=o_dt)
                ops_plain.linear(a, w, ref := out_cpu.clone(), scale, bias, accumulate)
                a_gpu, w_gpu = a.cuda(), w.cuda()
                sc, bi = (None if scale is None else scale.cuda()), (None if bias is None else bias.cuda())
                side = torch.cuda.Stream()
                for rep in range(3):
                    out1, out2 = out_cpu.cuda(), out_cpu.cuda()
                    torch.cuda.synchronize()
                    ops.linear(a_gpu, w_gpu, out1, sc, bi, accumulate)
                    with torch.cuda.stream(side):
                        ops.linear(a_gpu, w_gpu, out2, sc, bi, accumulate)
                    torch.cuda.synchronize()
                    ops.check_errors()
                    for got in (out1, out2):
                        err = (ref.double() - got.cpu().double()).abs().max().item()
                        assert err <= TOL[o_dt] * ref.double().abs().max().item(), f"{M}x{N}x{K}, run {rep}: {err}"
                    assert torch.equal(out1, out2), "two runs of the same product differ"
    finally:
        ops.linear_split_override(0)


@pytest.mark.parametrize("split", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("M,N,K", [(33, 2048, 4096), (64, 8240, 2048), (20, 200, 520), (64, 1000, 1096), (48, 128, 264), (17, 272, 136),
                                   (32, 336, 2056), (100, 2048, 520), (128, 1000, 1096), (65, 400, 264)])
def test_linear_of_17_to_64_rows_with_the_weights_on_the_wide_side(M, N, K, split):
    """Products of 17..128 rows: tiles of 128 weight rows x 32, 64 or 128 activation rows on tcgen05.mma, the K-steps of a
    tile shared among the 1, 2, 4 or 8 blocks of a cluster whose sums meet through distributed shared memory (more
    blocks than K-steps: some have none).  A last tile past N, K that ends inside a stage, fewer rows than the tile
    has columns; plain, into a 32-bit sum, with column scales and biases, and the SwiGLU epilogue; twice each, the
    same bits both times; and within rounding of the kernels that run these sizes otherwise."""
    g = gen(37)
    a = rnd(g, M, K, dtype=torch.bfloat16)
    w = rnd(g, N, K, dtype=torch.bfloat16, scale=1 / math.sqrt(K))
    cs, cb = 1 + rnd(g, N, scale=0.3), rnd(g, N)
    try:
        for accumulate, scale, bias, o_dt in ((True, None, None, torch.float32), (False, cs, cb, torch.bfloat16),
                                              (False, None, None, torch.float32)):
            out_cpu = rnd(g, M, N + 3, dtype=o_dt)
            ops_plain.linear(a, w, (ref := out_cpu.clone())[:, :N], scale, bias, accumulate)
            outs = []
            for on in (True, True, False):
                ops.linear_few_rows(on, split)
                out = out_cpu.cuda()
                ops.linear(a.cuda(), w.cuda(), out[:, :N], None if scale is None else scale.cuda(),
                           None if bias is None else bias.cuda(), accumulate)
                torch.cuda.synchronize()
                ops.check_errors()
                err = (ref.double() - out.cpu().double()).abs().max().item()
                assert err <= TOL[o_dt] * ref.double().abs().max().item(), f"{M}x{N}x{K}, few-rows kernel {on}: {err}"
                assert torch.equal(out.cpu()[:, N:], out_cpu[:, N:]), "wrote past N"
                outs.append(out)
            assert torch.equal(outs[0], outs[1]), "two runs of the same product differ"
        if N % 16 == 0:
            ops.linear_few_rows(True, split)
            for o_dt in (torch.bfloat16, torch.float32):
                cmp("linear_swiglu", [a, w, torch.empty(M, N // 2, dtype=o_dt), cs, cb], [2], tol_of=TOL[torch.bfloat16] * 2)
            ops.check_errors()
    finally:
        ops.linear_few_rows(True, 0)


@pytest.mark.parametrize("pairs", [1, 2])
@pytest.mark.parametrize("M,N,K,pad", [(300, 128, 64, 0), (129, 260, 200, 4), (2048, 384, 512, 0), (100, 1000, 520, 8), (513, 776, 1096, 0),
                                       (70, 2072, 264, 0), (1000, 8240, 136, 0)])
def test_linear_32_bit_outputs_through_the_copy_engine(M, N, K, pad, pairs):
    """32-bit outputs leave the tensor-core product as 32 x 32 tiles by bulk tensor copies: plain stores, and
    adds made at the L2 when the product is summed into its output.  Edges inside a tile in both directions,
    rows longer than N (the columns past N stay as they were), column scales and biases, single blocks and
    pairs; twice each (the staging tile is used again), and the same bits as the epilogue of plain stores."""
    g = gen(36)
    a = rnd(g, M, K, dtype=torch.bfloat16)
    w = rnd(g, N, K, dtype=torch.bfloat16, scale=1 / math.sqrt(K))
    cs, cb = 1 + rnd(g, N, scale=0.3), rnd(g, N)
    try:
        ops.linear_pair_override(pairs)
        for accumulate, scale, bias in ((True, None, None), (False, cs, cb), (True, cs, None), (False, None, None)):
            out_cpu = rnd(g, M, N + pad)
            ops_plain.linear(a, w, (ref := out_cpu.clone())[:, :N], scale, bias, accumulate)
            outs = []
            for tma in (True, True, False):
                try:
                    ops.linear_tma_out(tma)
                    out = out_cpu.cuda()
                    ops.linear(a.cuda(), w.cuda(), out[:, :N], None if scale is None else scale.cuda(),
                               None if bias is None else bias.cuda(), accumulate)
                    torch.cuda.synchronize()
                finally:
                    ops.linear_tma_out(True)
                ops.check_errors()
                err = (ref.double() - out.cpu().double()).abs().max().item()
                assert err <= TOL[torch.float32] * ref.double().abs().max().item(), f"copy engine {tma}: {err}"
                assert torch.equal(out.cpu()[:, N:], out_cpu[:, N:]), "wrote past N"
                outs.append(out)
            assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), "the two epilogues differ"
    finally:
        ops.linear_pair_override(0)


@pytest.mark.parametrize("M,N,K", [(1, 40, 2056), (8, 2048, 4096), (5, 67, 4104), (16, 130, 1096), (13, 2000, 3000), (3, 16, 8200)])
def test_linear_of_few_rows_with_k_halved_between_two_blocks(M, N, K):
    """Few rows times a matrix with fewer 16-column tiles than the GPU has SMs and more than one round of K:
    two blocks of a cluster take one half of K each and the second hands its sums to the first through
    distributed shared memory.  Odd numbers of K-steps, a last tile past N, one and two groups of eight rows;
    plain, into a 32-bit sum and with column scales; twice each, and the same bits both times."""
    g = gen(35)
    a = rnd(g, M, K, dtype=torch.bfloat16)
    w = rnd(g, N, K, dtype=torch.bfloat16, scale=1 / math.sqrt(K))
    cs, cb = 1 + rnd(g, N, scale=0.3), rnd(g, N)
    for accumulate, scale, bias, o_dt in ((True, None, None, torch.float32), (False, cs, cb, torch.bfloat16),
                                          (False, None, None, torch.float32)):
        out_cpu = rnd(g, M, N, dtype=o_dt)
        ops_plain.linear(a, w, ref := out_cpu.clone(), scale, bias, accumulate)
        outs = []
        for paired in (True, True, False):
            try:
                ops.linear_skinny_pairs(paired)
                out = out_cpu.cuda()
                ops.linear(a.cuda(), w.cuda(), out, None if scale is None else scale.cuda(),
                           None if bias is None else bias.cuda(), accumulate)
                torch.cuda.synchronize()
            finally:
                ops.linear_skinny_pairs(True)
            ops.check_errors()
            err = (ref.double() - out.cpu().double()).abs().max().item()
            assert err <= TOL[o_dt] * ref.double().abs().max().item(), f"{M}x{N}x{K}, paired {paired}: {err}"
            outs.append(out)
        assert torch.equal(outs[0], outs[1]), "two runs of the same product differ"


@pytest.mark.parametrize("M,N,K", [(300, 128, 64), (129, 257, 200), (2048, 384, 512), (100, 1000, 520), (256, 512, 4096),
                                   (1000, 520, 264), (513, 776, 1096)])
def test_linear_on_pairs_of_blocks(M, N, K):
    """Tiles of 256 x 256 shared by two blocks (tcgen05.mma.cta_group::2), forced at sizes whose edges fall inside
    a tile, inside one block's half of it, and between the two blocks; plain, into a 32-bit sum, with column
    scales, and with the SwiGLU epilogue.  Twice each: the ring and the barriers' phases carry on across tiles."""
    assert ops.linear_pairs() > 0, "this GPU runs no clusters of two blocks of the product"
    g = gen(33)
    a = rnd(g, M, K, dtype=torch.bfloat16)
    w = rnd(g, N, K, dtype=torch.bfloat16, scale=1 / math.sqrt(K))
    cs, cb = 1 + rnd(g, N, scale=0.3), rnd(g, N)
    try:
        ops.linear_pair_override(2)
        for accumulate, scale, bias, o_dt in ((True, None, None, torch.float32), (False, cs, cb, torch.bfloat16),
                                              (False, None, None, torch.bfloat16)):
            out_cpu = rnd(g, M, N, dtype=o_dt)
            ops_plain.linear(a, w, ref := out_cpu.clone(), scale, bias, accumulate)
            for rep in range(2):
                out = out_cpu.cuda()
                ops.linear(a.cuda(), w.cuda(), out, None if scale is None else scale.cuda(),
                           None if bias is None else bias.cuda(), accumulate)
                torch.cuda.synchronize()
                ops.check_errors()
                err = (ref.double() - out.cpu().double()).abs().max().item()
                assert err <= TOL[o_dt] * ref.double().abs().max().item(), f"{M}x{N}x{K}, run {rep}: {err}"
        if N % 16 == 0:
            cmp("linear_swiglu", [a, w, torch.empty(M, N // 2, dtype=torch.bfloat16), cs, cb], [2], tol_of=TOL[torch.bfloat16] * 2)
            ops.check_errors()
    finally:
        ops.linear_pair_override(0)


def _paged_setup(g, B, lens_total, KV, hd, dtype, n_slots=5, extra_pages=3):
    """Random slots and shuffled pages for sequences of the given total lengths."""
    pages_needed = [(n + 63) // 64 for n in lens_total]
    n_pages = sum(pages_needed) + extra_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_pages = max(pages_needed) + 1
    table = torch.full((n_slots, max_pages), 0, dtype=torch.int32)
    slots = torch.randperm(n_slots, generator=g)[:B].to(torch.int32)
    for b in range(B):
        for i in range(pages_needed[b]):
            table[int(slots[b]), i] = perm.pop()
    k_pages = rnd(g, n_pages, KV, 64, hd, dtype=dtype)
    v_pages = rnd(g, n_pages, KV, 64, hd, dtype=dtype)
    return slots, table, k_pages, v_pages


def _step_arrays(starts, lens):
    pos, row_seq, cu = [], [], [0]
    for b, (s, n) in enumerate(zip(starts, lens)):
        pos += list(range(s, s + n))
        row_seq += [b] * n
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    return i32(pos), i32(row_seq), i32(cu), i32(starts)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("aligned", [False, True])
@pytest.mark.parametrize("H,KV,hd,rope", [(6, 3, 24, 24), (4, 1, 48, 32), (8, 2, 128, 128), (5, 5, 16, 0), (3, 1, 80, 64)])
def test_rope_kv_store(dtype, H, KV, hd, rope, aligned):
    """aligned: the projection's pieces lie on 16-byte boundaries, which the vector kernel needs (a rotated
    width that is a multiple of 8, 32-bit projections); otherwise an element at a time."""
    g = gen(5)
    lead, extra = (4, 8) if aligned else (2, 5)
    starts, lens = [0, 70, 130], [5, 3, 66]
    pos, row_seq, cu, _ = _step_arrays(starts, lens)
    slots, table, k_pages, v_pages = _paged_setup(g, 3, [s + n for s, n in zip(starts, lens)], KV, hd, DT[dtype])
    T = sum(lens)
    width = (H + 2 * KV) * hd
    qkv = rnd(g, T, width + extra, dtype=torch.float32 if H != 4 else DT[dtype])
    inv = (1.0 / torch.pow(torch.tensor(1e6, dtype=torch.float64),
                           torch.arange(rope // 2, dtype=torch.float64) * 2 / max(rope, 1))).float()
    args = [qkv[:, lead:lead + width], 0, H * hd, (H + KV) * hd, torch.empty(T, H * hd, dtype=DT[dtype]), k_pages, v_pages,
            inv, pos, row_seq, slots, table, H, KV, hd, True]
    gpu = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args]
    gpu[0] = qkv.cuda()[:, lead:lead + width]
    ops.rope_kv_store(*gpu)
    ops_plain.rope_kv_store(*args)
    for i in (4, 5, 6):
        ref, got = args[i].double(), gpu[i].cpu().double()
        assert (ref - got).abs().max() <= TOL[DT[dtype]] * ref.abs().max() * 2, f"output {i}"
    # a layer that reads another layer's cache rotates its queries and leaves the pages alone
    k_before, v_before = gpu[5].clone(), gpu[6].clone()
    gpu[4].zero_()
    gpu[-1] = False
    ops.rope_kv_store(*gpu)
    assert torch.equal(gpu[5], k_before) and torch.equal(gpu[6], v_before)
    assert (args[4].double() - gpu[4].cpu().double()).abs().max() <= TOL[DT[dtype]] * args[4].double().abs().max() * 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd,window", [(6, 3, 24, 0), (4, 1, 48, 0), (8, 2, 128, 0), (6, 2, 16, 37), (4, 4, 80, 70)])
def test_attention(dtype, H, KV, hd, window):
    g = gen(6)
    starts, lens = [0, 200, 63, 5], [70, 1, 2, 1]
    pos, row_seq, cu, _ = _step_arrays(starts, lens)
    slots, table, k_pages, v_pages = _paged_setup(g, 4, [s + n for s, n in zip(starts, lens)], KV, hd, DT[dtype])
    T = sum(lens)
    q = rnd(g, T, H * hd, dtype=DT[dtype])
    # one far key stands out for the single-token query of the 201-position sequence
    b1_page = int(table[int(slots[1]), 0])
    k_pages[b1_page, :, 3, :] *= 6.0
    cmp("attention", [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(T, H * hd, dtype=DT[dtype]), H, KV,
                      hd, 1.0 / math.sqrt(hd), window], [7], tol_of=TOL[DT[dtype]] * 2)


@pytest.mark.parametrize("H,KV,hd,window", [(8, 2, 128, 0), (6, 3, 64, 0), (4, 4, 128, 100), (2, 1, 64, 17)])
def test_attention_of_prompts_on_tensor_cores(H, KV, hd, window):
    g = gen(13)
    starts, lens = [0, 130, 63, 5, 0], [200, 70, 2, 65, 1]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    slots, table, k_pages, v_pages = _paged_setup(g, 5, [s + n for s, n in zip(starts, lens)], KV, hd, torch.bfloat16,
                                                  n_slots=7)
    T = sum(lens)
    q = rnd(g, T, H * hd, dtype=torch.bfloat16)
    k_pages[int(table[int(slots[0]), 0]), :, 5, :] *= 5.0        # a far key stands out for late rows
    args = [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(T, H * hd, dtype=torch.bfloat16), H, KV, hd,
            1.0 / math.sqrt(hd), window, 0, cu, start_pos]
    # probabilities are rounded to bfloat16 before the second product: 2^-9 of the output's scale more
    cmp("attention", args, [7], tol_of=TOL[torch.bfloat16] * 2.5)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("H,KV,hd,window", [(8, 2, 128, 0), (6, 3, 64, 0), (4, 4, 128, 100), (2, 1, 64, 17), (3, 1, 128, 0)])
def test_attention_of_prompts_on_tcgen05(H, KV, hd, window, mode):
    """The tcgen05 kernel (mode 0) and the mma.sync one (mode 1) on the same step: prompts that cross 128-row tiles,
    one that continues at position 130, single rows, a window.  One early key and one late key are scaled up: the
    late one makes a row's maximum jump by far more than 2^8 in a late key tile, which is where the output
    accumulator in tensor memory is rescaled."""
    g = gen(33)
    starts, lens = [0, 130, 63, 5, 0], [333, 200, 2, 129, 1]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    totals = [s + n for s, n in zip(starts, lens)]
    slots, table, k_pages, v_pages = _paged_setup(g, 5, totals, KV, hd, torch.bfloat16, n_slots=7)
    T = sum(lens)
    q = rnd(g, T, H * hd, dtype=torch.bfloat16)
    k_pages[int(table[int(slots[0]), 0]), :, 5, :] *= 5.0        # position 5: stands out from the first tile on
    k_pages[int(table[int(slots[0]), 3]), :, 10, :] *= 12.0      # position 202: a jump in the fourth key tile
    args = [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(T, H * hd, dtype=torch.bfloat16), H, KV, hd,
            1.0 / math.sqrt(hd), window, 0, cu, start_pos, max(totals)]
    ops.prompt_attention_override(mode)
    try:
        cmp("attention", args, [7], tol_of=TOL[torch.bfloat16] * 2.5)
        torch.cuda.synchronize()
        ops.check_errors()
    finally:
        ops.prompt_attention_override(0)


@pytest.mark.parametrize("max_blocks", [1, 3, 7, 1000])
@pytest.mark.parametrize("H,KV,hd,window", [(8, 2, 128, 0), (3, 1, 64, 0), (4, 4, 128, 100)])
def test_attention_of_prompts_on_a_bounded_number_of_blocks(H, KV, hd, window, max_blocks):
    """The tcgen05 kernel with fewer blocks than (tile, head) items: a block works through several items one after
    the other (long and short ones, tiles of different sequences and heads, tiles past the step's last), its
    barriers made anew in between, tensor memory and shared memory used again.  The same bits as one block an item."""
    g = gen(34)
    starts, lens = [0, 130, 63, 5, 0], [333, 200, 2, 129, 1]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    totals = [s + n for s, n in zip(starts, lens)]
    slots, table, k_pages, v_pages = _paged_setup(g, 5, totals, KV, hd, torch.bfloat16, n_slots=7)
    T = sum(lens)
    q = rnd(g, T, H * hd, dtype=torch.bfloat16)
    k_pages[int(table[int(slots[0]), 3]), :, 10, :] *= 12.0      # a jump of a row's maximum in the fourth key tile
    args = [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(T, H * hd, dtype=torch.bfloat16), H, KV, hd,
            1.0 / math.sqrt(hd), window, 0, cu, start_pos, max(totals)]
    cmp("attention", args + [max_blocks], [7], tol_of=TOL[torch.bfloat16] * 2.5)
    outs = []
    for mb in (0, max_blocks, max_blocks):
        out = torch.empty(T, H * hd, dtype=torch.bfloat16, device="cuda")
        gpu = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args]
        gpu[7] = out
        ops.attention(*gpu, mb)
        torch.cuda.synchronize()
        ops.check_errors()
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2]), "the result depends on the number of blocks"


@pytest.mark.parametrize("key_ranges", [0, 2, 3, 8])
@pytest.mark.parametrize("H,KV,hd,window", [(8, 2, 128, 0), (3, 1, 64, 0), (4, 4, 128, 700)])
def test_attention_of_prompt_pieces_with_the_keys_in_ranges(H, KV, hd, window, key_ranges):
    """The tcgen05 kernel with the keys of every row tile cut into ranges that run as items of their own and are added
    up by a second kernel: a 70-row piece at position 3,000 (what the kernel chooses ranges for by itself), a
    200-row piece at position 130, short sequences most of whose ranges are empty, a window; a far key stands out."""
    g = gen(38)
    starts, lens = [3000, 130, 0, 2100], [70, 200, 3, 129]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    totals = [s + n for s, n in zip(starts, lens)]
    slots, table, k_pages, v_pages = _paged_setup(g, 4, totals, KV, hd, torch.bfloat16, n_slots=6)
    T = sum(lens)
    q = rnd(g, T, H * hd, dtype=torch.bfloat16)
    k_pages[int(table[int(slots[0]), 1]), :, 9, :] *= 4.0        # position 73 of the long sequence: in the first range
    k_pages[int(table[int(slots[0]), 40]), :, 10, :] *= 6.0      # position 2,570: in a late range
    args = [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(T, H * hd, dtype=torch.bfloat16), H, KV, hd,
            1.0 / math.sqrt(hd), window, 0, cu, start_pos, max(totals), 0, key_ranges]
    cmp("attention", args, [7], tol_of=TOL[torch.bfloat16] * 2.5)
    torch.cuda.synchronize()
    ops.check_errors()


@pytest.mark.parametrize("H,KV,hd,window", [(4, 2, 128, 0), (2, 1, 64, 0), (4, 4, 64, 700)])
def test_attention_of_long_prompts_in_pieces(H, KV, hd, window):
    """Key ranges of more than 8 pages are cut into pieces that run side by side and are merged: a prompt of
    1,500 rows, one that continues at position 900, and a short one whose rows are written whole."""
    g = gen(23)
    starts, lens = [0, 900, 40], [1500, 300, 30]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    slots, table, k_pages, v_pages = _paged_setup(g, 3, [s + n for s, n in zip(starts, lens)], KV, hd, torch.bfloat16,
                                                  n_slots=4)
    T = sum(lens)
    q = rnd(g, T, H * hd, dtype=torch.bfloat16)
    k_pages[int(table[int(slots[0]), 1]), :, 9, :] *= 4.0        # a far key (position 73) stands out for late rows
    args = [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(T, H * hd, dtype=torch.bfloat16), H, KV, hd,
            1.0 / math.sqrt(hd), window, 0, cu, start_pos, 1500]
    cmp("attention", args, [7], tol_of=TOL[torch.bfloat16] * 2.5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd,window", [(6, 3, 24, 0), (4, 1, 48, 0), (8, 2, 128, 0), (6, 2, 16, 37), (8, 1, 80, 170)])
def test_attention_of_single_token_steps(dtype, H, KV, hd, window):
    g = gen(12)
    starts, lens = [0, 200, 63, 700, 128], [1, 1, 1, 1, 1]
    pos, row_seq, cu, _ = _step_arrays(starts, lens)
    slots, table, k_pages, v_pages = _paged_setup(g, 5, [s + n for s, n in zip(starts, lens)], KV, hd, DT[dtype], n_slots=6)
    q = rnd(g, 5, H * hd, dtype=DT[dtype])
    k_pages[int(table[int(slots[3]), 0]), :, 3, :] *= 6.0        # a far key stands out
    for max_keys in (701, 1024):
        cmp("attention", [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(5, H * hd, dtype=DT[dtype]), H, KV,
                          hd, 1.0 / math.sqrt(hd), window, max_keys], [7], tol_of=TOL[DT[dtype]] * 2)


@pytest.mark.parametrize("write", [True, False])
@pytest.mark.parametrize("H,KV,hd,rope,window,longest", [
    (8, 2, 128, 128, 0, 700), (6, 3, 64, 32, 0, 700), (4, 4, 128, 0, 100, 700), (7, 1, 64, 64, 17, 700), (2, 2, 256, 128, 0, 700),
    (8, 2, 128, 128, 0, 5000), (6, 3, 64, 64, 300, 3400)])
def test_attention_of_single_token_steps_in_one_kernel(H, KV, hd, rope, window, longest, write):
    """Rotation, store of the new row and attention in one launch, against the three plain steps;
    run several times so that the arrival counters are seen to come back to zero.  The long
    contexts take pieces of 256 keys, several a block; then the number of pieces a block takes one after
    the other is fixed: two, three, and all of them (one block per row and head group, which writes the
    output itself)."""
    g = gen(14)
    starts = [0, 200, 63, longest, 127, 128]
    lens = [1] * len(starts)
    B = len(starts)
    pos, row_seq, cu, _ = _step_arrays(starts, lens)
    slots, table, k_pages, v_pages = _paged_setup(g, B, [s + 1 for s in starts], KV, hd, torch.bfloat16, n_slots=7)
    k_pages[int(table[int(slots[3]), 0]), :, 3, :] *= 4.0        # a far key stands out
    width = (H + 2 * KV) * hd
    qkv = rnd(g, B, width + 7)
    view = lambda t: t[:, 3:3 + width]
    inv = (1.0 / torch.pow(torch.tensor(1e4, dtype=torch.float64),
                           torch.arange(rope // 2, dtype=torch.float64) * 2 / max(rope, 1))).float()
    scale = 1.0 / math.sqrt(hd)
    # plain: rotate and store, then attend
    k_ref, v_ref = k_pages.clone(), v_pages.clone()
    q_ref = torch.empty(B, H * hd, dtype=torch.bfloat16)
    ops_plain.rope_kv_store(view(qkv), 0, H * hd, (H + KV) * hd, q_ref, k_ref, v_ref, inv, pos, row_seq, slots, table, H, KV,
                            hd, write)
    out_ref = torch.empty(B, H * hd, dtype=torch.bfloat16)
    ops_plain.attention(q_ref, k_ref, v_ref, table, pos, row_seq, slots, out_ref, H, KV, hd, scale, window)
    counters = ops.new_arrival_counters("cuda")
    try:
        for max_keys, passes in ((longest + 1, 0), ((longest // 1024 + 1) * 1024, 0), (longest + 1, 0), (longest + 1, 2),
                                 ((longest // 1024 + 1) * 1024, 3), (longest + 1, 1000), (longest + 200, 1000)):
            ops.attention_decode_fused_passes(passes)
            k_gpu, v_gpu = k_pages.cuda(), v_pages.cuda()
            out = torch.empty(B, H * hd, dtype=torch.bfloat16, device="cuda")
            qkv_gpu = qkv.cuda()
            assert ops.attention_decode_fused_ok(view(qkv_gpu), torch.bfloat16, H, KV, hd)
            ops.attention_decode_fused(view(qkv_gpu), 0, H * hd, (H + KV) * hd, k_gpu, v_gpu, inv.cuda(), write, table.cuda(),
                                       pos.cuda(), row_seq.cuda(), slots.cuda(), out, H, KV, hd, scale, window, max_keys,
                                       counters)
            assert int(counters.abs().sum()) == 0        # every launch leaves its counters at zero
            ref = out_ref.double()
            assert (ref - out.cpu().double()).abs().max() <= TOL[torch.bfloat16] * 2 * ref.abs().max()
            for name, got, want in (("keys", k_gpu, k_ref), ("values", v_gpu, v_ref)):
                d = (got.cpu().double() - want.double()).abs().max()
                assert d <= TOL[torch.bfloat16] * want.double().abs().max(), f"{name} in the pages differ by {d}"
                if not write:
                    assert torch.equal(got.cpu(), want), f"{name} were written although the layer only reads"
    finally:
        ops.attention_decode_fused_passes(0)
    assert not ops.attention_decode_fused_ok(view(qkv_gpu), torch.bfloat16, H, KV, 80)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd", [(4, 2, 64), (8, 2, 128), (6, 3, 24)])
def test_outputs_into_columns_of_a_wider_buffer(dtype, H, KV, hd):
    """Attention (every kernel of it) and the gated norm write into a range of the columns of a wider
    buffer exactly what they write into a dense output, and nothing beside it; the gated norm's
    output scale multiplies its result."""
    g = gen(31)
    dt = DT[dtype]
    W, off = H * hd, 40
    wide = lambda T: torch.full((T, W + 104), 7.0, dtype=dt, device="cuda")

    def both(run, T):
        dense, buf = torch.empty(T, W, dtype=dt, device="cuda"), wide(T)
        run(dense)
        run(buf[:, off:off + W])
        torch.cuda.synchronize()
        assert torch.equal(buf[:, off:off + W], dense)
        assert bool((buf[:, :off] == 7.0).all()) and bool((buf[:, off + W:] == 7.0).all()), "wrote outside its columns"
        return dense

    scale = 1.0 / math.sqrt(hd)
    # prompts (the tiled kernel for bfloat16 heads of 64 and 128, whole and in pieces; else a warp per row and head)
    starts, lens = [0, 130, 5], [700, 70, 65]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    slots, table, k_pages, v_pages = _paged_setup(g, 3, [s + n for s, n in zip(starts, lens)], KV, hd, dt, n_slots=4)
    T = sum(lens)
    q = rnd(g, T, W, dtype=dt).cuda()
    dev = [t.cuda() for t in (k_pages, v_pages, table, pos, row_seq, slots, cu, start_pos)]
    for max_keys in (0, 700):
        both(lambda out: ops.attention(q, dev[0], dev[1], dev[2], dev[3], dev[4], dev[5], out, H, KV, hd, scale, 0, 0,
                                       dev[6], dev[7], max_keys), T)
    # single-token steps: split keys with a merge, and the one-kernel form
    starts, lens = [699, 199, 69], [1, 1, 1]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    pos, row_seq = pos.cuda(), row_seq.cuda()
    q1 = rnd(g, 3, W, dtype=dt).cuda()
    both(lambda out: ops.attention(q1, dev[0], dev[1], dev[2], pos, row_seq, dev[5], out, H, KV, hd, scale, 0, 700), 3)
    qkv = rnd(g, 3, (H + 2 * KV) * hd).cuda()
    inv = (1.0 / torch.pow(torch.tensor(1e4, dtype=torch.float64), torch.arange(hd // 2, dtype=torch.float64) * 2 / hd)).float().cuda()
    if ops.attention_decode_fused_ok(qkv, dt, H, KV, hd):
        counters = ops.new_arrival_counters("cuda")
        for max_keys in (700, 128):          # several blocks a row with a merge; one block a row
            if max_keys == 128:
                pos = torch.tensor([100, 90, 69], dtype=torch.int32, device="cuda")
            both(lambda out: ops.attention_decode_fused(qkv, 0, H * hd, (H + KV) * hd, dev[0], dev[1], inv, False, dev[2],
                                                        pos, row_seq, dev[5], out, H, KV, hd, scale, 0, max_keys, counters), 3)
    # gated norm: vector and scalar kernels, with and without weights, scaled
    y = rnd(g, 5, W, scale=2.0).cuda()
    for zdt, w in ((torch.float32, 1 + rnd(g, W, scale=0.2).cuda()), (dt, 1 + rnd(g, W, scale=0.2).cuda()), (dt, None)):
        z = rnd(g, 5, W, dtype=zdt).cuda()
        plain = both(lambda out: ops.gated_rmsnorm(y, z, w, 1e-5, 2, False, out), 5)
        scaled = both(lambda out: ops.gated_rmsnorm(y, z, w, 1e-5, 2, False, out, 0.75), 5)
        assert (scaled.double() - 0.75 * plain.double()).abs().max() <= TOL[dt] * 2 * plain.double().abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Di,G,N,K,Hs,bias", [(48, 1, 16, 4, 3, True), (144, 2, 32, 3, 6, False), (40, 1, 8, 2, 5, True)])
def test_mamba_conv(dtype, Di, G, N, K, Hs, bias):
    g = gen(7)
    Cd = Di + 2 * G * N
    Pd = Di + Cd + Hs
    starts, lens = [0, 9, 0, 31], [7, 1, 2, 5]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    slots = torch.tensor([4, 0, 2, 1], dtype=torch.int32)
    T = sum(lens)
    proj = rnd(g, T, Pd, dtype=DT[dtype])
    state = rnd(g, 5, K - 1, Cd)
    args = [proj, Di, Di + Cd, rnd(g, Cd, K, scale=0.5), rnd(g, Cd) if bias else None, rnd(g, Hs),
            -torch.rand(Hs, generator=g) * 8, state, cu, row_seq, slots, start_pos, torch.empty(T, Cd),
            torch.empty(T, Hs), torch.empty(T, Hs)]
    cmp("mamba_conv", args, [7, 12, 13, 14], tol_of=2e-5)
    # x|B|C written in bfloat16, as the scan in matrix form takes it
    args16 = list(args)
    args16[7], args16[12] = state.clone(), torch.empty(T, Cd, dtype=torch.bfloat16)
    cmp("mamba_conv", args16, [12], tol_of=6e-3)
    cmp("mamba_conv", args16[:7] + [state.clone()] + args16[8:], [7, 13, 14], tol_of=2e-5)
    # long sequences: blocks of 8 rows that lie inside one sequence, three or more rows from its start, take a path
    # of their own (no window, no per-row branches); the blocks around them (a sequence's first rows, a block across
    # two sequences, the last rows of the step) do not
    starts, lens = [0, 40, 0, 5], [45, 3, 26, 13]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    T = sum(lens)
    for o_dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 6e-3)):
        long_args = [rnd(g, T, Pd, dtype=DT[dtype]), Di, Di + Cd, args[3], args[4], args[5], args[6], state.clone(), cu, row_seq,
                     slots, start_pos, torch.empty(T, Cd, dtype=o_dt), torch.empty(T, Hs), torch.empty(T, Hs)]
        cmp("mamba_conv", long_args, [7, 12, 13, 14], tol_of=tol)
    # every sequence at position 0: the rows' kernel leaves the new windows itself (sequences shorter than the
    # window, of exactly its length, ending inside a block of 8 rows and on its last row)
    starts, lens = [0, 0, 0, 0], [1, K - 1, 30, 9]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    T = sum(lens)
    for o_dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 6e-3)):
        fresh_args = [rnd(g, T, Pd, dtype=DT[dtype]), Di, Di + Cd, args[3], args[4], args[5], args[6], state.clone(), cu, row_seq,
                      slots, start_pos, torch.empty(T, Cd, dtype=o_dt), torch.empty(T, Hs), torch.empty(T, Hs), False, False, True]
        cmp("mamba_conv", fresh_args, [7, 12, 13, 14], tol_of=tol)
    # one row per sequence: the fused kernel of decode steps
    starts, lens = [0, 9, 1, 31, 2], [1, 1, 1, 1, 1]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    slots = torch.tensor([4, 0, 2, 1, 3], dtype=torch.int32)
    args = [rnd(g, 5, Pd, dtype=DT[dtype]), Di, Di + Cd, args[3], args[4], args[5], args[6], rnd(g, 5, K - 1, Cd), cu,
            row_seq, slots, start_pos, torch.empty(5, Cd), torch.empty(5, Hs), torch.empty(5, Hs), True]
    cmp("mamba_conv", args, [7, 12, 13, 14], tol_of=2e-5)


@pytest.mark.parametrize("Hs,P,N,G", [(3, 16, 16, 1), (6, 24, 32, 2), (4, 64, 256, 1), (2, 20, 100, 2), (5, 7, 40, 1)])
def test_ssm_scan(Hs, P, N, G):
    g = gen(8)
    Di, Cd = Hs * P, Hs * P + 2 * G * N
    starts, lens = [0, 9, 0], [19, 1, 3]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    T = sum(lens)
    dt = torch.rand(T, Hs, generator=g) * 0.1
    dA = torch.exp(-dt * torch.rand(Hs, generator=g) * 8)
    args = [rnd(g, T, Cd), dt, dA, 1 + rnd(g, Hs, scale=0.1), rnd(g, 4, Hs, P, N), cu, slots, start_pos,
            torch.empty(T, Di), Hs, P, N, G]
    cmp("ssm_scan", args, [4, 8], tol_of=2e-5)


@pytest.mark.parametrize("Hs,P,N,G", [(3, 16, 16, 1), (4, 64, 256, 1), (2, 20, 100, 2)])
def test_ssm_scan_in_parallel_chunks(Hs, P, N, G):
    """Sequences cut into chunks of unequal sizes, one continuing from its slot's state."""
    g = gen(14)
    Di, Cd = Hs * P, Hs * P + 2 * G * N
    starts, lens = [0, 9, 0], [300, 70, 1]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    T = sum(lens)
    seg_start, seg_seq, seq_seg_start = [], [], [0]
    for b, n in enumerate(lens):
        for off in range(0, n, 128):
            seg_start.append(int(cu[b]) + off)
            seg_seq.append(b)
        seq_seg_start.append(len(seg_seq))
    seg_start.append(T)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    dt = torch.rand(T, Hs, generator=g) * 0.1
    dA = torch.exp(-dt * torch.rand(Hs, generator=g) * 8)
    args = [rnd(g, T, Cd), dt, dA, 1 + rnd(g, Hs, scale=0.1), rnd(g, 4, Hs, P, N), cu, slots, start_pos,
            torch.empty(T, Di), Hs, P, N, G, (i32(seg_start), i32(seg_seq), i32(seq_seg_start))]
    gpu = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args]
    gpu[13] = tuple(t.cuda() for t in args[13])
    ops.ssm_scan(*gpu)
    ops_plain.ssm_scan(*args)
    for i in (4, 8):
        ref, got = args[i].double(), gpu[i].cpu().double()
        assert (ref - got).abs().max() <= 3e-5 * ref.abs().max(), f"output {i}"


@pytest.mark.parametrize("Hs,P,N,G", [(4, 64, 256, 1), (6, 64, 64, 2), (2, 128, 128, 1), (3, 32, 192, 1), (2, 96, 64, 2)])
def test_ssm_scan_in_matrix_form_on_tensor_cores(Hs, P, N, G):
    """The chunked matrix form (bfloat16 operands, the state carried on chip from chunk to chunk) against the
    sequential recurrence on the same bfloat16 x|B|C; one sequence continues from its slot's state, one is
    shorter than a chunk, one ends one row into its second chunk, one is a single row."""
    g = gen(15)
    Di, Cd = Hs * P, Hs * P + 2 * G * N
    starts, lens = [0, 9, 0, 77], [300, 70, 129, 1]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    slots = torch.tensor([2, 0, 3, 1], dtype=torch.int32)
    T = sum(lens)
    seg_start, seg_seq, seq_seg_start = [], [], [0]
    for b, n in enumerate(lens):
        for off in range(0, n, 128):
            seg_start.append(int(cu[b]) + off)
            seg_seq.append(b)
        seq_seg_start.append(len(seg_seq))
    seg_start.append(T)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    dt = torch.rand(T, Hs, generator=g) * 0.1
    A = -torch.rand(Hs, generator=g) * 8
    dA = torch.exp(dt * A)
    args = [rnd(g, T, Cd, dtype=torch.bfloat16), dt, dA, 1 + rnd(g, Hs, scale=0.1), rnd(g, 4, Hs, P, N), cu, slots, start_pos,
            torch.empty(T, Di), Hs, P, N, G, (i32(seg_start), i32(seg_seq), i32(seq_seg_start)), A]
    args0 = [a.clone() if isinstance(a, torch.Tensor) else a for a in args]       # the plain scan updates its state in place
    assert ops.ssd_ok(Hs, P, N, G)
    ops_plain.ssm_scan(*args)
    # states of 128 or 256 columns: the walk with tcgen05.mma and the state in tensor memory (the outputs in one
    # piece, and as two summands of which one is computed on a second stream), and the mma.sync walk
    # (and the tcgen05 walk with one block and with three for all of its (sequence, head, rows) items: a block then
    # walks several sequences in turn, its barriers made anew and its tensor memory used again)
    variants = ((0, False, 0), (0, True, 0), (1, False, 0), (1, True, 0), (0, True, 1), (0, False, 3)) if N in (128, 256) \
        else ((0, False, 0), (0, True, 0))
    for mode, in_two, blocks in variants:
        gpu = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args0]
        gpu[13] = tuple(t.cuda() for t in args0[13])
        y_part = torch.full((T, Di), float("nan"), device="cuda") if in_two else None
        ops.ssd_walk_override(mode)
        ops.ssd_walk_blocks(blocks)
        try:
            used = ops.ssm_scan(*gpu, y_part=y_part)
            torch.cuda.synchronize()
            ops.check_errors()
        finally:
            ops.ssd_walk_override(0)
            ops.ssd_walk_blocks(0)
        assert used == (in_two and mode == 0 and N in (128, 256)), "which walks leave two summands"
        if used:
            gpu[8] = gpu[8] + y_part
        for i in (4, 8):
            ref, got = args[i].double(), gpu[i].cpu().double()
            # bfloat16 operands carry 8 bits: C B^T, the score matrix, the weighted x and the carried state's copy are
            # each rounded to 2^-9 of their size before a product; sums over up to 128 rows and N columns of them
            assert (ref - got).abs().max() <= 1.5e-2 * ref.abs().max(), \
                f"walk {mode}, output {i}: {(ref - got).abs().max()} of {ref.abs().max()}"
            assert (ref - got).abs().mean() <= 1.5e-3 * ref.abs().max(), f"walk {mode}, output {i} (mean)"


@pytest.mark.parametrize("N", [64, 128, 256])
def test_ssm_scan_in_matrix_form_finds_one_far_row(N):
    """One row's x is 100 times the others' and decay is slow: its contribution must reach rows in later chunks
    through the carried state with the right decay (a chunk's state dropped or doubled shows at once)."""
    Hs, P, G = 2, 64, 1
    g = gen(16)
    Di, Cd = Hs * P, Hs * P + 2 * G * N
    lens, starts = [400], [0]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    slots = torch.tensor([1], dtype=torch.int32)
    T = 400
    xbc = rnd(g, T, Cd, scale=0.3)
    xbc[5, :Di] *= 100.0
    xbc = xbc.to(torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    chunks = (i32([0, 128, 256, 384, 400]), i32([0, 0, 0, 0]), i32([0, 4]))
    dt = torch.full((T, Hs), 0.01)
    A = torch.tensor([-0.5, -1.0])
    args = [xbc, dt, torch.exp(dt * A), torch.ones(Hs), torch.zeros(2, Hs, P, N), cu, slots, start_pos,
            torch.empty(T, Di), Hs, P, N, G, chunks, A]
    gpu = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args]
    gpu[13] = tuple(t.cuda() for t in chunks)
    ops.ssm_scan(*gpu)
    ops_plain.ssm_scan(*args)
    ref, got = args[8].double(), gpu[8].cpu().double()
    for lo, hi in ((0, 128), (128, 256), (256, 384), (384, 400)):
        scale = ref[lo:hi].abs().max()
        assert (ref[lo:hi] - got[lo:hi]).abs().max() <= 1.5e-2 * scale, f"rows {lo}..{hi}"


def test_argmax_takes_the_first_maximum():
    g = gen(9)
    logits = rnd(g, 6, 1000)
    logits[2, 17] = logits[2, 900] = 50.0
    logits[4, 999] = 60.0
    cmp("argmax", [logits, torch.empty(6, dtype=torch.int32)], [1], tol_of=0.0)
    # a row spread over blocks of 2,048 values: ties across blocks, negative rows, a vocabulary that is no multiple
    # of the slice; the workspace is zero again afterwards, so a second launch on it works
    big = rnd(g, 5, 70001)
    big[0, 5] = big[0, 69999] = 90.0          # equal maxima in the first and the last slice: the first wins
    big[1] = -big[1].abs() - 1.0
    big[1, 4097] = -0.5
    big[3, 70000] = 95.0
    work = ops.new_argmax_work(5, "cuda")
    for _ in range(2):
        cmp("argmax", [big, torch.empty(5, dtype=torch.int32), work], [1], tol_of=0.0)
        assert int(work.abs().sum()) == 0


@pytest.mark.parametrize("params", [
    dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.05, rp=1.1, fp=0.0, pp=0.0),
    dict(temperature=1.3, top_k=0, top_p=0.7, min_p=0.0, rp=1.0, fp=0.2, pp=0.1),
    dict(temperature=0.5, top_k=5, top_p=1.0, min_p=0.0, rp=1.0, fp=0.0, pp=0.0),
    dict(temperature=1.0, top_k=0, top_p=1.0, min_p=0.2, rp=1.3, fp=0.0, pp=0.0),
    dict(temperature=0.0, top_k=40, top_p=0.9, min_p=0.05, rp=1.2, fp=0.0, pp=0.0),
])
def test_sample_equals_the_plain_sampler(params):
    g = gen(10)
    R, V = 24, 777
    logits = rnd(g, R, V, scale=2.5)
    hist = torch.randint(0, V, (R, 20), generator=g, dtype=torch.int32)
    hist[:, 15:] = -1
    hist[3, :4] = 5
    u = torch.rand(R, generator=g)
    args = [logits, torch.empty(R, V), hist, u, params["temperature"], params["top_k"], params["top_p"],
            params["min_p"], params["rp"], params["fp"], params["pp"], torch.empty(R, dtype=torch.int32)]
    gpu = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args]
    ops.sample(*gpu)
    ops_plain.sample(*args)
    got, ref = gpu[11].cpu(), args[11]
    # a draw that lands within float32 rounding of a boundary of the CDF may pick the neighbour
    assert (got != ref).sum().item() <= 1, f"{(got != ref).sum().item()} of {R} draws differ: {got} vs {ref}"


@pytest.mark.parametrize("case", ["ties at the cut", "fewer positive than top-k", "top-k 1024", "top-k 1500", "large vocabulary"])
def test_sample_cuts_and_ties(case):
    """The cuts where they are decided by order rather than by value: equal probabilities at the top-k and
    top-p cuts (the first in token-id order stay), probabilities that underflow to zero, and a top-k at and
    beyond what the short-list kernel holds."""
    g = gen(12)
    R, V, T, k, top_p, min_p = 16, 3000, 0.8, 40, 0.9, 0.0
    logits = rnd(g, R, V, scale=2.5)
    if case == "ties at the cut":
        logits = (logits * 2).round() / 2          # steps of 0.5: dozens of tokens share each of the top values
        k = 12
    elif case == "fewer positive than top-k":
        logits, T, k = logits * 40, 0.05, 200      # exp((l - max) / T) underflows for all but a few tokens
    elif case == "top-k 1024":
        k, top_p = 1024, 0.97
    elif case == "top-k 1500":
        k, top_p = 1500, 0.97
    elif case == "large vocabulary":
        V = 130048
        logits = rnd(g, R, V, scale=3.0)
        logits[:, 7::1000] += 6.0
    u = torch.rand(R, generator=g)
    u[0], u[1] = 0.0, 0.9999999
    args = [logits, torch.empty(R, V), None, u, T, k, top_p, min_p, 1.0, 0.0, 0.0, torch.empty(R, dtype=torch.int32)]
    gpu = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args]
    ops.sample(*gpu)
    ops_plain.sample(*args)
    got, ref = gpu[11].cpu(), args[11]
    assert (got != ref).sum().item() <= 1, f"{case}: {(got != ref).sum().item()} of {R} draws differ: {got} vs {ref}"


def test_sample_frequencies_follow_the_filtered_distribution():
    g = gen(11)
    V, R = 50, 4000
    row = rnd(g, 1, V, scale=1.5)
    logits = row.repeat(R, 1).contiguous()
    u = torch.rand(R, generator=g)
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(logits.cuda(), torch.empty(R, V, device="cuda"), None, u.cuda(), 0.9, 8, 0.95, 0.02, 1.0, 0.0, 0.0, out)
    from plain.falcon_h1_plain import filtered_distribution
    ids, probs = filtered_distribution(row[0].numpy(), 0.9, 8, 0.95, 0.02)
    counts = torch.bincount(out.cpu().long(), minlength=V).double() / R
    assert set(counts.nonzero().flatten().tolist()) <= set(int(i) for i in ids)
    for i, p in zip(ids, probs):
        assert abs(counts[int(i)].item() - p) < 4 * math.sqrt(p * (1 - p) / R) + 2e-3
