"""Tensor-level entry points of the CUDA kernels.

Each function checks devices, element types and strides, then calls one exported C
function of the kernel library on the current CUDA stream.  Nothing here computes on
the CPU or calls a library kernel: if the tensors are not on a GPU, or the library
cannot be built, the call raises.  Parts of the model call these through the module
(``ops.linear(...)``), which is also the seam a test uses to observe calls.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
PAGE = 64          # tokens per page of the key/value store (TLC_PAGE in tinyllama_c_b200.h)
# What the kernels are built for; a part checks its sizes against these when it is constructed, so that a
# configuration they do not cover is refused when the model is built, not at its first step.
MAX_HEAD_DIM = 256        # attention.cu: ATT_MAXD lanes-strided dims of a head (32 * 8)
MAX_STATE_SIZE = 256      # mamba.cu: state columns a warp keeps in registers (32 * 8)
MAX_CONV_TAPS = 17        # mamba.cu: CONV_MAX_TAPS + 1
MAX_HEADS = 65535         # a grid dimension
SSD_CHUNK = 128           # mamba_ssd.cu: rows of a chunk of the scan in matrix form

_vp, _i, _f, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
# Every function that csrc/tinyllama_c_b200.h declares: name -> (result, arguments).  A test parses the
# header and compares the kinds (pointer, int, float, long long), so that this table cannot drift from
# the definitions the compiler checked against the same header.
_SIGNATURES = {
    "tlc_last_error": (ctypes.c_char_p, []),
    "tlc_set_pdl": (None, [_i]),
    "tlc_linear_init": (_i, []),
    "tlc_attention_prefill_init": (_i, []),
    "tlc_ssd_init": (_i, []),
    "tlc_linear_error": (_i, []),
    "tlc_linear_error_clear": (None, []),
    "tlc_wait_limit_cycles": (_i, [_ll]),
    "tlc_selftest_bounded_wait": (_i, [_vp]),
    "tlc_embed": (_i, [_vp, _vp, _i, _i, _i, _i, _f, _vp, _vp]),
    "tlc_rmsnorm": (_i, [_vp, _vp, _vp, _f, _i, _i, _vp, _i, _vp]),
    "tlc_gated_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, _vp, _f, _i, _i, _i, _i, _vp, _i, _i, _f, _vp]),
    "tlc_swiglu": (_i, [_vp, _i, _i, _i, _i, _vp, _i, _i, _vp]),
    "tlc_gather_rows": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "tlc_linear": (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "tlc_linear_swiglu": (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "tlc_linear_simt": (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "tlc_linear_skinny_ok": (_i, [_i, _i, _vp, _i, _i, _vp, _i, _i]),
    "tlc_linear_skinny": (_i, [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "tlc_linear_skinny_swiglu": (_i, [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _vp]),
    "tlc_linear_tcgen05_ok": (_i, [_i, _i, _vp, _i, _i, _vp, _i]),
    "tlc_linear_tile_override": (None, [_i]),
    "tlc_linear_split_override": (None, [_i]),
    "tlc_linear_pair_override": (None, [_i]),
    "tlc_linear_skinny_pairs": (None, [_i]),
    "tlc_linear_tma_out": (None, [_i]),
    "tlc_linear_few_rows": (None, [_i]),
    "tlc_linear_few_rows_split": (None, [_i]),
    "tlc_linear_few_rows_min_tiles": (None, [_i]),
    "tlc_linear_few_rows_max_rows": (None, [_i]),
    "tlc_linear_few_rows_ok": (_i, [_i, _i, _vp, _i, _i, _vp, _i, _i, _i]),
    "tlc_linear_pairs": (_i, []),
    "tlc_rope_kv_store": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                               _i, _i, _vp]),
    "tlc_attention": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _vp]),
    "tlc_attention_decode": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i,
                                  _i, _vp]),
    "tlc_attention_decode_fused_ok": (_i, [_i, _i, _i]),
    "tlc_attention_decode_fused_passes": (_i, [_i]),
    "tlc_attention_decode_fused": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp,
                                        _vp, _i, _i, _i, _i, _f, _i, _i, _i, _vp]),
    "tlc_attention_prefill_ok": (_i, [_i, _i]),
    "tlc_attention_prefill_chunks": (_i, [_i, _i, _i, _vp]),
    "tlc_attention_prefill": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _vp,
                                   _vp, _i, _i, _vp]),
    "tlc_attention_prefill_tc_ok": (_i, [_i, _i, _i, _i]),
    "tlc_attention_prefill_tc": (_i, [_vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i,
                                      _i, _i, _i, _i, _vp, _vp, _vp]),
    "tlc_attention_prefill_tc_splits": (_i, [_i, _i, _i]),
    "tlc_mamba_conv": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i,
                            _i, _i, _i, _i, _i, _i, _vp]),
    "tlc_ssm_scan": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "tlc_ssm_scan_chunked": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i,
                                  _vp]),
    "tlc_ssd_ok": (_i, [_i, _i, _i, _i, _i]),
    "tlc_ssd_walk_override": (None, [_i]),
    "tlc_ssd_walk_blocks": (None, [_i]),
    "tlc_ssd_scratch_floats": (_ll, [_i, _i, _i, _i, _i, _i]),
    "tlc_ssm_scan_ssd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                              _i, _i, _vp, _vp]),
    "tlc_argmax": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "tlc_sample": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _i, _f, _f, _f, _i, _f, _f, _vp, _vp]),
    "tlc_attention_decode_no_alloc": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i,
                                           _vp]),
}
_lib = None


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """Loads (building first if needed) the kernel library and declares its functions."""
    global _lib
    if _lib is None:
        lib = _build.load()
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
        if torch.cuda.is_available():                                     # before any stream capture
            for init in (lib.tlc_linear_init, lib.tlc_attention_prefill_init, lib.tlc_ssd_init):
                if init() != 0:
                    raise KernelError(f"kernel library set-up: {lib.tlc_last_error().decode()}")
        # Programmatic dependent launch for every kernel of the library, captured or not: a kernel's blocks are
        # scheduled (and fetch what does not depend on its predecessor) while the predecessor's last blocks finish.
        lib.tlc_set_pdl(1 if USE_PDL else 0)
    return _lib


USE_PDL = bool(int(os.environ.get("TLC_PDL", "1")))
_launches = 0


def launch_count() -> int:
    """How many kernel-launching library calls were made (captured calls count once at capture;
    a graph replay adds its calls through count_launches)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += int(n)


def _call(name: str, *args) -> None:
    global _launches
    lib = library()
    _launches += 1
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(f"{name}: {lib.tlc_last_error().decode()}")


# The current stream's handle is asked for by every call; torch.cuda.current_stream() builds a Stream object each
# time (several microseconds: a prompt step makes hundreds of calls and is bound by the host up to about 2,000
# tokens), torch's own raw query does not.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _get_device is not None:
        return _raw_stream(_get_device())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {dt}; the kernels take float32 and bfloat16")


def _gpu(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("tinyllama.c_b200 kernels run on a CUDA device only (got a CPU tensor); "
                              "there is no CPU path")


def _gpu_required() -> None:
    if not torch.cuda.is_available():
        raise KernelError("tinyllama.c_b200 kernels need a CUDA device; there is no CPU path")


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are dense."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what}: expected a 2-D tensor with dense rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _out_rows(out: torch.Tensor, T: int, width: int, what: str) -> int:
    """Row stride of an output [T, width] whose rows are dense: the tensor itself, or a range of the
    columns of a wider buffer (several producers then fill one input of a following product)."""
    if tuple(out.shape) != (T, width):
        raise KernelError(f"{what}: output of shape {tuple(out.shape)}, expected {(T, width)}")
    return _rows(out, what + " output")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _f32vec(t: Optional[torch.Tensor], n: int, what: str) -> None:
    if t is None:
        return
    if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n:
        raise KernelError(f"{what}: expected {n} contiguous float32 values, got {tuple(t.shape)} {t.dtype}")


def _i32(t: torch.Tensor, what: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what}: expected a contiguous int32 tensor, got {t.dtype}")


# ---- elementwise ---------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    """out[t] = table[tokens[t]] * scale; out is float32 [T, D]."""
    _gpu(tokens, table, out)
    _i32(tokens, "embed tokens")
    T, (V, D) = tokens.numel(), table.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or tuple(out.shape) != (T, D) or not table.is_contiguous():
        raise KernelError("embed: out must be contiguous float32 [T, D] and the table contiguous")
    _call("tlc_embed", tokens.data_ptr(), table.data_ptr(), dtype_code(table.dtype), T, D, V, float(scale),
          out.data_ptr(), _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight; x float32 [*, D]."""
    _gpu(x, weight, out, rows)
    D = x.shape[1]
    R = out.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or out.shape[1] != D:
        raise KernelError("rmsnorm: x must be contiguous float32 and out contiguous [R, D]")
    _f32vec(weight, D, "rmsnorm weight")
    if rows is not None:
        _i32(rows, "rmsnorm rows")
        if rows.numel() != R:
            raise KernelError("rmsnorm: one row index per output row")
    elif x.shape[0] != R:
        raise KernelError("rmsnorm: x and out differ in rows")
    _call("tlc_rmsnorm", x.data_ptr(), _p(rows), weight.data_ptr(), float(eps), R, D, out.data_ptr(),
          dtype_code(out.dtype), _stream())


def gated_rmsnorm(y: torch.Tensor, z: torch.Tensor, weight: Optional[torch.Tensor], eps: float, n_groups: int,
                  norm_before_gate: bool, out: torch.Tensor, out_scale: float = 1.0,
                  y_add: Optional[torch.Tensor] = None) -> None:
    """Gate y by silu(z) and RMS-normalise per group (either order); weight None = gate only.  The
    result is multiplied by out_scale; out [T, Di] may be a range of the columns of a wider buffer.
    y_add: a second summand of the input (the scan of prompts leaves its outputs as two), same shape as y."""
    _gpu(y, z, weight, out, y_add)
    T, Di = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous():
        raise KernelError("gated_rmsnorm: y must be contiguous float32 [T, Di]")
    if y_add is not None and (y_add.dtype != torch.float32 or not y_add.is_contiguous() or y_add.shape != y.shape):
        raise KernelError("gated_rmsnorm: y_add must be contiguous float32 of y's shape")
    out_ld = _out_rows(out, T, Di, "gated_rmsnorm")
    if z.shape != y.shape:
        raise KernelError("gated_rmsnorm: gate and input differ in shape")
    _f32vec(weight, Di, "gated_rmsnorm weight")
    _call("tlc_gated_rmsnorm", y.data_ptr(), _p(y_add), z.data_ptr(), dtype_code(z.dtype), _rows(z, "gate"), _p(weight),
          float(eps), T, Di, int(n_groups), int(bool(norm_before_gate)), out.data_ptr(), dtype_code(out.dtype),
          out_ld, float(out_scale), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out = silu(gate) * up, where gate_up holds gate | up as two halves, or (interleaved) in
    groups of 16 columns: 8 gates followed by their 8 ups."""
    _gpu(gate_up, out)
    T, F2 = gate_up.shape
    F = F2 // 2
    if not out.is_contiguous() or tuple(out.shape) != (T, F) or F2 != 2 * F:
        raise KernelError("swiglu: out must be contiguous [T, F]")
    if interleaved and F % 8:
        raise KernelError("swiglu: the interleaved layout needs a multiple of 8 features")
    _call("tlc_swiglu", gate_up.data_ptr(), dtype_code(gate_up.dtype), _rows(gate_up, "gate_up"), F, T,
          out.data_ptr(), dtype_code(out.dtype), int(bool(interleaved)), _stream())


def gather_rows(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _gpu(x, rows, out)
    _i32(rows, "gather rows")
    if x.dtype != torch.float32 or out.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("gather_rows: float32 contiguous tensors")
    _call("tlc_gather_rows", x.data_ptr(), rows.data_ptr(), rows.numel(), x.shape[1], out.data_ptr(), _stream())


# ---- linear -----------------------------------------------------------------------------
# Fewest rows for which bfloat16 products may go to the tiled tcgen05 kernel; with fewer rows
# (and, up to 64 rows, for narrow outputs) the weight matrix is streamed once by the mma.sync
# kernel.  TLC_TENSOR_CORE_MIN_ROWS overrides it (a huge value keeps the tiled kernel out).
TENSOR_CORE_MIN_ROWS = int(os.environ.get("TLC_TENSOR_CORE_MIN_ROWS", "33"))


def linear_split_override(splits: int) -> None:
    """Fixes how many blocks share the K-steps of a tile of the tensor-core product (0: chosen from the
    sizes, 1: none); for tests."""
    library().tlc_linear_split_override(int(splits))


def linear_pair_override(mode: int) -> None:
    """Pairs of blocks on 256 x 256 tiles in the tensor-core product: 0 where they pay, 1 never, 2 wherever
    the GPU can run them; for tests."""
    library().tlc_linear_pair_override(int(mode))


def linear_few_rows(on: bool, split: int = 0) -> None:
    """Whether products of 17..64 rows take the tensor-core kernel that puts the weights on the 128-row side and
    shares a tile's K-steps among the blocks of a cluster; split fixes the number of blocks per tile (1, 2, 4, 8;
    0: chosen from the sizes).  For tests and comparisons."""
    library().tlc_linear_few_rows(int(bool(on)))
    library().tlc_linear_few_rows_split(int(split))


def linear_tma_out(on: bool) -> None:
    """Whether 32-bit outputs of the tensor-core product leave through the copy engine (bulk tensor stores, and
    adds made at the L2 for sums into the output); for tests and comparisons."""
    library().tlc_linear_tma_out(int(bool(on)))


def linear_skinny_pairs(on: bool) -> None:
    """Whether the few-row product may give a tile of 16 columns to two blocks of a cluster, each with one half
    of K (it does where the matrix has fewer tiles than the GPU has SMs); for tests and comparisons."""
    library().tlc_linear_skinny_pairs(int(bool(on)))


def linear_pairs() -> int:
    """How many pairs of blocks (clusters of two) of the tensor-core product the GPU runs at once."""
    return int(library().tlc_linear_pairs())


def linear_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, colscale: Optional[torch.Tensor] = None,
                  colbias: Optional[torch.Tensor] = None) -> None:
    """out[M, F] = silu(gate) * up with gate | up = (a w^T) * colscale + colbias, the 2F rows of w in
    groups of 16 (8 gate rows followed by their 8 up rows).  One kernel where the operands allow it
    (bfloat16, 16-byte aligned rows), else the product and the activation one after the other."""
    _gpu(a, w, out, colscale, colbias)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or N % 16 or tuple(out.shape) != (M, N // 2) or not out.is_contiguous():
        raise KernelError(f"linear_swiglu: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    _f32vec(colscale, N, "linear colscale")
    _f32vec(colbias, N, "linear colbias")
    global _launches
    lib = library()
    _launches += 1
    rc = lib.tlc_linear_swiglu(a.data_ptr(), dtype_code(a.dtype), _rows(a, "linear input"), w.data_ptr(), dtype_code(w.dtype),
                               _rows(w, "linear weight"), out.data_ptr(), dtype_code(out.dtype), N // 2, _p(colscale),
                               _p(colbias), M, N, K, TENSOR_CORE_MIN_ROWS, _stream())
    if rc == 1:                                   # no fused kernel for these operands
        _launches -= 1
        gu = torch.empty((M, N), dtype=torch.float32, device=a.device)
        linear(a, w, gu, colscale, colbias)
        swiglu(gu, out, interleaved=True)
    elif rc != 0:
        raise KernelError(f"tlc_linear_swiglu: {lib.tlc_last_error().decode()}")


def check_errors() -> None:
    """Raises if a tensor-core kernel gave up on a bounded wait (does not synchronise)."""
    code = library().tlc_linear_error()
    if code:
        library().tlc_linear_error_clear()
        raise KernelError(f"a kernel gave up on a bounded wait (code {code}: 1 loader, 2 issuer, 3 epilogue, 4 drain, "
                          f"5 accumulator of the tensor-core product; 9 the self-test); its output is incomplete")


def wait_limit_cycles(cycles: int) -> None:
    """How many clock cycles a bounded wait inside a kernel may spin before it gives up and reports
    (0: the default, about a second)."""
    lib = library()
    if lib.tlc_wait_limit_cycles(int(cycles)) != 0:
        raise KernelError(f"tlc_wait_limit_cycles: {lib.tlc_last_error().decode()}")


def selftest_bounded_wait() -> None:
    """Launches the error channel's self-test: a block waits on a barrier nobody arrives at, gives up at the
    limit and records code 9; check_errors() raises once the kernel has run."""
    _gpu_required()
    _call("tlc_selftest_bounded_wait", _stream())


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, colscale: Optional[torch.Tensor] = None,
           colbias: Optional[torch.Tensor] = None, accumulate: bool = False) -> None:
    """out[m, n] (+)= (sum_k a[m, k] w[n, k]) * colscale[n] + colbias[n].

    a [M, K] and out [M, N] may be row-strided views; w is [N, K].  Accumulation is
    32-bit.  float32 operands run on the CUDA cores in true 32-bit arithmetic."""
    _gpu(a, w, out, colscale, colbias)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"linear: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    _f32vec(colscale, N, "linear colscale")
    _f32vec(colbias, N, "linear colbias")
    _call("tlc_linear", a.data_ptr(), dtype_code(a.dtype), _rows(a, "linear input"), w.data_ptr(),
          dtype_code(w.dtype), _rows(w, "linear weight"), out.data_ptr(), dtype_code(out.dtype),
          _rows(out, "linear output"), _p(colscale), _p(colbias), int(bool(accumulate)), M, N, K,
          TENSOR_CORE_MIN_ROWS, _stream())


# ---- attention -------------------------------------------------------------------------------
DISABLE_TILED_ATTENTION = bool(int(os.environ.get("TLC_DISABLE_TILED_ATTENTION", "0")))
# Prompt attention on tcgen05 (0) or the mma.sync kernel everywhere (1); TLC_PROMPT_ATTENTION sets the start value,
# prompt_attention_override() changes it (tests run both).
_prompt_attention = int(os.environ.get("TLC_PROMPT_ATTENTION", "0"))


def prompt_attention_override(mode: int) -> None:
    """0: prompts of a bfloat16 cache with heads of 64 or 128 take the tcgen05 attention kernel; 1: the mma.sync one."""
    global _prompt_attention
    _prompt_attention = int(mode)


def rope_kv_store(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor, k_pages: torch.Tensor,
                  v_pages: torch.Tensor, inv_freq: torch.Tensor, positions: torch.Tensor, row_seq: torch.Tensor,
                  slots: torch.Tensor, block_table: torch.Tensor, H: int, KV: int, hd: int,
                  write_kv: bool = True) -> None:
    """Rotates q and k at their absolute positions; writes q to q_out [T, H*hd] and k, v into
    the pages of their sequences ([page, KV, 64, hd])."""
    _gpu(qkv, q_out, k_pages, v_pages, inv_freq, positions, row_seq, slots, block_table)
    T = qkv.shape[0]
    for t, n in ((positions, "positions"), (row_seq, "row_seq"), (slots, "slots"), (block_table, "block_table")):
        _i32(t, n)
    if k_pages.dtype != q_out.dtype or v_pages.dtype != q_out.dtype:
        raise KernelError("rope_kv_store: q and the pages must share one element type")
    if not q_out.is_contiguous() or tuple(q_out.shape) != (T, H * hd) or not k_pages.is_contiguous() \
            or not v_pages.is_contiguous() or tuple(k_pages.shape[1:]) != (KV, PAGE, hd):
        raise KernelError("rope_kv_store: q_out must be contiguous [T, H*hd], pages contiguous [n, KV, 64, hd]")
    _f32vec(inv_freq, inv_freq.numel(), "rope inv_freq")
    _call("tlc_rope_kv_store", qkv.data_ptr(), dtype_code(qkv.dtype), dtype_code(q_out.dtype), _rows(qkv, "qkv"),
          q_off, k_off, v_off,
          q_out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), inv_freq.data_ptr(), 2 * inv_freq.numel(),
          positions.data_ptr(), row_seq.data_ptr(), slots.data_ptr(), block_table.data_ptr(), block_table.shape[1],
          T, H, KV, hd, int(bool(write_kv)), _stream())


def attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
              positions: torch.Tensor, row_seq: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, H: int, KV: int,
              hd: int, scale: float, window: int = 0, decode_max_keys: int = 0,
              cu_seqlens: Optional[torch.Tensor] = None, start_pos: Optional[torch.Tensor] = None,
              max_keys: int = 0, max_blocks: int = 0, key_ranges: int = 0) -> None:
    """Causal grouped-query attention of every row over its sequence's pages (keys 0..position,
    or the last `window` of them).  decode_max_keys > 0 says that the rows are single-token
    steps of sequences no longer than that: keys are then split across blocks.  With
    cu_seqlens and start_pos (rows of a sequence are consecutive positions from start_pos) the
    tiled tensor-core kernel serves bfloat16 heads of 64 or 128; with max_keys (the longest sequence
    after this step) it cuts the key range of long rows into pieces that run side by side.  max_blocks > 0
    bounds how many blocks (hence SMs) the tensor-core kernel of prompts holds at a time, for a caller that runs
    other kernels beside it; the result does not depend on it.  key_ranges > 0 fixes into how many ranges that
    kernel cuts the keys of a row tile (0: chosen: more than one for few rows over many keys)."""
    _gpu(q, k_pages, v_pages, block_table, positions, row_seq, slots, out)
    T = q.shape[0]
    if not q.is_contiguous() or tuple(q.shape) != (T, H * hd) or out.dtype != q.dtype or k_pages.dtype != q.dtype:
        raise KernelError("attention: q must be contiguous [T, H*hd], q and out of the pages' type")
    out_ld = _out_rows(out, T, H * hd, "attention")
    if decode_max_keys > 0 and H // KV <= 8:
        n_splits = (int(decode_max_keys) + 127) // 128
        part_o = torch.empty((T, H, n_splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T, H, n_splits, 2), dtype=torch.float32, device=q.device)
        _call("tlc_attention_decode", q.data_ptr(), dtype_code(q.dtype), k_pages.data_ptr(), v_pages.data_ptr(),
              block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), row_seq.data_ptr(),
              slots.data_ptr(), out.data_ptr(), part_o.data_ptr(), part_ml.data_ptr(), T, H, KV, hd, float(scale),
              int(window or 0), int(decode_max_keys), out_ld, _stream())
        return
    tiled = decode_max_keys <= 0 and cu_seqlens is not None and start_pos is not None and q.dtype == torch.bfloat16 \
        and hd in (64, 128) and not DISABLE_TILED_ATTENTION
    if tiled and _prompt_attention == 0 and max_keys > 0 and out_ld % 8 == 0 \
            and library().tlc_attention_prefill_tc_ok(BF16, hd, H, KV):
        B = slots.numel()
        # few row tiles and many keys (a piece of a long prompt): the keys in ranges that run side by side
        n_split = key_ranges if key_ranges > 0 else library().tlc_attention_prefill_tc_splits(T // 128 + B, H, int(max_keys))
        part_o = part_ml = None
        if n_split > 1:
            part_o = torch.empty((T, H, n_split, hd), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((T, H, n_split, 2), dtype=torch.float32, device=q.device)
        _call("tlc_attention_prefill_tc", q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
              block_table.data_ptr(), block_table.shape[1], cu_seqlens.data_ptr(), slots.data_ptr(), start_pos.data_ptr(),
              out.data_ptr(), B, T // 128 + B, H, KV, hd, float(scale), int(window or 0), int(max_keys), T,
              out_ld, int(max_blocks), int(n_split), _p(part_o), _p(part_ml), _stream())
        return
    if tiled:
        B = slots.numel()
        n_tiles = T // 64 + B
        chunk = ctypes.c_int(0)
        n_chunks = library().tlc_attention_prefill_chunks(n_tiles, H, (int(max_keys) + 63) // 64, ctypes.byref(chunk)) \
            if max_keys > 0 else 1
        part_o = part_ml = None
        if n_chunks > 1:
            part_o = torch.empty((T, H, n_chunks, hd), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((T, H, n_chunks, 2), dtype=torch.float32, device=q.device)
        _call("tlc_attention_prefill", q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], cu_seqlens.data_ptr(), slots.data_ptr(), start_pos.data_ptr(), out.data_ptr(), B,
              n_tiles, H, KV, hd, float(scale), int(window or 0), (int(max_keys) + 63) // 64 if n_chunks > 1 else 0,
              row_seq.data_ptr(), _p(part_o), _p(part_ml), T, out_ld, _stream())
        return
    _call("tlc_attention", q.data_ptr(), dtype_code(q.dtype), k_pages.data_ptr(), v_pages.data_ptr(),
          block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), row_seq.data_ptr(), slots.data_ptr(),
          out.data_ptr(), T, H, KV, hd, float(scale), int(window or 0), out_ld, _stream())


DISABLE_FUSED_DECODE_ATTENTION = bool(int(os.environ.get("TLC_DISABLE_FUSED_DECODE_ATTENTION", "0")))
FUSED_DECODE_COUNTERS = 65536      # arrival counters a caller of attention_decode_fused provides (rows x kv heads at most)


def new_arrival_counters(device) -> torch.Tensor:
    """Zeroed arrival counters for attention_decode_fused.  They belong to whoever launches the kernel (an
    attention mixer keeps its own): launches that share counters must not overlap on the GPU; every launch
    leaves them at zero.  Allocate them outside any stream capture."""
    return torch.zeros(FUSED_DECODE_COUNTERS, dtype=torch.int32, device=device)


def attention_decode_fused_ok(qkv: torch.Tensor, cache_dtype: torch.dtype, H: int, KV: int, hd: int) -> bool:
    """Whether attention_decode_fused takes this projection, cache type and these sizes."""
    return bool(qkv.is_cuda and qkv.dtype == torch.float32 and cache_dtype == torch.bfloat16
                and qkv.shape[0] * KV <= FUSED_DECODE_COUNTERS
                and not DISABLE_FUSED_DECODE_ATTENTION and library().tlc_attention_decode_fused_ok(H, KV, hd))


def attention_decode_fused(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, k_pages: torch.Tensor,
                           v_pages: torch.Tensor, inv_freq: torch.Tensor, write_kv: bool, block_table: torch.Tensor,
                           positions: torch.Tensor, row_seq: torch.Tensor, slots: torch.Tensor, out: torch.Tensor,
                           H: int, KV: int, hd: int, scale: float, window: int, max_keys: int,
                           arrivals: torch.Tensor) -> None:
    """Single-token steps in one kernel: rotates the row's queries and new key (2 * len(inv_freq)
    leading dims of each head), stores the new key/value row into its page when write_kv, attends
    over the sequence's pages and writes out [T, H*hd] bfloat16.  qkv is float32 with dense rows.
    arrivals: the caller's counters (new_arrival_counters)."""
    _gpu(qkv, k_pages, v_pages, inv_freq, block_table, positions, row_seq, slots, out)
    T = qkv.shape[0]
    for t, n in ((positions, "positions"), (row_seq, "row_seq"), (slots, "slots"), (block_table, "block_table")):
        _i32(t, n)
    if qkv.dtype != torch.float32 or k_pages.dtype != torch.bfloat16 or v_pages.dtype != torch.bfloat16 \
            or out.dtype != torch.bfloat16:
        raise KernelError("attention_decode_fused: float32 projections, bfloat16 pages and output")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[1:]) != (KV, PAGE, hd) \
            or v_pages.shape != k_pages.shape:
        raise KernelError("attention_decode_fused: pages must be contiguous [n, KV, 64, hd]")
    out_ld = _out_rows(out, T, H * hd, "attention_decode_fused")
    ld = _rows(qkv, "qkv")
    if max(q_off + H * hd, k_off + KV * hd, v_off + KV * hd) > max(ld, qkv.shape[1]):
        raise KernelError("attention_decode_fused: q, k or v lies outside the projection's row")
    _f32vec(inv_freq, inv_freq.numel(), "rope inv_freq")
    n_splits = (int(max_keys) + 127) // 128
    part_o = torch.empty((T, H, n_splits, hd), dtype=torch.float32, device=qkv.device)
    part_ml = torch.empty((T, H, n_splits, 2), dtype=torch.float32, device=qkv.device)
    _gpu(arrivals)
    _i32(arrivals, "arrival counters")
    if arrivals.numel() < T * KV:
        raise KernelError(f"attention_decode_fused: {T * KV} (row, kv head) pairs need as many arrival counters, "
                          f"{arrivals.numel()} given")
    _call("tlc_attention_decode_fused", qkv.data_ptr(), ld, q_off, k_off, v_off, k_pages.data_ptr(), v_pages.data_ptr(),
          inv_freq.data_ptr(), 2 * inv_freq.numel(), int(bool(write_kv)), block_table.data_ptr(), block_table.shape[1],
          positions.data_ptr(), row_seq.data_ptr(), slots.data_ptr(), out.data_ptr(), part_o.data_ptr(),
          part_ml.data_ptr(), arrivals.data_ptr(), T, H, KV, hd, float(scale), int(window or 0), int(max_keys), out_ld, _stream())


def attention_decode_fused_passes(passes: int) -> None:
    """Fixes how many rounds of chunks a block of the fused single-token attention takes one after the
    other (0: chosen from the grid); for tests of the running statistics."""
    library().tlc_attention_decode_fused_passes(int(passes))


DISABLE_SSD = bool(int(os.environ.get("TLC_DISABLE_SSD", "0")))


# ---- Mamba2 -------------------------------------------------------------------------------------
def mamba_conv(proj: torch.Tensor, xbc_off: int, dt_off: int, w: torch.Tensor, bias: Optional[torch.Tensor],
               dt_bias: torch.Tensor, A: torch.Tensor, conv_state: torch.Tensor, cu_seqlens: torch.Tensor,
               row_seq: torch.Tensor, slots: torch.Tensor, start_pos: torch.Tensor, xbc_out: torch.Tensor,
               dt_out: torch.Tensor, dA_out: torch.Tensor, single_rows: bool = False, bf16_run: bool = False,
               all_fresh: bool = False) -> None:
    """Causal depthwise convolution + SiLU of the xBC columns of proj, continuing each
    sequence's window (conv_state [n_slots, K-1, Cd], updated in place); also
    dt = softplus(dt + dt_bias) and dA = exp(dt * A) per row and head.  single_rows says
    that every sequence brings exactly one row (row b belongs to sequence b); bf16_run says that the
    model computes in bfloat16: x|B|C, operands of the scan's matrix products, are then rounded to
    bfloat16 values whatever type they are stored in, and the SiLU of prompts takes the fast exponential
    and reciprocal.  xbc_out is float32, or
    bfloat16 where the scan that follows takes its operands in that type (ssm_scan with A).  all_fresh says that
    every sequence of the step starts at position 0 (the caller knows the start positions on the host): no stored
    window is read then, and the convolution's own kernel leaves the new windows (one launch less)."""
    _gpu(proj, w, bias, dt_bias, A, conv_state, cu_seqlens, row_seq, slots, start_pos, xbc_out, dt_out, dA_out)
    T = proj.shape[0]
    Cd, K = w.shape
    Hs = dt_bias.numel()
    B = slots.numel()
    _f32vec(w, Cd * K, "conv weight")
    _f32vec(bias, Cd, "conv bias")
    _f32vec(dt_bias, Hs, "dt_bias")
    _f32vec(A, Hs, "A")
    for t, n in ((cu_seqlens, "cu_seqlens"), (row_seq, "row_seq"), (slots, "slots"), (start_pos, "start_pos")):
        _i32(t, n)
    if conv_state.dtype != torch.float32 or not conv_state.is_contiguous() or tuple(conv_state.shape[1:]) != (K - 1, Cd):
        raise KernelError("mamba_conv: conv_state must be contiguous float32 [n_slots, K-1, Cd]")
    for t, shp, n in ((dt_out, (T, Hs), "dt_out"), (dA_out, (T, Hs), "dA_out")):
        if t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != shp:
            raise KernelError(f"mamba_conv: {n} must be contiguous float32 {shp}")
    if not xbc_out.is_contiguous() or tuple(xbc_out.shape) != (T, Cd):
        raise KernelError(f"mamba_conv: xbc_out must be contiguous {(T, Cd)}")
    _call("tlc_mamba_conv", proj.data_ptr(), dtype_code(proj.dtype), _rows(proj, "proj"), xbc_off, dt_off,
          w.data_ptr(), _p(bias), dt_bias.data_ptr(), A.data_ptr(), conv_state.data_ptr(), cu_seqlens.data_ptr(),
          row_seq.data_ptr(), slots.data_ptr(), start_pos.data_ptr(), xbc_out.data_ptr(), dtype_code(xbc_out.dtype),
          dt_out.data_ptr(), dA_out.data_ptr(), T, B, Cd, K, Hs, int(bool(single_rows)), int(bool(bf16_run)),
          int(bool(all_fresh)), _stream())


def ssd_walk_blocks(blocks: int) -> None:
    """How many blocks of the tcgen05 walk work through the (sequence, head, rows) items (0: one an SM at most);
    for tests: with few blocks each walks many sequences in turn."""
    library().tlc_ssd_walk_blocks(int(blocks))


def ssd_walk_override(mode: int) -> None:
    """Which kernel walks a sequence's chunks where both are built (0: tcgen05 with the state in tensor memory for
    states of 128 or 256 columns; 1: always mma.sync with the state in registers); for tests."""
    library().tlc_ssd_walk_override(int(mode))


def ssd_ok(Hs: int, P: int, N: int, G: int) -> bool:
    """Whether the scan of prompts in matrix form (bfloat16 operands, ssm_scan with A) is built for these sizes."""
    return bool(not DISABLE_SSD and library().tlc_ssd_ok(Hs, P, N, G, Hs * P + 2 * G * N))


_aux_streams: dict = {}


def _aux_stream(device) -> "torch.cuda.Stream":
    """A second stream per device and current stream, for work that runs beside a kernel chain of the current one."""
    key = (torch.device(device).index, _stream())        # (the raw handle: torch.cuda.current_stream() costs 10 us)
    if key not in _aux_streams:
        if len(_aux_streams) > 64:
            _aux_streams.clear()
        _aux_streams[key] = torch.cuda.Stream(device=device)
    return _aux_streams[key]


def ssm_scan(xbc: torch.Tensor, dt: torch.Tensor, dA: torch.Tensor, Dskip: torch.Tensor, state: torch.Tensor,
             cu_seqlens: torch.Tensor, slots: torch.Tensor, start_pos: torch.Tensor, y: torch.Tensor, Hs: int, P: int,
             N: int, G: int, chunks=None, A: Optional[torch.Tensor] = None, y_part: Optional[torch.Tensor] = None) -> bool:
    """Selective scan of every sequence in order, from its slot's state (zero at position 0);
    state [n_slots, Hs, P, N] float32 is updated in place; y [T, Hs*P] float32 is before gating.
    chunks = (seg_start [n+1], seg_seq [n], seq_seg_start [B+1]) cuts the sequences into
    chunks that run in parallel (same result up to rounding).  With a bfloat16 xbc and A (the per-head
    decay rate, dA = exp(dt * A)) the chunks, of at most 128 rows, run in matrix form on the tensor cores
    with bfloat16 operands (see ssd_ok for the sizes); every 32-bit run passes a float32 xbc.
    y_part (float32, y's shape; matrix form only): the outputs may then come as two summands, what needs no state in
    y_part (computed on a second stream beside the walk over the chunks) and the state's share in y; returns True
    if they did (the caller adds them), False if y holds the outputs."""
    _gpu(xbc, dt, dA, Dskip, state, cu_seqlens, slots, start_pos, y, y_part)
    T, Cd = xbc.shape
    if Cd != Hs * P + 2 * G * N:
        raise KernelError("ssm_scan: xbc width does not match Hs*P + 2*G*N")
    matrix_form = xbc.dtype == torch.bfloat16
    for t, shp, n in ((xbc, (T, Cd), "xbc"), (dt, (T, Hs), "dt"), (dA, (T, Hs), "dA"), (y, (T, Hs * P), "y")):
        want = torch.bfloat16 if (n == "xbc" and matrix_form) else torch.float32
        if t.dtype != want or not t.is_contiguous() or tuple(t.shape) != shp:
            raise KernelError(f"ssm_scan: {n} must be contiguous {want} {shp}")
    _f32vec(Dskip, Hs, "D")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (Hs, P, N):
        raise KernelError("ssm_scan: state must be contiguous float32 [n_slots, Hs, P, N]")
    if matrix_form and (chunks is None or A is None or not ssd_ok(Hs, P, N, G)):
        raise KernelError("ssm_scan: a bfloat16 x|B|C is for the chunked scan in matrix form (chunks, A, sizes of ssd_ok)")
    if chunks is not None:
        seg_start, seg_seq, seq_seg_start = chunks
        for t, n in ((seg_start, "seg_start"), (seg_seq, "seg_seq"), (seq_seg_start, "seq_seg_start")):
            _gpu(t)
            _i32(t, n)
        n_seg = seg_seq.numel()
        lib = library()
        if matrix_form:
            _f32vec(A, Hs, "A")
            scratch = torch.empty(lib.tlc_ssd_scratch_floats(n_seg, T, Hs, P, N, G), dtype=torch.float32, device=xbc.device)
            if y_part is not None and (y_part.dtype != torch.float32 or not y_part.is_contiguous() or y_part.shape != y.shape):
                raise KernelError("ssm_scan: y_part must be contiguous float32 of y's shape")
            used = ctypes.c_int(0)
            aux = _aux_stream(xbc.device).cuda_stream if y_part is not None and not torch.cuda.is_current_stream_capturing() else None
            _call("tlc_ssm_scan_ssd", xbc.data_ptr(), dt.data_ptr(), A.data_ptr(), Dskip.data_ptr(), state.data_ptr(),
                  scratch.data_ptr(), seg_start.data_ptr(), seg_seq.data_ptr(), seq_seg_start.data_ptr(),
                  slots.data_ptr(), start_pos.data_ptr(), y.data_ptr(), _p(y_part), ctypes.byref(used), slots.numel(), n_seg,
                  T, Hs, P, N, G, Cd, _stream(), aux)
            return bool(used.value)
        scratch = torch.empty(n_seg * Hs * (P * N + 1), dtype=torch.float32, device=xbc.device)
        _call("tlc_ssm_scan_chunked", xbc.data_ptr(), dt.data_ptr(), dA.data_ptr(), Dskip.data_ptr(), state.data_ptr(),
              scratch.data_ptr(), seg_start.data_ptr(), seg_seq.data_ptr(), seq_seg_start.data_ptr(), slots.data_ptr(),
              start_pos.data_ptr(), y.data_ptr(), slots.numel(), n_seg, Hs, P, N, G, Cd, _stream())
        return False
    _call("tlc_ssm_scan", xbc.data_ptr(), dt.data_ptr(), dA.data_ptr(), Dskip.data_ptr(), state.data_ptr(),
          cu_seqlens.data_ptr(), slots.data_ptr(), start_pos.data_ptr(), y.data_ptr(), slots.numel(), Hs, P, N, G, Cd,
          _stream())
    return False


# ---- sampling -------------------------------------------------------------------------------------
def new_argmax_work(rows: int, device) -> torch.Tensor:
    """Zeroed workspace for argmax over `rows` rows (every launch leaves it zero); its owner's launches must not
    overlap on the GPU.  Allocate it outside any stream capture."""
    return torch.zeros(2 * max(1, int(rows)), dtype=torch.int64, device=device)


def argmax(logits: torch.Tensor, out: torch.Tensor, work: Optional[torch.Tensor] = None) -> None:
    """out[r] = first index of the maximum of logits[r].  With `work` (new_argmax_work) a row is spread over
    many blocks; without, one block takes a row."""
    _gpu(logits, out, work)
    _i32(out, "argmax out")
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("argmax: logits must be contiguous float32")
    if work is not None and (work.dtype != torch.int64 or not work.is_contiguous() or work.numel() < 2 * logits.shape[0]):
        raise KernelError("argmax: work must be a contiguous int64 tensor of at least 2 values per row")
    _call("tlc_argmax", logits.data_ptr(), logits.shape[0], logits.shape[1], out.data_ptr(), _p(work), _stream())


def sample(logits: torch.Tensor, work: torch.Tensor, history: Optional[torch.Tensor], uniforms: torch.Tensor,
           temperature: float, top_k: int, top_p: float, min_p: float, repeat_penalty: float,
           frequency_penalty: float, presence_penalty: float, out: torch.Tensor) -> None:
    """One token per row from penalised, temperature-scaled, top-k / min-p / top-p filtered
    logits; `history` [R, n] int32 (-1 = empty) is the penalty window, `uniforms` [R] the draws,
    `work` a [R, V] float32 scratch."""
    _gpu(logits, work, history, uniforms, out)
    R, V = logits.shape
    _i32(out, "sample out")
    if logits.dtype != torch.float32 or not logits.is_contiguous() or work.dtype != torch.float32 \
            or not work.is_contiguous() or work.numel() < R * V:
        raise KernelError("sample: logits and work must be contiguous float32 [R, V]")
    _f32vec(uniforms, R, "sample uniforms")
    n_hist = 0
    if history is not None:
        _i32(history, "sample history")
        n_hist = history.shape[1]
    _call("tlc_sample", logits.data_ptr(), work.data_ptr(), _p(history), uniforms.data_ptr(), R, V,
          float(temperature), int(top_k), float(top_p), float(min_p), float(repeat_penalty), n_hist,
          float(frequency_penalty), float(presence_penalty), out.data_ptr(), _stream())
