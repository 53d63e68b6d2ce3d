"""Python face of the CUDA kernels: thin, checked wrappers over the ``extern "C"`` launchers.

Every function here launches hand-written sm_100a kernels on torch's current CUDA stream.
There is no CPU path and no library stand-in: a tensor that is not on a CUDA device, or a
missing extension, raises.  The only library product on the engine's path is the bfloat16
matrix product (cuBLAS through ``torch.mm``), where the reference's engine also calls a
library (rollout/monkey_patch/qwen3.py:21-22,29-31,56).
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"the kernels take float32 and bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("the engine's kernels run on a CUDA device only; got a CPU tensor")
    return t.data_ptr()              # an int: ctypes makes the pointer from it (argtypes are set)


try:                                                  # the raw handle, without building a Stream object
    _raw_stream, _device_index = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:                                # a torch without these: the public way, slower
    _raw_stream = None


def _stream():
    """The current stream of the current device (each launch asks: a graph capture changes it)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(_device_index()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


# kernels of this package launched by this process (a captured graph counts once, at capture)
launch_count = 0


def _check(code: int, what: str, kernels: int = 1) -> None:
    global launch_count
    launch_count += kernels
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")


# How kernels of a step overlap through programmatic dependent launch (csrc/common.cuh): every kernel waits for
# its predecessor before it touches what that wrote, and lets its successor start when its main loop is done.
PDL_MODE = 2

_core = None

_CORE_SOURCES = ["elementwise.cu", "gemm_f32.cu", "gemm_skinny.cu", "rope_cache.cu", "attention_simt.cu", "sampling.cu"]


def core() -> ctypes.CDLL:
    """The library of kernels that need no specialisation."""
    global _core
    if _core is None:
        lib = build.load("return_core", _CORE_SOURCES, {"RB_PDL_MODE": PDL_MODE})
        P, I, F = c_void_p, c_int, c_float
        lib.rb_embedding.argtypes = [P, I, P, P, I, I, I, P]
        lib.rb_add_rmsnorm.argtypes = [P, P, P, P, I, F, F, P, I, I, I, P]
        lib.rb_rmsnorm_rows.argtypes = [P, P, I, F, F, P, I, I, I, P]
        lib.rb_swiglu.argtypes = [P, P, I, I, I, I, P]
        lib.rb_gemm_f32.argtypes = [P, P, P, I, I, I, I, I, I, P]
        lib.rb_gemm_skinny.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P]
        lib.rb_gemm_skinny.restype = c_int
        lib.rb_gemm_skinny_fused.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P, I, I, F, P, P, I, F, P, I, P]
        lib.rb_gemm_skinny_fused.restype = c_int
        lib.rb_gemm_skinny_ctas.argtypes = [I]
        lib.rb_gemm_skinny_ctas.restype = c_int
        lib.rb_qk_norm_rope_write.argtypes = [P, I, P, P, I, F, F, P, P, I, P, P, P, I, I, P, P, I, I, I, I, I, I, P]
        lib.rb_attention_simt.argtypes = [P, I, P, P, P, P, P, I, I, P, I, I, I, I, I, F, I, P]
        lib.rb_sample.argtypes = [P, I, I, I, P, P, P, P, P, P, I, P]
        lib.rb_argmax.argtypes = [P, I, I, I, P, P]
        for name in ("rb_embedding", "rb_add_rmsnorm", "rb_rmsnorm_rows", "rb_swiglu", "rb_gemm_f32",
                     "rb_qk_norm_rope_write", "rb_attention_simt", "rb_sample", "rb_argmax"):
            getattr(lib, name).restype = c_int
        _core = lib
    return _core


# head sizes compiled ahead of time by build_all(); any other multiple of 16 compiles on first use
PREBUILT_HEAD_DIMS = (16, 32, 48, 64, 128)


def build_all():
    """Compiles every library of the package (nvcc cross-compiles, no GPU needed); returns the paths."""
    paths = [build.library_path("return_core", _CORE_SOURCES, {"RB_PDL_MODE": PDL_MODE})]
    paths.append(build.library_path("return_tc5", _TC5_SOURCES, _tc5_defines()))
    for d in TC5_ATTENTION_HEAD_DIMS:
        paths.append(build.library_path(f"return_attn_tc5_d{d}", ["attention_tc5.cu"], _attn_tc5_defines(d)))
    for d in PREBUILT_HEAD_DIMS:
        paths.append(build.library_path(f"return_attn_d{d}", ["attention_mma.cu"], _attn_defines(d)))
    return paths


# ------------------------------------------------------------------------------- elementwise

def embedding(table: torch.Tensor, tokens: torch.Tensor, stream_out: torch.Tensor) -> None:
    """stream_out[t] = float32(table[tokens[t]]); tokens int32 [T], stream_out float32 [T, H]."""
    T, H = stream_out.shape
    assert tokens.dtype == torch.int32 and stream_out.dtype == torch.float32
    assert table.shape[1] == H and table.is_contiguous() and stream_out.is_contiguous()
    _check(core().rb_embedding(_ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(stream_out),
                               T, H, table.shape[0], _stream()), "embedding")


def add_rmsnorm(stream: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, offset: float = 0.0) -> None:
    """stream += delta (written back unless ``rows``); out = rmsnorm(stream) * (offset + weight).

    ``rows`` (int32) picks the rows to normalise; out then has one row per entry of ``rows``.
    """
    H = stream.shape[1]
    n = out.shape[0]
    assert stream.dtype == torch.float32 and stream.is_contiguous() and out.is_contiguous()
    assert out.shape[1] == H and weight.numel() == H
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape == stream.shape and delta.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n
    else:
        assert n == stream.shape[0]
    _check(core().rb_add_rmsnorm(_ptr(stream), _ptr(delta), _ptr(rows), _ptr(weight), dtype_code(weight.dtype),
                                 eps, offset, _ptr(out), dtype_code(out.dtype), n, H, _stream()), "add_rmsnorm")


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, offset: float = 0.0) -> None:
    """out = rmsnorm over the last dim of contiguous x [..., N]."""
    N = x.shape[-1]
    assert x.is_contiguous() and out.is_contiguous() and out.dtype == x.dtype and weight.numel() == N
    _check(core().rb_rmsnorm_rows(_ptr(x), _ptr(weight), dtype_code(weight.dtype), eps, offset, _ptr(out),
                                  dtype_code(x.dtype), x.numel() // N, N, _stream()), "rmsnorm_rows")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> None:
    """out = silu(gate) * up.  ``interleave`` 0: gate_up[t] = [gate | up]; 8: blocks of 8 gate then 8 up."""
    T, I2 = gate_up.shape
    assert out.shape == (T, I2 // 2) and gate_up.is_contiguous() and out.is_contiguous()
    assert out.dtype == gate_up.dtype and interleave in (0, 8)
    _check(core().rb_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), T, I2 // 2, interleave, _stream()), "swiglu")


# ------------------------------------------------------------------------------- matrix products

def gemm_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T in true float32 (FFMA, fixed order over K)."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == out.dtype == torch.float32
    assert w.shape[1] == K and out.shape == (M, N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(core().rb_gemm_f32(_ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                              _stream()), "gemm_f32")


SKINNY_KERNEL_MAX_ROWS = 32     # what the kernel takes
SKINNY_MAX_ROWS = 8             # what the engine gives it: beyond 8 rows the library is faster (38 us against 58 at
                                # 16 rows and 106 at 32, for N = 24576, K = 4096)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 32 in bfloat16: the weight-streaming kernel of decode steps
    (the engine uses it up to 8 rows).
    ``gated``: w holds gate and up rows interleaved in blocks of 8; out[M, N/2] = silu(gate) * up."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    assert w.shape[1] == K and out.shape == (M, N // 2 if gated else N) and M <= SKINNY_KERNEL_MAX_ROWS
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(core().rb_gemm_skinny(_ptr(x), _ptr(w), _ptr(out), 1 if out.dtype == torch.float32 else 0,
                                 1 if gated else 0, M, N, K, x.stride(0), w.stride(0), out.stride(0), _stream()),
           "gemm_skinny")


class RowSums:
    """Where a product in its residual form leaves each CTA's share of sum(v^2) per token, for the norm that follows:
    the product that takes the normed rows multiplies its result by rstd = 1 / sqrt(sum / dim + eps) instead of
    anyone norming them.  ``parts``: float32 [8, width]; ``count``: the shares that were written; ``dim``: the length
    of the normed row."""
    WIDTH = 512

    def __init__(self, parts: torch.Tensor, dim: int, count: int = 0):
        self.parts, self.dim, self.count = parts, dim, count


def gemm_skinny_fused(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], gated: bool = False, scale=None,
                      residual=None) -> None:
    """The weight-streaming product for up to 8 rows with the norm and the residual add around it folded in.

    ``scale`` = (RowSums, eps): the accumulators are multiplied by each token's rstd, the factor that the norm
    before this product would have applied (its input rows are v * (offset + weight), not normed).
    ``residual`` = (stream, next_norm, sums): v = stream + acc goes to ``stream`` (float32 [M, N]); with
    ``next_norm`` = (weight, offset), ``out`` [M, N] gets v * (offset + weight) for the next product; ``sums``
    (a RowSums, or None) gets the shares of sum(v^2)."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and M <= 8 and w.shape[1] == K
    assert x.stride(1) == 1 and w.stride(1) == 1
    lib = core()
    ssq_in, ssq_in_count, norm_dim, eps = None, 0, 0, 0.0
    if scale is not None:
        sums_in, eps = scale
        assert sums_in.count > 0 and sums_in.parts.dtype == torch.float32 and sums_in.parts.is_contiguous()
        ssq_in, ssq_in_count, norm_dim = sums_in.parts, sums_in.count, sums_in.dim
    stream = norm_w = ssq_out = None
    norm_w_dtype, offset = F32, 0.0
    if residual is not None:
        stream, next_norm, sums_out = residual
        assert not gated and stream.dtype == torch.float32 and stream.is_contiguous() and stream.shape == (M, N)
        if next_norm is not None:
            norm_w, offset = next_norm
            assert out is not None and norm_w.numel() == N
            norm_w_dtype = dtype_code(norm_w.dtype)
        if sums_out is not None:
            assert sums_out.parts.dtype == torch.float32 and sums_out.parts.is_contiguous() and sums_out.dim == N
            sums_out.count = lib.rb_gemm_skinny_ctas(N)
            assert sums_out.count <= sums_out.parts.shape[1]
            ssq_out = sums_out.parts
    if out is not None:
        assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.shape == (M, N // 2 if gated else N)
    ld_sums = (ssq_in if ssq_in is not None else ssq_out).shape[1] if (ssq_in is not None or ssq_out is not None) else 0
    if ssq_in is not None and ssq_out is not None:
        assert ssq_in.shape[1] == ssq_out.shape[1]
    _check(lib.rb_gemm_skinny_fused(_ptr(x), _ptr(w), _ptr(out), 1 if residual is not None else 0, 1 if gated else 0,
                                    M, N, K, x.stride(0), w.stride(0), out.stride(0) if out is not None else 0,
                                    _ptr(ssq_in), ssq_in_count, norm_dim, eps, _ptr(stream), _ptr(norm_w), norm_w_dtype,
                                    offset, _ptr(ssq_out), ld_sums, _stream()), "gemm_skinny_fused")


def skinny_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes this product (few rows, 16-byte aligned rows)."""
    return (x.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_MAX_ROWS and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


# From this many rows on, the gated product of a feed-forward runs as 256 x 256 tiles by pairs of CTAs with the gating
# in the epilogue: measured against cuBLAS + the SwiGLU kernel at [rows, 4096] x [24576, 4096]: 83 / 81 us at 512 rows,
# 111 / 112 at 768, 276 / 302 at 2,048, 508 / 623 at 4,096.
PAIR_MIN_ROWS = 768


def pair_ok(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tcgen05 kernels (TMA-fed) take this product: bfloat16, rows of whole 16-byte pieces."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and w.shape[0] % 16 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gated_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, interleave: int, ctx=None) -> None:
    """out[T, I] = silu(x @ gate^T) * (x @ up^T) for the fused weight ``w`` [2I, K] of a gated
    feed-forward.  With the interleaved layout the product's epilogue does the gating where an own kernel
    is the fastest: for few rows (weight streaming) and for many (tcgen05, pairs of CTAs); otherwise a product
    into a [T, 2I] buffer (from ``ctx``, a parts.base.LayerContext, if given) is followed by the SwiGLU kernel."""
    if interleave == 8 and skinny_ok(x, w):
        gemm_skinny(x, w, out, gated=True)
        return
    if interleave == 8 and x.shape[0] >= PAIR_MIN_ROWS and pair_ok(x, w, out):
        gemm_tc5(x, w, out, gated=True, pair=True)
        return
    if ctx is not None:
        gu = ctx.buffer("gated_linear.gate_up", (x.shape[0], w.shape[0]), x.dtype, x.device)
    else:
        gu = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
    linear(x, w, gu)
    swiglu(gu, out, interleave)


_tc5 = None
_TC5_SOURCES = ["gemm_tc5.cu", "gemm_stream.cu"]


def _tc5_defines():
    return {"RB_PDL_MODE": PDL_MODE}


def tc5_lib() -> ctypes.CDLL:
    """The tcgen05 / TMA matrix-product library."""
    global _tc5
    if _tc5 is None:
        lib = build.load("return_tc5", _TC5_SOURCES, _tc5_defines())
        P, I = c_void_p, c_int
        lib.rb_gemm_stream.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P, P]
        lib.rb_gemm_stream.restype = c_int
        lib.rb_gemm_stream_plan.argtypes = [I, I, I, I, P]
        lib.rb_gemm_stream_plan.restype = None
        lib.rb_tc5_gemm.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P, P]
        lib.rb_tc5_gemm_pair.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P, P]
        lib.rb_tc5_gemm_pair.restype = c_int
        lib.rb_tc5_gemm_simple.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P, P]
        lib.rb_tc5_gemm_bmn.argtypes = [P, P, P, I, I, I, I, I, I, I, P, P]
        lib.rb_tc5_gemm.restype = lib.rb_tc5_gemm_simple.restype = lib.rb_tc5_gemm_bmn.restype = c_int
        _tc5 = lib
    return _tc5


_tc5_status = {}


def tc5_status(device) -> torch.Tensor:
    """One int per device that a tcgen05 kernel raises when one of its bounded waits gave up."""
    t = _tc5_status.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _tc5_status[device] = t
    return t


_tc5_launched = set()          # devices on which a kernel with bounded waits ran since the status word was last read


def check_status(device) -> None:
    """Reads the status word of the tcgen05 kernels if one of them ran on ``device`` since the last check, and
    raises ``KernelError`` if a bounded wait gave up (the kernel's output is then not to be trusted).  It
    synchronises, so callers use it where they wait for the step anyway (after sampling, after a replayed step)."""
    device = torch.device(device)
    if device not in _tc5_launched:
        return
    _tc5_launched.discard(device)
    t = _tc5_status.get(device)
    if t is None:
        return
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise KernelError(f"a kernel on {device} gave up a bounded wait (an mbarrier, or the other CTAs of its grid) or "
                          f"found its shared memory misaligned (status {code}); the step's output is not valid")


def gemm_tc5(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False, simple_bn: int = 0,
             pair: bool = False) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA-fed).  ``gated``: SwiGLU epilogue over
    woven gate/up rows of w, out [M, N/2].  ``simple_bn``: run the one-stage twin with that tile width.
    ``pair``: 256 x 256 tiles by pairs of CTAs (two-SM MMAs)."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    assert w.shape[1] == K and out.shape == (M, N // 2 if gated else N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    status = tc5_status(x.device)
    f32 = 1 if out.dtype == torch.float32 else 0
    if simple_bn:
        rc = tc5_lib().rb_tc5_gemm_simple(_ptr(x), _ptr(w), _ptr(out), f32, simple_bn, M, N, K, x.stride(0),
                                          w.stride(0), out.stride(0), _ptr(status), _stream())
    else:
        fn = tc5_lib().rb_tc5_gemm_pair if pair else tc5_lib().rb_tc5_gemm
        rc = fn(_ptr(x), _ptr(w), _ptr(out), f32, 1 if gated else 0, M, N, K, x.stride(0),
                w.stride(0), out.stride(0), _ptr(status), _stream())
    _tc5_launched.add(x.device)
    _check(rc, "gemm_tc5")


STREAM_MAX_ROWS = 128


def stream_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 weight-streaming kernel takes this product."""
    return (x.dtype == torch.bfloat16 and x.shape[0] <= STREAM_MAX_ROWS and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 128 in bfloat16: weights streamed by TMA through tcgen05 with the
    operand roles exchanged (weight rows on the 128 tensor-memory lanes, tokens as columns), the rows dealt out
    evenly to one CTA per SM.  ``gated``: w holds gate and up rows woven in blocks of 8; out[M, N/2] = silu(gate) * up."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    assert w.shape[1] == K and out.shape == (M, N // 2 if gated else N) and M <= STREAM_MAX_ROWS
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(tc5_lib().rb_gemm_stream(_ptr(x), _ptr(w), _ptr(out), 1 if out.dtype == torch.float32 else 0,
                                    1 if gated else 0, M, N, K, x.stride(0), w.stride(0), out.stride(0),
                                    _ptr(tc5_status(x.device)), _stream()), "gemm_stream")


def gemm_stream_plan(M: int, N: int, K: int, gated: bool = False):
    """(rows of the largest range, chunks per CTA, rows of the tallest chunk, parts of K side by side on the lanes)
    on the current device."""
    buf = (c_int * 4)()
    tc5_lib().rb_gemm_stream_plan(M, N, K, 1 if gated else 0, buf)
    return tuple(buf)


def gemm_tc5_bmn(x: torch.Tensor, b: torch.Tensor, out: torch.Tensor, bn: int = 128) -> None:
    """out[M, N] (float32) = x[M, K] @ b[K, N], b row-major: the tcgen05 twin with an MN-major B operand."""
    M, K = x.shape
    N = b.shape[1]
    assert x.dtype == b.dtype == torch.bfloat16 and out.dtype == torch.float32 and b.shape[0] == K
    _check(tc5_lib().rb_tc5_gemm_bmn(_ptr(x), _ptr(b), _ptr(out), bn, M, N, K, x.stride(0), b.stride(0), out.stride(0),
                                     _ptr(tc5_status(x.device)), _stream()), "gemm_tc5_bmn")


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = x @ w^T.  float32: the engine's own FFMA kernel.  bfloat16 with up to 8 rows: the
    engine's weight-streaming kernel.  bfloat16 with more rows: cuBLAS with float32 accumulation.
    The output is bfloat16 or float32 (``out``'s dtype)."""
    if x.dtype == torch.float32:
        gemm_f32(x, w, out)
        return
    if not x.is_cuda:
        raise KernelError("the engine's kernels run on a CUDA device only; got a CPU tensor")
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if skinny_ok(x, w):
        gemm_skinny(x, w, out)
        return
    if out.dtype == torch.float32:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        torch.mm(x, w.t(), out=out)


# ------------------------------------------------------------------------------- attention

def qk_norm_rope_write(qkv, q_weight, k_weight, eps, cos, sin, rot_dim, pos, tok_seg, block_table,
                       page_size, k_pool, v_pool, num_heads, num_kv_heads, head_dim, write_kv=True,
                       offset=0.0) -> None:
    """In place on qkv [T, (Hq+2Hkv)*D]: q heads normed and rotated; k heads normed, rotated and
    written to ``k_pool``; v heads written to ``v_pool``.  Pools: [pages, Hkv, P, D]."""
    T = qkv.shape[0]
    assert qkv.stride(1) == 1
    assert pos.dtype == tok_seg.dtype == block_table.dtype == torch.int32
    assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype
    if rot_dim:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32
        assert cos.shape[1] * 2 == rot_dim and cos.is_contiguous() and sin.is_contiguous()
        assert rot_dim <= head_dim
    else:
        cos = sin = pos            # never read: a rotary width of zero rotates nothing
    wd = dtype_code(q_weight.dtype) if q_weight is not None else F32
    if q_weight is not None:
        assert k_weight is not None and k_weight.dtype == q_weight.dtype
    _check(core().rb_qk_norm_rope_write(
        _ptr(qkv), qkv.stride(0), _ptr(q_weight), _ptr(k_weight), wd, eps, offset, _ptr(cos), _ptr(sin),
        rot_dim, _ptr(pos), _ptr(tok_seg), _ptr(block_table), block_table.stride(0), page_size,
        _ptr(k_pool), _ptr(v_pool), dtype_code(qkv.dtype), T, num_heads, num_kv_heads, head_dim,
        1 if write_kv else 0, _stream()), "qk_norm_rope_write")


def attention_simt(qkv, k_pool, v_pool, pos, tok_seg, block_table, page_size, out, num_heads,
                   num_kv_heads, head_dim, scale, window=0) -> None:
    """Paged causal attention, one warp per (token, head); out [T, Hq*D]."""
    T = qkv.shape[0]
    assert out.is_contiguous() and out.dtype == qkv.dtype and k_pool.dtype == qkv.dtype
    _check(core().rb_attention_simt(
        _ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(pos), _ptr(tok_seg), _ptr(block_table),
        block_table.stride(0), page_size, _ptr(out), dtype_code(qkv.dtype), T, num_heads, num_kv_heads,
        head_dim, scale, int(window or 0), _stream()), "attention_simt")


_attn_libs = {}


def _attn_defines(head_dim: int):
    return {"HEAD_DIM": head_dim, "RB_PDL_MODE": PDL_MODE}


def attention_lib(head_dim: int) -> ctypes.CDLL:
    """The tensor-core attention kernels, compiled for this head size on first use."""
    lib = _attn_libs.get(head_dim)
    if lib is None:
        if head_dim % 16 or not (16 <= head_dim <= 256):
            raise KernelError(f"head_dim={head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        lib = build.load(f"return_attn_d{head_dim}", ["attention_mma.cu"], _attn_defines(head_dim))
        P, I, F = c_void_p, c_int, c_float
        lib.rb_attn_prefill.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, I, I, F, I, P]
        lib.rb_attn_decode.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, P, I, I, F, I, I, P]
        lib.rb_attn_decode_fused.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, P, I, I, F, I, I, P, P, I, F, F, P, P, I, I, P]
        lib.rb_attn_decode_fused.restype = c_int
        lib.rb_attn_decode_scratch_floats.argtypes = [I, I, I]
        lib.rb_attn_decode_scratch_floats.restype = ctypes.c_longlong
        lib.rb_attn_prefill.restype = lib.rb_attn_decode.restype = lib.rb_attn_head_dim.restype = c_int
        if lib.rb_attn_head_dim() != head_dim:
            raise KernelError("attention library was compiled for another head size")
        _attn_libs[head_dim] = lib
    return lib


_attn_tc5_libs = {}
TC5_ATTENTION_HEAD_DIMS = (64, 128)
TC5_TILE_ROWS = 256            # query rows of one CTA of the tcgen05 prefill attention kernel
MMA_TILE_ROWS = 64             # query rows of one CTA of the mma.sync prefill attention kernel
TILES_TC5, TILES_MMA = "attention.rows256", "attention.rows64"     # the names of their tables in a step's batch

_num_sms = None


def num_sms() -> int:
    """Streaming multiprocessors of the current device (asked of the driver once).  Where no device is
    visible (the dispatch rules are also tested on the host) the count of a B200 stands in."""
    global _num_sms
    if _num_sms is None:
        _num_sms = (torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
                    if torch.cuda.is_available() else 148)
    return _num_sms


def _attn_tc5_defines(head_dim: int):
    return {"HEAD_DIM": head_dim}


def attention_tc5_lib(head_dim: int) -> ctypes.CDLL:
    """The tcgen05 prefill attention kernel, compiled for this head size (64 or 128) on first use."""
    lib = _attn_tc5_libs.get(head_dim)
    if lib is None:
        if head_dim not in TC5_ATTENTION_HEAD_DIMS:
            raise KernelError(f"head_dim={head_dim}: the tcgen05 attention kernel takes {TC5_ATTENTION_HEAD_DIMS}")
        lib = build.load(f"return_attn_tc5_d{head_dim}", ["attention_tc5.cu"], _attn_tc5_defines(head_dim))
        P, I, F = c_void_p, c_int, c_float
        lib.rb_attn_prefill_tc5.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, I, I, F, I, I, P, I, P, P]
        lib.rb_attn_tc5_split_floats.argtypes = [I, I, I]
        lib.rb_attn_tc5_split_floats.restype = ctypes.c_longlong
        lib.rb_attn_prefill_tc5.restype = c_int
        _attn_tc5_libs[head_dim] = lib
    return lib


def attention_prefill_tc5(qkv, k_pool, v_pool, tiles, cu_q, seg_pos0, block_table, page_size, out, num_heads,
                          num_kv_heads, head_dim, scale, window=0, num_splits=1, held=None) -> None:
    """tcgen05 attention for the listed (segment, first row) blocks of up to TC5_TILE_ROWS query rows
    (the blocks with the longest contexts should come first: they take longest).  ``num_splits`` > 1 splits
    every block's keys over that many CTAs and merges them in a second launch; ``held``: the step's map of
    work buffers, so that the layers share the buffer of the partial results."""
    assert qkv.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    assert tiles.dtype == torch.int32 and tiles.is_contiguous()
    lib = attention_tc5_lib(head_dim)
    T = qkv.shape[0]
    _tc5_launched.add(qkv.device)
    scratch = None
    if num_splits > 1:
        key = ("attention.prefill_split_scratch", num_splits, T, num_heads, head_dim)
        scratch = held.get(key) if held is not None else None
        if scratch is None:
            scratch = torch.empty(lib.rb_attn_tc5_split_floats(num_splits, T, num_heads), dtype=torch.float32, device=qkv.device)
            if held is not None:
                held[key] = scratch
    _check(lib.rb_attn_prefill_tc5(_ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(tiles),
                                   tiles.shape[0], _ptr(cu_q), _ptr(seg_pos0), _ptr(block_table),
                                   block_table.stride(0), page_size, _ptr(out), num_heads, num_kv_heads, scale,
                                   int(window or 0), num_splits, _ptr(scratch), T, _ptr(tc5_status(qkv.device)),
                                   _stream()), "attention_prefill_tc5", 2 if num_splits > 1 else 1)


PREFILL_SPLIT_MIN_KEYS = 512       # a CTA of a split block keeps at least this many keys


def prefill_splits(n_ctas: int, longest_context: int) -> int:
    """How many ways the keys of the prompt blocks are split: a CTA owns an SM, so blocks x heads below
    the SM count leave SMs idle (a short portion of a long prompt); the keys are then shared out until the
    CTAs fill the GPU once, as long as every share keeps PREFILL_SPLIT_MIN_KEYS keys."""
    return max(1, min(num_sms() // max(1, n_ctas), longest_context // PREFILL_SPLIT_MIN_KEYS, 64))


def _prefill_split_count(batch, num_heads, window) -> int:
    held = getattr(batch, "scratch", None)
    key = ("attention.prefill_splits", num_heads, window)
    if held is not None and key in held:
        return held[key]
    host = batch.host
    tiles = host.tiles[TILES_TC5]
    longest = int(host.seg_kv_len[tiles[:, 0]].max())
    if window:
        longest = min(longest, int(window) + TC5_TILE_ROWS)
    n = prefill_splits(tiles.shape[0] * num_heads, longest)
    if held is not None:
        held[key] = n
    return n


def decode_splits(n_ctas_base: int, max_kv_len: int, ctas_per_sm: int = 2) -> int:
    """How many ways the keys of a decoded token are split.  Two CTAs share an SM (head sizes up to
    128), so the time of the launch goes with (waves of CTAs) x (keys per CTA); the split count that
    makes this smallest wins, with at least 128 keys per CTA and the smaller count on a tie."""
    tiles = max(1, (max_kv_len + 15) // 16)
    slots = num_sms() * ctas_per_sm
    best, best_cost = 1, None
    for s in range(1, 65):
        if s > 1 and (max_kv_len + s - 1) // s < 128:
            break
        waves = (n_ctas_base * s + slots - 1) // slots
        cost = waves * ((tiles + s - 1) // s + 16)         # + the fixed work of a CTA, about 16 tiles' worth (3 us)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def attention_prefill_mma(qkv, k_pool, v_pool, tiles, cu_q, seg_pos0, block_table, page_size, out, num_heads,
                          num_kv_heads, head_dim, scale, window=0) -> None:
    """Tensor-core attention for the listed (segment, first row) tiles of up to 64 query rows."""
    assert qkv.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    assert tiles.dtype == torch.int32 and tiles.is_contiguous()
    lib = attention_lib(head_dim)
    _check(lib.rb_attn_prefill(_ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(tiles), tiles.shape[0],
                               _ptr(cu_q), _ptr(seg_pos0), _ptr(block_table), block_table.stride(0), page_size,
                               _ptr(out), num_heads, num_kv_heads, scale, int(window or 0), _stream()),
           "attention_prefill")


def _split_scratch(lib, n, num_heads, num_splits, device, held=None):
    """The buffer in which the splits of the keys leave their partial results (none for one split).
    ``held``: the step's map of work buffers; every layer of the step then shares one."""
    key = ("attention.split_scratch", n, num_heads, num_splits)
    if held is not None and key in held:
        return held[key]
    floats = lib.rb_attn_decode_scratch_floats(n, num_heads, num_splits)
    scratch = torch.empty(floats, dtype=torch.float32, device=device) if floats else None
    if held is not None:
        held[key] = scratch
    return scratch


def attention_decode_mma(qkv, k_pool, v_pool, decode_segs, cu_q, seg_kv_len, block_table, page_size, out,
                         num_heads, num_kv_heads, head_dim, scale, window=0, num_splits=1, held=None) -> None:
    """Tensor-core attention for segments of one token, the keys split ``num_splits`` ways."""
    assert qkv.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    lib = attention_lib(head_dim)
    n = decode_segs.shape[0]
    scratch = _split_scratch(lib, n, num_heads, num_splits, qkv.device, held)
    _check(lib.rb_attn_decode(_ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(decode_segs), n,
                              _ptr(cu_q), _ptr(seg_kv_len), _ptr(block_table), block_table.stride(0), page_size,
                              _ptr(scratch), _ptr(out), num_heads, num_kv_heads, scale, int(window or 0),
                              num_splits, _stream()), "attention_decode", 2 if num_splits > 1 else 1)


def _decode_split_count(batch, num_heads, num_kv_heads, window) -> int:
    """The split count of this step's decoded tokens, worked out once per step and kind of layer."""
    held = getattr(batch, "scratch", None)
    if held is None:
        return _decode_split_count_now(batch, num_heads, num_kv_heads, window)
    key = ("attention.splits", num_heads, num_kv_heads, window)
    n = held.get(key)
    if n is None:
        n = held[key] = _decode_split_count_now(batch, num_heads, num_kv_heads, window)
    return n


def _decode_split_count_now(batch, num_heads, num_kv_heads, window) -> int:
    host = batch.host
    n_dec = host.decode_segs.shape[0]
    group = num_heads // num_kv_heads
    base = n_dec * num_kv_heads * ((group + 15) // 16)
    longest = int(host.seg_kv_len[host.decode_segs].max())
    if window:
        longest = min(longest, int(window))
    fixed = getattr(batch, "variant", {}).get(decode_splits_key(num_heads, num_kv_heads, window))
    return fixed or decode_splits(base, longest)


def decode_splits_key(num_heads, num_kv_heads, window):
    """Under this key a captured step holds the split count of its decoded tokens (``batch.variant``)."""
    return ("attention.decode_splits", num_heads, num_kv_heads, window or 0)


def decode_splits_for(n_tokens: int, longest: int, num_heads: int, num_kv_heads: int, window=None) -> int:
    """The split count of a step of ``n_tokens`` single tokens whose contexts reach ``longest`` keys."""
    group = num_heads // num_kv_heads
    if window:
        longest = min(longest, int(window))
    return decode_splits(n_tokens * num_kv_heads * ((group + 15) // 16), longest)


def decode_only(batch, dtype, num_heads, num_kv_heads, window=None) -> bool:
    """Whether the step holds single decoded tokens only, runs on the tensor-core path, and is small enough
    that the decode attention kernel should norm, rotate and cache those tokens itself: the saved launch
    pays while the kernel's CTAs fit on the GPU at once; with more, the work added to every CTA costs
    more than the small kernel it replaces (measured: +1 % at 8 requests, -2 % at 64)."""
    host = batch.host
    if not (dtype == torch.bfloat16 and host.num_multi == 0
            and host.decode_segs.shape[0] == host.num_tokens and host.num_tokens > 0):
        return False
    group = num_heads // num_kv_heads
    ctas = host.num_tokens * num_kv_heads * ((group + 15) // 16) * _decode_split_count(batch, num_heads, num_kv_heads, window)
    return ctas <= 2 * num_sms()


def attention_decode_fused(qkv, q_weight, k_weight, eps, offset, cos, sin, rot_dim, k_pool, v_pool, batch,
                           block_table, page_size, out, num_heads, num_kv_heads, head_dim, scale, window=None,
                           write_kv=True) -> None:
    """A step of single tokens: per-head q/k norm, rotation, cache write and split-KV attention in one kernel
    (plus the merge of the splits).  ``qkv`` holds the raw projections and is left as it is."""
    assert qkv.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    lib = attention_lib(head_dim)
    n = batch.decode_segs.shape[0]
    splits = _decode_split_count(batch, num_heads, num_kv_heads, window)
    scratch = _split_scratch(lib, n, num_heads, splits, qkv.device, getattr(batch, "scratch", None))
    if rot_dim:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape[1] * 2 == rot_dim
        assert cos.is_contiguous() and sin.is_contiguous()
    else:
        cos = sin = batch.cu_q          # never read: a rotary width of zero rotates nothing
    wd = dtype_code(q_weight.dtype) if q_weight is not None else F32
    _check(lib.rb_attn_decode_fused(_ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(batch.decode_segs), n,
                                    _ptr(batch.cu_q), _ptr(batch.seg_kv_len), _ptr(block_table), block_table.stride(0),
                                    page_size, _ptr(scratch), _ptr(out), num_heads, num_kv_heads, scale,
                                    int(window or 0), splits, _ptr(q_weight), _ptr(k_weight), wd, eps, offset,
                                    _ptr(cos), _ptr(sin), rot_dim, 1 if write_kv else 0, _stream()),
           "attention_decode_fused", 2 if splits > 1 else 1)


def paged_attention(qkv, k_pool, v_pool, batch, block_table, page_size, out, num_heads, num_kv_heads,
                    head_dim, scale, window=None) -> None:
    """Attention of every token of the step over its request's cached keys (its own included).

    float32: the CUDA-core kernel, whose result does not depend on how the work was cut.
    bfloat16: the tensor-core kernels, one for prompt portions and one (split over the keys) for
    single decoded tokens."""
    if qkv.dtype == torch.float32:
        attention_simt(qkv, k_pool, v_pool, batch.pos, batch.tok_seg, block_table, page_size, out,
                       num_heads, num_kv_heads, head_dim, scale, window or 0)
        return
    host = batch.host
    if host.num_multi:
        if head_dim in TC5_ATTENTION_HEAD_DIMS:
            attention_prefill_tc5(qkv, k_pool, v_pool, batch.tiles[TILES_TC5], batch.cu_q, batch.seg_pos0, block_table,
                                  page_size, out, num_heads, num_kv_heads, head_dim, scale, window or 0,
                                  _prefill_split_count(batch, num_heads, window), getattr(batch, "scratch", None))
        else:
            attention_prefill_mma(qkv, k_pool, v_pool, batch.tiles[TILES_MMA], batch.cu_q, batch.seg_pos0, block_table,
                                  page_size, out, num_heads, num_kv_heads, head_dim, scale, window or 0)
    n_dec = host.decode_segs.shape[0]
    if n_dec:
        attention_decode_mma(qkv, k_pool, v_pool, batch.decode_segs, batch.cu_q, batch.seg_kv_len, block_table,
                             page_size, out, num_heads, num_kv_heads, head_dim, scale, window or 0,
                             _decode_split_count(batch, num_heads, num_kv_heads, window), getattr(batch, "scratch", None))


# ------------------------------------------------------------------------------- sampling

def sample(logits, temperature, top_k, top_p, uniform, tokens_out, logprobs_out=None, one_cta: bool = False) -> None:
    """One token per row of float32 logits [n, V]; per-row temperature, top_k, top_p and uniform draw.
    A cluster of eight CTAs takes a row (its parts in their shared memories); ``one_cta``: the kernel with one CTA
    a row, which takes rows of any length and is what rows too long for eight shared memories fall back to."""
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and uniform.dtype == torch.float32
    assert top_k.dtype == torch.int32 and tokens_out.dtype == torch.int32
    _check(core().rb_sample(_ptr(logits), logits.stride(0), n, V, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                            _ptr(uniform), _ptr(tokens_out), _ptr(logprobs_out), 1 if one_cta else 0, _stream()), "sample")


def argmax(logits, tokens_out) -> None:
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and tokens_out.dtype == torch.int32
    _check(core().rb_argmax(_ptr(logits), logits.stride(0), n, V, _ptr(tokens_out), _stream()), "argmax")
