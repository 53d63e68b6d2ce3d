"""rb_attn_decode_static, the decode-attention entry point that allocates nothing.

Some users of the kernels cannot allocate device memory when they call: a host that gave all free
memory to the KV pool at start-up, a decode loop that must never enter cudaMalloc, a program that
links the library without PyTorch.  For them the split kernel's scratch sits in a device array
inside the library.  This test calls the entry point through its exported C symbol, with raw
pointers, twice in a row on different inputs (the array keeps the first call's contents, which
must not leak into the second).  Each result is compared with the plain float32 attention of the
tests (the oracle of every other attention test) and with the ordinary entry point that takes a
scratch buffer, and the device memory in use is read before and after a call to see that the call
took none.  It is collected last, so a run that stops at the first failure has run everything else.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

import helpers
from helpers import plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HQ, HKV, D, P = 8, 2, 64, 16


def _library():
    from return_b200.ext import build, ops
    lib = ctypes.CDLL(build.library_path(f"return_attn_d{D}", ["attention_mma.cu"],
                                         {"HEAD_DIM": D, "RB_PDL_MODE": ops.PDL_MODE}))
    Ptr, I = c_void_p, c_int
    lib.rb_attn_decode_static.argtypes = [Ptr, I, Ptr, Ptr, Ptr, I, Ptr, Ptr, Ptr, I, I, Ptr, I, I, c_float, I, I, Ptr]
    lib.rb_attn_decode_static.restype = c_int
    lib.rb_attn_decode_static_capacity.restype = ctypes.c_longlong
    return lib


def _case(seed, kv_lens):
    g = torch.Generator().manual_seed(seed)
    n = len(kv_lens)
    blocks = [(L + P - 1) // P for L in kv_lens]
    n_pages = sum(blocks) + 2
    perm = iter(torch.randperm(n_pages, generator=g).tolist())
    kpool = torch.randn(n_pages, HKV, P, D, generator=g).bfloat16()
    vpool = torch.randn(n_pages, HKV, P, D, generator=g).bfloat16()
    bt = torch.full((n, max(blocks)), -1, dtype=torch.int32)
    for i, nb in enumerate(blocks):
        for b in range(nb):
            bt[i, b] = next(perm)
    qkv = torch.randn(n, (HQ + 2 * HKV) * D, generator=g).bfloat16()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return dict(qkv=qkv.to(DEV), kpool=kpool.to(DEV), vpool=vpool.to(DEV), bt=bt.to(DEV), segs=i32(list(range(n))),
                cu_q=i32(list(range(n + 1))), kv_len=i32(kv_lens), n=n,
                host=dict(qkv=qkv, kpool=kpool, vpool=vpool, bt=bt, kv_lens=kv_lens))


def _plain(c, window=0):
    """The plain float32 attention over the same (bfloat16-rounded) numbers, request by request."""
    h = c["host"]
    outs = []
    for i, L in enumerate(h["kv_lens"]):
        pages = h["bt"][i, :(L + P - 1) // P].long()
        k = h["kpool"][pages].float().permute(0, 2, 1, 3).reshape(-1, HKV, D)[:L]       # [L, Hkv, D]
        v = h["vpool"][pages].float().permute(0, 2, 1, 3).reshape(-1, HKV, D)[:L]
        q = h["qkv"][i, :HQ * D].float().reshape(1, HQ, D)
        o = plain.attention_scores_softmax_pv(q, k, v, torch.tensor([L - 1]), torch.arange(L), 1.0 / math.sqrt(D),
                                              window or None)
        outs.append(o.reshape(1, -1))
    return torch.cat(outs)


def _static(lib, c, splits, window=0):
    out = torch.full((c["n"], HQ * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    ptr = lambda t: c_void_p(t.data_ptr())
    rc = lib.rb_attn_decode_static(ptr(c["qkv"]), c["qkv"].stride(0), ptr(c["kpool"]), ptr(c["vpool"]), ptr(c["segs"]),
                                   c["n"], ptr(c["cu_q"]), ptr(c["kv_len"]), ptr(c["bt"]), c["bt"].stride(0), P,
                                   ptr(out), HQ, HKV, 1.0 / math.sqrt(D), window, splits,
                                   c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, out


def _ordinary(c, splits, window=0):
    from return_b200.ext import ops
    out = torch.full((c["n"], HQ * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_decode_mma(c["qkv"], c["kpool"], c["vpool"], c["segs"], c["cu_q"], c["kv_len"], c["bt"], P, out,
                             HQ, HKV, D, 1.0 / math.sqrt(D), window, num_splits=splits)
    torch.cuda.synchronize()
    return out


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = _library()
    first = _case(1, [300, 17, 129, 64, 511])
    second = _case(2, [40, 200, 333])                      # fewer, other requests: stale scratch must not show
    for case, splits, window in ((first, 4, 0), (second, 3, 0), (first, 1, 0), (second, 5, 90)):
        rc, got = _static(lib, case, splits, window)
        assert rc == 0
        assert torch.isfinite(got.float()).all()
        assert torch.allclose(got.float().cpu(), _plain(case, window), atol=3e-2, rtol=3e-2)
        assert torch.allclose(got.float(), _ordinary(case, splits, window).float(), atol=3e-2, rtol=3e-2)


def test_static_scratch_entry_point_takes_no_device_memory():
    """What the entry point is for: a call allocates nothing, neither through torch's allocator nor from
    the driver.  After a first call (which looks up the array's address), the memory in use on the device
    is read, the entry point is called on inputs that already exist, and the memory is read again."""
    lib = _library()
    c = _case(4, [257, 90, 33, 400])
    out = torch.empty((c["n"], HQ * D), dtype=torch.bfloat16, device=DEV)
    ptr = lambda t: c_void_p(t.data_ptr())
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(splits):
        return lib.rb_attn_decode_static(ptr(c["qkv"]), c["qkv"].stride(0), ptr(c["kpool"]), ptr(c["vpool"]),
                                         ptr(c["segs"]), c["n"], ptr(c["cu_q"]), ptr(c["kv_len"]), ptr(c["bt"]),
                                         c["bt"].stride(0), P, ptr(out), HQ, HKV, 1.0 / math.sqrt(D), 0, splits, stream)

    assert call(4) == 0
    torch.cuda.synchronize()
    torch_before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
    free_before, _ = torch.cuda.mem_get_info()
    for splits in (4, 7, 1):
        assert call(splits) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == torch_before
    assert free_after == free_before, (free_before, free_after)
    assert torch.allclose(out.float().cpu(), _plain(c), atol=3e-2, rtol=3e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _library()
    cap = lib.rb_attn_decode_static_capacity()
    assert cap == 1 << 20
    c = _case(3, [64] * 8)
    # n_dec * Hq * splits * (D + 2) floats must fit: 8 * 8 * 64 * 66 = 270k fits, a made-up huge head count does not
    rc, _ = _static(lib, c, 64)
    assert rc == 0
    out = torch.empty((8, HQ * D), dtype=torch.bfloat16, device=DEV)
    ptr = lambda t: c_void_p(t.data_ptr())
    rc = lib.rb_attn_decode_static(ptr(c["qkv"]), c["qkv"].stride(0), ptr(c["kpool"]), ptr(c["vpool"]), ptr(c["segs"]),
                                   c["n"], ptr(c["cu_q"]), ptr(c["kv_len"]), ptr(c["bt"]), c["bt"].stride(0), P,
                                   ptr(out), 4096, 1024, 0.125, 0, 64, c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -2                                        # RB_ERR_SCRATCH_TOO_LARGE: nothing was launched
    torch.cuda.synchronize()
