"""Each CUDA kernel alone against its plain float32 reference, at sizes other than the engine's."""
import math

import pytest
import torch

import helpers
from helpers import plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops():
    from return_b200.ext import ops
    return ops


def _tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


# ------------------------------------------------------------------------------- elementwise

@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embedding(table_dtype):
    ops = _ops()
    V, H = 301, 136
    table = torch.randn(V, H, device=DEV).to(table_dtype)
    tokens = torch.randint(0, V, (37,), device=DEV, dtype=torch.int32)
    out = torch.empty(37, H, device=DEV)
    ops.embedding(table, tokens, out)
    assert torch.equal(out, table[tokens.long()].float())
    bad = torch.tensor([5, V, -1], device=DEV, dtype=torch.int32)      # outside the table: NaN, no foreign read
    out = torch.zeros(3, H, device=DEV)
    ops.embedding(table, bad, out)
    assert torch.isfinite(out[0]).all() and torch.isnan(out[1:]).all()


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [24, 200, 4096 + 8])
def test_add_rmsnorm(act, wdt, H):
    ops = _ops()
    T, eps = 19, 3e-5
    stream = torch.randn(T, H, device=DEV)
    delta = torch.randn(T, H, device=DEV).to(act)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(wdt)
    want_stream = stream + delta.float()
    want = plain.rms_norm(want_stream, w.float(), eps)
    out = torch.empty(T, H, device=DEV, dtype=act)
    s2 = stream.clone()
    ops.add_rmsnorm(s2, delta, w, eps, out)
    assert torch.allclose(s2, want_stream, atol=1e-6)
    assert torch.allclose(out.float(), want, **_tol(act))
    # no delta: the stream is only read
    s3 = stream.clone()
    ops.add_rmsnorm(s3, None, w, eps, out)
    assert torch.equal(s3, stream)
    assert torch.allclose(out.float(), plain.rms_norm(stream, w.float(), eps), **_tol(act))
    # rows: only the listed rows, a row may be listed twice, the stream stays as it is
    rows = torch.tensor([3, 3, 18, 0], device=DEV, dtype=torch.int32)
    out4 = torch.empty(4, H, device=DEV, dtype=act)
    s4 = stream.clone()
    ops.add_rmsnorm(s4, delta, w, eps, out4, rows=rows)
    assert torch.equal(s4, stream)
    assert torch.allclose(out4.float(), want[rows.long()], **_tol(act))


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [16, 48, 80, 256])
def test_rmsnorm_rows(act, N):
    ops = _ops()
    x = torch.randn(7, 5, N, device=DEV).to(act)
    w = (1 + 0.1 * torch.randn(N, device=DEV))
    out = torch.empty_like(x)
    ops.rmsnorm_rows(x, w, 1e-6, out, offset=1.0)
    want = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * (1.0 + w)
    assert torch.allclose(out.float(), want, **_tol(act))


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I", [8, 100, 224, 1000])
def test_swiglu(act, I):
    ops = _ops()
    gu = (3 * torch.randn(13, 2 * I, device=DEV)).to(act)
    out = torch.empty(13, I, device=DEV, dtype=act)
    ops.swiglu(gu, out)
    g, u = gu.float()[:, :I], gu.float()[:, I:]
    assert torch.allclose(out.float(), g * torch.sigmoid(g) * u, **_tol(act))
    if I % 8 == 0:                       # the woven layout: blocks of 8 gate columns then 8 up columns
        woven = torch.stack([gu[:, :I].reshape(13, -1, 8), gu[:, I:].reshape(13, -1, 8)], dim=2).reshape(13, 2 * I).contiguous()
        out2 = torch.empty_like(out)
        ops.swiglu(woven, out2, interleave=8)
        assert torch.equal(out2, out)


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 257), (65, 64, 16), (100, 200, 96), (2, 384, 96)])
def test_gemm_f32_is_exact_float32(M, N, K):
    ops = _ops()
    x = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV)
    out = torch.empty(M, N, device=DEV)
    ops.gemm_f32(x, w, out)
    want = (x.double() @ w.double().T)
    assert (out.double() - want).abs().max() < 1e-4 * max(1.0, K ** 0.5)
    # a row's result does not depend on which other rows are in the product
    one = torch.empty(1, N, device=DEV)
    ops.gemm_f32(x[M - 1:M], w, one)
    assert torch.equal(one[0], out[M - 1])
    # no TF32: a value that TF32 would round away survives
    x2 = torch.tensor([[1.0, 2.0 ** -12]], device=DEV)
    w2 = torch.tensor([[1.0, 1.0]], device=DEV)
    o2 = torch.empty(1, 1, device=DEV)
    ops.gemm_f32(x2, w2, o2)
    assert o2.item() == 1.0 + 2.0 ** -12


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("N,K", [(16, 32), (100, 72), (384, 96), (1000, 4096), (4104, 1544)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_skinny(M, N, K, out_dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16().to(DEV)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.gemm_skinny(x, w, out)
    want = x.double() @ w.double().T
    tol = 2e-3 if out_dtype == torch.float32 else 2e-2
    assert (out.double() - want).abs().max() < tol
    # a view with a row stride (the q part of a qkv buffer) works too
    big = torch.zeros(M, K + 64, dtype=torch.bfloat16, device=DEV)
    big[:, :K] = x
    out2 = torch.empty_like(out)
    ops.gemm_skinny(big[:, :K], w, out2)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("M", [1, 8, 13, 32, 50])
@pytest.mark.parametrize("I,K", [(8, 32), (104, 40), (224, 96), (3072, 1024)])
def test_gated_linear(M, I, K):
    """The gated product (SwiGLU in the epilogue for few rows, product + kernel otherwise) against plain math."""
    ops = _ops()
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    gate = (torch.randn(I, K, generator=g) / K ** 0.5).bfloat16()
    up = (torch.randn(I, K, generator=g) / K ** 0.5).bfloat16()
    woven = torch.stack([gate.view(-1, 8, K), up.view(-1, 8, K)], dim=1).reshape(2 * I, K).contiguous().to(DEV)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gated_linear(x, woven, out, 8)
    gg, uu = x.float().cpu() @ gate.float().T, x.float().cpu() @ up.float().T
    assert torch.allclose(out.float().cpu(), gg * torch.sigmoid(gg) * uu, atol=2e-2, rtol=3e-2)
    plain_layout = torch.cat([gate, up]).to(DEV)
    out2 = torch.empty_like(out)
    ops.gated_linear(x, plain_layout, out2, 0)
    assert torch.allclose(out2.float(), out.float(), atol=2e-2, rtol=3e-2)


def test_linear_bf16_float32_out():
    ops = _ops()
    for M in (5, 70):                      # few rows: the engine's kernel; more: the library
        x = torch.randn(M, 96, device=DEV).bfloat16()
        w = torch.randn(384, 96, device=DEV).bfloat16()
        out = torch.empty(M, 384, device=DEV)
        ops.linear(x, w, out)
        assert torch.allclose(out, x.float() @ w.float().T, atol=1e-3, rtol=1e-3)
    with pytest.raises(ops.KernelError):
        ops.linear(x.cpu(), w.cpu(), out.cpu())


# ------------------------------------------------------------------------------- cache layout helpers

class Paged:
    """Random requests laid out in pages in a scrambled order, with the step's tables."""

    def __init__(self, kv_lens, q_lens, Hq, Hkv, D, P, dtype, seed=0, poison=True):
        g = torch.Generator().manual_seed(seed)
        self.n = len(kv_lens)
        self.Hq, self.Hkv, self.D, self.P = Hq, Hkv, D, P
        self.kv_lens, self.q_lens = kv_lens, q_lens
        blocks = [(L + P - 1) // P for L in kv_lens]
        n_pages = sum(blocks) + 3
        perm = torch.randperm(n_pages, generator=g).tolist()
        self.k = [torch.randn(L, Hkv, D, generator=g) for L in kv_lens]
        self.v = [torch.randn(L, Hkv, D, generator=g) for L in kv_lens]
        self.q = [torch.randn(ql, Hq, D, generator=g) for ql in q_lens]
        fill = float("nan") if poison else 0.0
        kpool = torch.full((n_pages, Hkv, P, D), fill)
        vpool = torch.full((n_pages, Hkv, P, D), fill)
        bt = torch.full((self.n, max(blocks)), -1, dtype=torch.int32)
        it = iter(perm)
        for i, L in enumerate(kv_lens):
            for b in range(blocks[i]):
                page = next(it)
                bt[i, b] = page
                rows = min(P, L - b * P)
                kpool[page, :, :rows] = self.k[i][b * P:b * P + rows].transpose(0, 1)
                vpool[page, :, :rows] = self.v[i][b * P:b * P + rows].transpose(0, 1)
        self.kpool, self.vpool, self.bt = kpool.to(dtype).to(DEV), vpool.to(dtype).to(DEV), bt.to(DEV)
        T = sum(q_lens)
        qkv = torch.zeros(T, (Hq + 2 * Hkv) * D)
        pos, tok_seg, cu_q = [], [], [0]
        row = 0
        for i, ql in enumerate(q_lens):
            qkv[row:row + ql, :Hq * D] = self.q[i].reshape(ql, -1)
            pos += list(range(kv_lens[i] - ql, kv_lens[i]))
            tok_seg += [i] * ql
            row += ql
            cu_q.append(row)
        self.qkv = qkv.to(dtype).to(DEV)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        self.pos, self.tok_seg, self.cu_q = i32(pos), i32(tok_seg), i32(cu_q)
        self.seg_pos0 = i32([kv_lens[i] - q_lens[i] for i in range(self.n)])
        self.seg_kv_len = i32(kv_lens)
        self.dtype = dtype

    def reference(self, scale, window=None):
        outs = []
        rd = lambda t: t.to(self.dtype).float()
        for i in range(self.n):
            L, ql = self.kv_lens[i], self.q_lens[i]
            o = plain.attention_scores_softmax_pv(rd(self.q[i]), rd(self.k[i]), rd(self.v[i]),
                                                  torch.arange(L - ql, L), torch.arange(L), scale, window)
            outs.append(o.reshape(ql, -1))
        return torch.cat(outs)


ATT_SHAPES = [  # Hq, Hkv, D, P
    (4, 2, 16, 16), (6, 3, 32, 8), (5, 1, 48, 16), (8, 8, 64, 4), (7, 7, 80, 32), (32, 8, 128, 16), (3, 1, 256, 64),
    (20, 1, 64, 16),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,P", ATT_SHAPES)
@pytest.mark.parametrize("window", [None, 37])
def test_attention_simt(dtype, Hq, Hkv, D, P, window):
    ops = _ops()
    pg = Paged([1, 70, 200, 33, 129], [1, 70, 1, 20, 3], Hq, Hkv, D, P, dtype, seed=D)
    out = torch.empty(sum(pg.q_lens), Hq * D, device=DEV, dtype=dtype)
    scale = 0.7 / math.sqrt(D)
    ops.attention_simt(pg.qkv, pg.kpool, pg.vpool, pg.pos, pg.tok_seg, pg.bt, P, out, Hq, Hkv, D, scale, window or 0)
    assert torch.allclose(out.float().cpu(), pg.reference(scale, window), **_tol(dtype))


@pytest.mark.parametrize("Hq,Hkv,D,P", ATT_SHAPES)
@pytest.mark.parametrize("window", [None, 37, 100])
def test_attention_prefill_mma(Hq, Hkv, D, P, window):
    ops = _ops()
    kv_lens, q_lens = [2, 70, 200, 64, 129, 300], [2, 70, 3, 64, 65, 130]
    pg = Paged(kv_lens, q_lens, Hq, Hkv, D, P, torch.bfloat16, seed=D + 1)
    tiles = [(i, r0) for i, ql in enumerate(q_lens) for r0 in range(0, ql, 64)]
    tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    out = torch.full((sum(q_lens), Hq * D), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 0.7 / math.sqrt(D)
    ops.attention_prefill_mma(pg.qkv, pg.kpool, pg.vpool, tiles, pg.cu_q, pg.seg_pos0, pg.bt, P, out, Hq, Hkv, D,
                              scale, window or 0)
    assert torch.allclose(out.float().cpu(), pg.reference(scale, window), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("Hq,Hkv,D,P", [(8, 8, 64, 4), (32, 8, 128, 16), (6, 2, 128, 8), (20, 1, 64, 16), (4, 4, 128, 64)])
@pytest.mark.parametrize("window", [None, 37, 100])
@pytest.mark.parametrize("splits", [1, 2, 5])
def test_attention_prefill_tc5(Hq, Hkv, D, P, window, splits):
    """The tcgen05 prefill kernel: blocks of 256 rows (two tiles of 128), tails, earlier keys in the cache, windows;
    and the keys of every block split over several CTAs, some of which then have no keys at all, or keys
    for the later rows only."""
    ops = _ops()
    kv_lens, q_lens = [2, 70, 200, 128, 129, 300, 640], [2, 70, 3, 128, 65, 130, 300]
    pg = Paged(kv_lens, q_lens, Hq, Hkv, D, P, torch.bfloat16, seed=D + 5)
    tiles = [(i, r0) for i, ql in enumerate(q_lens) for r0 in range(0, ql, ops.TC5_TILE_ROWS)]
    tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    out = torch.full((sum(q_lens), Hq * D), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 0.7 / math.sqrt(D)
    ops.attention_prefill_tc5(pg.qkv, pg.kpool, pg.vpool, tiles, pg.cu_q, pg.seg_pos0, pg.bt, P, out, Hq, Hkv, D,
                              scale, window or 0, num_splits=splits)
    torch.cuda.synchronize()
    st = ops.tc5_status(torch.device(DEV))
    flag = int(st.item())
    st.zero_()
    assert flag == 0, "a bounded wait inside the kernel gave up"
    assert torch.allclose(out.float().cpu(), pg.reference(scale, window), atol=3e-2, rtol=3e-2)


def test_prefill_split_choice():
    """Keys are split only while blocks x heads leave SMs idle and every share keeps enough keys."""
    ops = _ops()
    assert ops.prefill_splits(256, 8192) == 1 and ops.prefill_splits(100, 8192) == 1
    assert ops.prefill_splits(64, 4096) == 2 and ops.prefill_splits(32, 4096) == 4
    assert ops.prefill_splits(32, 1024) == 2 and ops.prefill_splits(32, 600) == 1 and ops.prefill_splits(2, 100000) == 64


@pytest.mark.parametrize("Hq,Hkv,D,P", ATT_SHAPES)
@pytest.mark.parametrize("window,rot_frac,norm", [(None, 1.0, True), (37, 0.5, True), (None, 1.0, False)])
def test_attention_decode_fused(Hq, Hkv, D, P, window, rot_frac, norm):
    """Norm, rotation, cache write and attention of single tokens in one kernel, against the two kernels
    it stands for; the new token's key and value must land in the cache bit for bit."""
    import types
    ops = _ops()
    kv_lens = [1, 70, 200, 16, 129, 511, 17, 64]
    n = len(kv_lens)
    pg = Paged(kv_lens, [1] * n, Hq, Hkv, D, P, torch.bfloat16, seed=D + 9)
    g = torch.Generator().manual_seed(5)
    raw = torch.randn(n, (Hq + 2 * Hkv) * D, generator=g).bfloat16().to(DEV)
    rot = int(D * rot_frac) // 4 * 4
    pos_max = max(kv_lens)
    inv = 1.0 / (10000.0 ** (torch.arange(rot // 2, dtype=torch.float32) / max(rot // 2, 1)))
    ang = torch.arange(pos_max, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous().to(DEV), ang.sin().contiguous().to(DEV)
    qw = (1 + 0.1 * torch.randn(D, generator=g)).to(DEV) if norm else None
    kw = (1 + 0.1 * torch.randn(D, generator=g)).to(DEV) if norm else None
    scale = 0.7 / math.sqrt(D)
    segs = torch.arange(n, dtype=torch.int32, device=DEV)
    # the last token of every request is not in the cache yet: poison its slot
    k0, v0 = pg.kpool.clone(), pg.vpool.clone()
    for i, L in enumerate(kv_lens):
        page, row = int(pg.bt[i, (L - 1) // P]), (L - 1) % P
        k0[page, :, row] = float("nan")
        v0[page, :, row] = float("nan")
    # the two kernels
    k1, v1, q1 = k0.clone(), v0.clone(), raw.clone()
    ops.qk_norm_rope_write(q1, qw, kw, 1e-6, cos, sin, rot, pg.pos, pg.tok_seg, pg.bt, P, k1, v1, Hq, Hkv, D)
    want = torch.empty(n, Hq * D, device=DEV, dtype=torch.bfloat16)
    ops.attention_decode_mma(q1, k1, v1, segs, pg.cu_q, pg.seg_kv_len, pg.bt, P, want, Hq, Hkv, D, scale, window or 0,
                             num_splits=3)
    # the one kernel
    host = types.SimpleNamespace(decode_segs=segs.cpu().numpy(), seg_kv_len=pg.seg_kv_len.cpu().numpy(), num_tokens=n,
                                 num_multi=0)
    batch = types.SimpleNamespace(decode_segs=segs, cu_q=pg.cu_q, seg_kv_len=pg.seg_kv_len, host=host,
                                  variant={ops.decode_splits_key(Hq, Hkv, window): 3})
    k2, v2, q2 = k0.clone(), v0.clone(), raw.clone()
    got = torch.full_like(want, float("nan"))
    ops.attention_decode_fused(q2, qw, kw, 1e-6, 0.0, cos, sin, rot, k2, v2, batch, pg.bt, P, got, Hq, Hkv, D, scale, window)
    assert torch.equal(q2, raw)
    assert torch.equal(torch.nan_to_num(k2, nan=7.0), torch.nan_to_num(k1, nan=7.0))
    assert torch.equal(torch.nan_to_num(v2, nan=7.0), torch.nan_to_num(v1, nan=7.0))
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("splits", [1, 3])
def test_attention_prefill_tc5_long(D, splits):
    """Dozens of key tiles per query tile with every SM busy: the loaders, the issuing thread and the
    softmax rows drift apart in time, which is where a barrier that is waited on out of step shows.
    One far key is made to stand out for one late query, so a lost or misplaced tile shows too."""
    ops = _ops()
    Hq, Hkv, P, L = 4, 1, 16, 5000
    pg = Paged([L, 700], [L, 300], Hq, Hkv, D, P, torch.bfloat16, seed=11)
    far, late = 37, L - 3
    page, off = int(pg.bt[0, far // P]), far % P
    pg.k[0][far] *= 6.0
    pg.kpool[page, :, off] = pg.k[0][far].to(torch.bfloat16).to(DEV)
    pg.q[0][late] = pg.k[0][far, 0].repeat(Hq, 1) * 0.5
    pg.qkv[late, :Hq * D] = pg.q[0][late].reshape(-1).to(torch.bfloat16).to(DEV)
    tiles = [(i, r0) for i, ql in enumerate(pg.q_lens) for r0 in range(0, ql, ops.TC5_TILE_ROWS)]
    tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    out = torch.full((sum(pg.q_lens), Hq * D), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    for _ in range(3):
        ops.attention_prefill_tc5(pg.qkv, pg.kpool, pg.vpool, tiles, pg.cu_q, pg.seg_pos0, pg.bt, P, out, Hq, Hkv, D,
                                  scale, 0, num_splits=splits)
    torch.cuda.synchronize()
    st = ops.tc5_status(torch.device(DEV))
    flag = int(st.item())
    st.zero_()
    assert flag == 0, "a bounded wait inside the kernel gave up"
    ref = pg.reference(scale, None)
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=3e-2)
    # the late query's output is the far key's value, almost alone
    assert torch.allclose(out[late].float().cpu().reshape(Hq, D), pg.v[0][far, 0].to(torch.bfloat16).float().expand(Hq, D),
                          atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("Hq,Hkv,D,P", ATT_SHAPES)
@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_attention_decode_mma(Hq, Hkv, D, P, window, splits):
    ops = _ops()
    kv_lens = [1, 70, 200, 16, 129, 511, 17]
    pg = Paged(kv_lens, [1] * len(kv_lens), Hq, Hkv, D, P, torch.bfloat16, seed=D + 2)
    segs = torch.arange(len(kv_lens), dtype=torch.int32, device=DEV)
    out = torch.full((len(kv_lens), Hq * D), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 0.7 / math.sqrt(D)
    ops.attention_decode_mma(pg.qkv, pg.kpool, pg.vpool, segs, pg.cu_q, pg.seg_kv_len, pg.bt, P, out, Hq, Hkv, D,
                             scale, window or 0, num_splits=splits)
    assert torch.allclose(out.float().cpu(), pg.reference(scale, window), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_far_key_among_hundreds_and_the_windows_edge(dtype):
    """Random keys would hide a wrong page or an off-by-one at the window's edge; here one key's score
    stands out, so the output must be (almost exactly) that key's value."""
    ops = _ops()
    Hq, Hkv, D, P = 4, 2, 32, 16
    L, W = 777, 200
    for target, window, visible in ((5, None, True), (L - 1, None, True), (L - W, W, True), (L - W - 1, W, False),
                                    (431, None, True)):
        for q_len in (1, 3):
            pg = Paged([L], [q_len], Hq, Hkv, D, P, dtype, seed=target)
            # every query head points along the target key of its kv head, strongly
            k_t = pg.k[0][target]                                     # [Hkv, D]
            q = (30.0 * k_t / k_t.norm(dim=-1, keepdim=True)).repeat_interleave(Hq // Hkv, 0)
            pg.qkv[:, :Hq * D] = q.reshape(1, -1).to(dtype).to(DEV)
            pg.q = [q.unsqueeze(0).expand(q_len, Hq, D).contiguous()]
            scale = 1.0
            want = pg.reference(scale, window)
            last_row_sees = visible
            outs = []
            o = torch.empty(q_len, Hq * D, device=DEV, dtype=dtype)
            ops.attention_simt(pg.qkv, pg.kpool, pg.vpool, pg.pos, pg.tok_seg, pg.bt, P, o, Hq, Hkv, D, scale, window or 0)
            outs.append(o)
            if dtype == torch.bfloat16:
                o2 = torch.empty_like(o)
                if q_len == 1:
                    ops.attention_decode_mma(pg.qkv, pg.kpool, pg.vpool, torch.zeros(1, dtype=torch.int32, device=DEV),
                                             pg.cu_q, pg.seg_kv_len, pg.bt, P, o2, Hq, Hkv, D, scale, window or 0, num_splits=5)
                else:
                    ops.attention_prefill_mma(pg.qkv, pg.kpool, pg.vpool, torch.tensor([[0, 0]], dtype=torch.int32, device=DEV),
                                              pg.cu_q, pg.seg_pos0, pg.bt, P, o2, Hq, Hkv, D, scale, window or 0)
                outs.append(o2)
            v_t = pg.v[0][target].repeat_interleave(Hq // Hkv, 0).reshape(-1)
            for o in outs:
                assert torch.allclose(o.float().cpu(), want, **_tol(dtype))
                close = torch.allclose(o[-1].float().cpu(), v_t.to(dtype).float(), atol=5e-2)
                assert close == last_row_sees


def _attention_all_kernels(ops, pg, Hq, Hkv, D, P, scale, window, dtype):
    """The outputs of every attention kernel that takes this case: name -> [T, Hq*D] float32 on the CPU."""
    T = sum(pg.q_lens)
    outs = {}
    o = torch.empty(T, Hq * D, device=DEV, dtype=dtype)
    ops.attention_simt(pg.qkv, pg.kpool, pg.vpool, pg.pos, pg.tok_seg, pg.bt, P, o, Hq, Hkv, D, scale, window or 0)
    outs["simt"] = o.float().cpu()
    if dtype != torch.bfloat16:
        return outs
    if all(q == 1 for q in pg.q_lens):
        segs = torch.arange(pg.n, dtype=torch.int32, device=DEV)
        for splits in (1, 4):
            o = torch.full((T, Hq * D), float("nan"), device=DEV, dtype=dtype)
            ops.attention_decode_mma(pg.qkv, pg.kpool, pg.vpool, segs, pg.cu_q, pg.seg_kv_len, pg.bt, P, o, Hq, Hkv, D, scale,
                                     window or 0, num_splits=splits)
            outs[f"decode_mma/{splits}"] = o.float().cpu()
    else:
        tiles = torch.tensor([(i, r0) for i, ql in enumerate(pg.q_lens) for r0 in range(0, ql, 64)], dtype=torch.int32, device=DEV)
        o = torch.full((T, Hq * D), float("nan"), device=DEV, dtype=dtype)
        ops.attention_prefill_mma(pg.qkv, pg.kpool, pg.vpool, tiles, pg.cu_q, pg.seg_pos0, pg.bt, P, o, Hq, Hkv, D, scale, window or 0)
        outs["prefill_mma"] = o.float().cpu()
        if D in ops.TC5_ATTENTION_HEAD_DIMS:
            tiles = torch.tensor([(i, r0) for i, ql in enumerate(pg.q_lens) for r0 in range(0, ql, ops.TC5_TILE_ROWS)],
                                 dtype=torch.int32, device=DEV)
            o = torch.full((T, Hq * D), float("nan"), device=DEV, dtype=dtype)
            ops.attention_prefill_tc5(pg.qkv, pg.kpool, pg.vpool, tiles, pg.cu_q, pg.seg_pos0, pg.bt, P, o, Hq, Hkv, D, scale, window or 0)
            torch.cuda.synchronize()
            st = ops.tc5_status(torch.device(DEV))
            assert int(st.item()) == 0
            outs["prefill_tc5"] = o.float().cpu()
    return outs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_len", [1, 200])
@pytest.mark.parametrize("D,P", [(64, 16), (128, 8)])
def test_one_far_key_stands_out_and_the_windows_edge_is_exact(dtype, q_len, D, P):
    """Random keys hide a lost tile or an edge that is off by one.  Here one key far back is made to
    dominate the last query (no window), and with a window the key just inside it dominates while the
    key just outside it, made as strong, must leave no trace."""
    ops = _ops()
    Hq, Hkv, L = 4, 2, 700
    scale = 1.0 / math.sqrt(D)
    for window, strong, silent in ((None, 5, None), (37, L - 37, L - 38)):
        pg = Paged([L], [q_len], Hq, Hkv, D, P, dtype, seed=3, poison=False)
        last = q_len - 1                                   # the last query: position L - 1

        def put_key(j, vec):
            page, off = int(pg.bt[0, j // P]), j % P
            pg.k[0][j] = vec
            pg.kpool[page, :, off] = vec.to(dtype).to(DEV)

        direction = torch.randn(D, generator=torch.Generator().manual_seed(9))
        direction = direction / direction.norm() * 12.0
        put_key(strong, direction.expand(Hkv, D).clone())
        if silent is not None:
            put_key(silent, (1.5 * direction).expand(Hkv, D).clone())      # stronger still, but outside the window
        pg.q[0][last] = direction.expand(Hq, D) * 1.2
        pg.qkv[last, :Hq * D] = pg.q[0][last].reshape(-1).to(dtype).to(DEV)
        ref = pg.reference(scale, window)
        want_v = pg.v[0][strong].to(dtype).float()                          # [Hkv, D]
        for name, got in _attention_all_kernels(ops, pg, Hq, Hkv, D, P, scale, window, dtype).items():
            tol = dict(atol=2e-4, rtol=2e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
            assert torch.allclose(got, ref, **tol), (name, window)
            row = got[last].reshape(Hq, D)
            for h in range(Hq):                                             # the output is the strong key's value, almost alone
                assert torch.allclose(row[h], want_v[h // (Hq // Hkv)], atol=6e-2, rtol=6e-2), (name, window, h)


# ------------------------------------------------------------------------------- rope + cache write

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,P,rot", [(4, 2, 16, 16, 16), (6, 3, 32, 8, 32), (5, 1, 48, 16, 48), (3, 1, 80, 4, 32),
                                             (32, 8, 128, 16, 128), (6, 2, 64, 8, 64), (3, 1, 256, 16, 256), (9, 3, 128, 16, 64)])
@pytest.mark.parametrize("with_norm", [True, False])
@pytest.mark.parametrize("long_first", [20, 1200, 3000])  # many tokens take the forms with several heads a warp (16-byte pieces
                                                          # for bfloat16 heads of 64, 128, 256 rotated over their whole width)
def test_qk_norm_rope_write(dtype, Hq, Hkv, D, P, rot, with_norm, long_first):
    ops = _ops()
    g = torch.Generator().manual_seed(D)
    starts, lens = [0, 37, 5], [long_first, 1, 9]
    T = sum(lens)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g).to(dtype)
    qw = (1 + 0.1 * torch.randn(D, generator=g)) if with_norm else None
    kw = (1 + 0.1 * torch.randn(D, generator=g)) if with_norm else None
    eps, theta = 2e-5, 5000.0
    half = rot // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32) / half))
    ang = torch.outer(torch.arange(max(64, long_first + 8), dtype=torch.float32), inv)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.tensor([s + i for s, L in zip(starts, lens) for i in range(L)], dtype=torch.int32)
    tok_seg = torch.tensor([i for i, L in enumerate(lens) for _ in range(L)], dtype=torch.int32)
    n_blocks = [(s + L + P - 1) // P for s, L in zip(starts, lens)]
    perm = torch.randperm(sum(n_blocks) + 2, generator=g).tolist()
    bt = torch.full((3, max(n_blocks)), -1, dtype=torch.int32)
    it = iter(perm)
    for i, nb in enumerate(n_blocks):
        for b in range(nb):
            bt[i, b] = next(it)
    n_pages = sum(n_blocks) + 2
    kpool = torch.full((n_pages, Hkv, P, D), float("nan"), dtype=dtype, device=DEV)
    vpool = torch.full((n_pages, Hkv, P, D), float("nan"), dtype=dtype, device=DEV)
    dev_qkv = qkv.clone().to(DEV)
    ops.qk_norm_rope_write(dev_qkv, qw.to(DEV) if with_norm else None, kw.to(DEV) if with_norm else None, eps,
                           cos.to(DEV), sin.to(DEV), rot, pos.to(DEV), tok_seg.to(DEV), bt.to(DEV), P, kpool, vpool,
                           Hq, Hkv, D)

    def norm_rot(x, w):                 # x [T, heads, D] float32
        if w is not None:
            x = plain.rms_norm(x, w, eps)
        c, s = cos[pos.long()][:, None, :], sin[pos.long()][:, None, :]
        x1, x2 = x[..., :half], x[..., half:rot]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, x[..., rot:]], -1)

    x = qkv.float()
    q_ref = norm_rot(x[:, :Hq * D].view(T, Hq, D), qw)
    k_ref = norm_rot(x[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D), kw)
    v_ref = x[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    tol = _tol(dtype)
    assert torch.allclose(dev_qkv[:, :Hq * D].float().cpu().view(T, Hq, D), q_ref, **tol)
    written = torch.zeros(n_pages, P, dtype=torch.bool)
    for t in range(T):
        page, row = int(bt[tok_seg[t], pos[t] // P]), int(pos[t]) % P
        written[page, row] = True
        assert torch.allclose(kpool[page, :, row].float().cpu(), k_ref[t], **tol)
        assert torch.equal(vpool[page, :, row].float().cpu(), v_ref[t])
    # nothing else was touched
    assert torch.isnan(kpool.float().cpu()[~written[:, None, :].expand(-1, Hkv, -1)]).all()
    # without a cache write, k is normed and rotated in place and the pools stay as they are
    dev2 = qkv.clone().to(DEV)
    kp2 = torch.full_like(kpool, float("nan"))
    ops.qk_norm_rope_write(dev2, qw.to(DEV) if with_norm else None, kw.to(DEV) if with_norm else None, eps,
                           cos.to(DEV), sin.to(DEV), rot, pos.to(DEV), tok_seg.to(DEV), bt.to(DEV), P, kp2, kp2,
                           Hq, Hkv, D, write_kv=False)
    assert torch.isnan(kp2.float()).all()
    assert torch.allclose(dev2[:, Hq * D:(Hq + Hkv) * D].float().cpu().view(T, Hkv, D), k_ref, **tol)


# ------------------------------------------------------------------------------- sampling

def test_argmax_and_greedy_rows():
    ops = _ops()
    V = 1531
    logits = torch.randn(9, V, device=DEV)
    logits[3, 77] = logits[3, 900] = 50.0                       # a tie: the lowest index wins
    toks = torch.empty(9, dtype=torch.int32, device=DEV)
    ops.argmax(logits, toks)
    want = logits.argmax(-1)
    want[3] = 77
    assert torch.equal(toks.long(), want)
    temp = torch.zeros(9, device=DEV)
    toks2 = torch.empty_like(toks)
    lp = torch.empty(9, device=DEV)
    ops.sample(logits, temp, torch.zeros(9, dtype=torch.int32, device=DEV), torch.ones(9, device=DEV),
               torch.rand(9, device=DEV), toks2, lp)
    assert torch.equal(toks2, toks)
    ref_lp = torch.log_softmax(logits.double(), -1).gather(1, want[:, None])[:, 0]
    assert torch.allclose(lp.double(), ref_lp, atol=1e-4)


@pytest.mark.parametrize("V", [50, 1000, 151936])
def test_sample_matches_the_filtered_distribution(V):
    """The chosen token is the one whose interval of the kept distribution's CDF (vocabulary order) holds u."""
    ops = _ops()
    g = torch.Generator().manual_seed(V)
    n = 24
    logits = (2.5 * torch.randn(n, V, generator=g))
    temps = [0.8, 1.0, 1.3, 0.5] * 6
    top_ks = [0, 0, 5, 40, 0, 1, 0, 3] * 3
    top_ps = [1.0, 0.9, 1.0, 0.7, 0.3, 1.0, 0.05, 0.95] * 3
    u = torch.rand(n, generator=g)
    toks = torch.empty(n, dtype=torch.int32, device=DEV)
    lp = torch.empty(n, device=DEV)
    ops.sample(logits.to(DEV), torch.tensor(temps, device=DEV), torch.tensor(top_ks, dtype=torch.int32, device=DEV),
               torch.tensor(top_ps, device=DEV), u.to(DEV), toks, lp)
    for i in range(n):
        probs = plain.filtered_probs(logits[i], temps[i], top_ks[i], top_ps[i])
        tok = int(toks[i])
        assert probs[tok] > 0, f"row {i}: token {tok} is outside the kept set"
        cdf = probs.cumsum(0)
        lo = float(cdf[tok] - probs[tok])
        assert lo - 1e-4 <= float(u[i]) <= float(cdf[tok]) + 1e-4, (i, tok, lo, float(u[i]), float(cdf[tok]))
        assert abs(float(lp[i]) - plain.logprob(logits[i], tok)) < 1e-3


@pytest.mark.parametrize("V", [7, 50, 4099, 151936, 262144])
def test_sample_by_a_cluster_and_by_one_cta_choose_the_same_tokens(V):
    """The kernel that spreads a row over the shared memories of eight CTAs against its twin with one CTA a row:
    greedy rows, temperature, top-k and top-p, with ties.  Masses are float32 sums in the one and exact fixed-point
    sums in the other, so a draw that falls on the edge between two tokens may go either way: at most one row in
    forty may differ, and then by a neighbour in the kept set."""
    ops = _ops()
    g = torch.Generator().manual_seed(V)
    n = 40
    for trial in range(3):
        logits = (2.5 * torch.randn(n, V, generator=g)).to(DEV)
        if trial == 2:
            logits[:, ::3] = logits[:, 1:2]                        # many equal values
        temps = torch.tensor([0.8, 1.0, 1.3, 0.5, 0.0] * 8, device=DEV)
        ks = torch.tensor([0, 0, 5, 40, 0, 1, 0, 3] * 5, dtype=torch.int32, device=DEV)
        ps = torch.tensor([1.0, 0.9, 1.0, 0.7, 0.3, 1.0, 0.05, 0.95] * 5, device=DEV)
        u = torch.rand(n, generator=g).to(DEV)
        got = []
        for one_cta in (True, False):
            toks = torch.full((n,), -7, dtype=torch.int32, device=DEV)
            lp = torch.full((n,), float("nan"), device=DEV)
            ops.sample(logits, temps, ks, ps, u, toks, lp, one_cta=one_cta)
            got.append((toks.cpu(), lp.cpu()))
        same = got[0][0] == got[1][0]
        assert int((~same).sum()) <= 1, (trial, got[0][0][~same], got[1][0][~same])
        assert torch.allclose(got[0][1][same], got[1][1][same], atol=1e-5)
        assert (got[1][0] >= 0).all() and (got[1][0] < V).all()
        # again: the same bits
        toks2 = torch.empty(n, dtype=torch.int32, device=DEV)
        ops.sample(logits, temps, ks, ps, u, toks2, None)
        assert torch.equal(toks2.cpu(), got[1][0])


def test_sample_frequencies():
    ops = _ops()
    V, n = 12, 4000
    logits = torch.tensor([2.0, 1.5, 1.0, 0.5, 0.0, -0.5, -1.0, -1.5, -2.0, -2.5, -3.0, -9.0])
    probs = plain.filtered_probs(logits, 0.9, 6, 0.85)
    rows = logits.repeat(n, 1).to(DEV)
    toks = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(rows, torch.full((n,), 0.9, device=DEV), torch.full((n,), 6, dtype=torch.int32, device=DEV),
               torch.full((n,), 0.85, device=DEV), torch.rand(n, device=DEV), toks, None)
    freq = torch.bincount(toks.long().cpu(), minlength=V).double() / n
    assert (freq[probs == 0] == 0).all()
    assert (freq - probs).abs().max() < 0.03


# ------------------------------------------------------------------------------- norms and residual adds inside the products

def _weave8(gate, up):
    return torch.stack([gate.view(-1, 8, gate.shape[1]), up.view(-1, 8, up.shape[1])], dim=1).reshape(-1, gate.shape[1])


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("H,Q,I,wdt", [(96, 192, 224, torch.float32), (64, 64, 128, torch.bfloat16), (4096, 4096, 12288, torch.bfloat16)])
def test_gemm_skinny_fused_forms_of_a_block(M, H, Q, I, wdt):
    """(product + residual add) -> (gated product scaled by the norm's rstd) -> (product + residual add), then the
    next block's first product from what was left for its norm, as the block runs them for a step of few rows;
    against plain float32 math: stream, norms, SwiGLU and all."""
    ops = _ops()
    g = torch.Generator().manual_seed(H + M)
    rnd = lambda *s: torch.randn(*s, generator=g)
    stream0 = rnd(M, H)
    n2, n_next = (1 + 0.1 * rnd(H)).to(wdt), (1 + 0.1 * rnd(H)).to(wdt)
    o = rnd(M, Q).bfloat16()
    w_o = (rnd(H, Q) / math.sqrt(Q)).bfloat16()
    gate, up = (rnd(I, H) / math.sqrt(H)).bfloat16(), (rnd(I, H) / math.sqrt(H)).bfloat16()
    down = (rnd(H, I) / math.sqrt(I)).bfloat16()
    w_in = (rnd(Q + 32, H) / math.sqrt(H)).bfloat16()
    eps = 1e-5
    d = lambda t: t.to(DEV)
    nan = lambda *shape, dt=torch.bfloat16: torch.full(shape, float("nan"), dtype=dt, device=DEV)

    def run(stream):
        rows2, act, rows3, proj = nan(M, H), nan(M, I), nan(M, H), nan(M, Q + 32)
        sums2 = ops.RowSums(nan(8, ops.RowSums.WIDTH, dt=torch.float32), H)
        sums3 = ops.RowSums(nan(8, ops.RowSums.WIDTH, dt=torch.float32), H)
        ops.gemm_skinny_fused(d(o), d(w_o), rows2, residual=(stream, (d(n2), 0.0), sums2))
        ops.gemm_skinny_fused(rows2, d(_weave8(gate, up)), act, gated=True, scale=(sums2, eps))
        ops.gemm_skinny_fused(act, d(down), rows3, residual=(stream, (d(n_next), 0.0), sums3))
        ops.gemm_skinny_fused(rows3, d(w_in), proj, scale=(sums3, eps))
        return act, rows3, sums3, proj

    stream = d(stream0.clone())
    act, rows3, sums3, proj = run(stream)
    # plain
    s1 = stream0 + o.float() @ w_o.float().T
    a2 = plain.rms_norm(s1, n2.float(), eps)
    gg, uu = a2 @ gate.float().T, a2 @ up.float().T
    act_want = gg * torch.sigmoid(gg) * uu
    s2 = s1 + act_want @ down.float().T
    assert torch.allclose(act.float().cpu(), act_want, atol=3e-2 * max(1.0, float(act_want.abs().max())), rtol=3e-2)
    assert torch.allclose(stream.cpu(), s2, atol=2e-2 * max(1.0, float(s2.abs().max())), rtol=2e-2)
    # the sums left for the next norm are those of the stream as the kernel left it
    got_ssq = sums3.parts[:M, :sums3.count].sum(dim=1).cpu()
    assert torch.allclose(got_ssq, (stream.cpu() ** 2).sum(dim=1), rtol=1e-5)
    want = plain.rms_norm(stream.cpu(), n_next.float(), eps) @ w_in.float().T
    assert torch.allclose(proj.float().cpu(), want, atol=3e-2 * max(1.0, float(want.abs().max())), rtol=3e-2)
    # a last product with nothing behind it: only the stream
    only = d(stream0.clone())
    ops.gemm_skinny_fused(d(o), d(w_o), None, residual=(only, None, None))
    assert torch.allclose(only.cpu(), s1, atol=2e-2 * max(1.0, float(s1.abs().max())), rtol=2e-2)
    # again from the same start: nothing depends on timing
    stream_b = d(stream0.clone())
    act_b, rows3_b, _, proj_b = run(stream_b)
    assert torch.equal(stream_b, stream) and torch.equal(act_b, act) and torch.equal(rows3_b, rows3) and torch.equal(proj_b, proj)
