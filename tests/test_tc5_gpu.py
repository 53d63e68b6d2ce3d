"""The tcgen05 / TMA matrix product against plain math: first the one-stage twin that pins the
descriptor encodings down, then the pipelined kernel, at sizes with tails in every dimension."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from return_b200.ext import ops
    return ops


def _case(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16().to(DEV)
    return x, w, x.double() @ w.double().T


def _status_clear(ops):
    st = ops.tc5_status(torch.device(DEV))
    torch.cuda.synchronize()
    flag = int(st.item())
    st.zero_()
    return flag


@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (128, 256, 128), (100, 200, 72), (300, 520, 1000)])
def test_one_stage_twin(bn, M, N, K):
    ops = _ops()
    x, w, want = _case(M, N, K, M + N + K)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tc5(x, w, out, simple_bn=bn)
    assert _status_clear(ops) == 0, "a bounded wait inside the kernel gave up"
    assert (out.double() - want).abs().max() < 2e-3


@pytest.mark.parametrize("pair", [False, True], ids=["one_cta", "cta_pair"])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (33, 40, 72), (300, 520, 1000), (2048, 1024, 4096),
                                   (129, 257 * 8, 264), (257, 256, 136), (1100, 1288, 328)])
def test_pipelined_product(M, N, K, out_dtype, pair):
    """One 128 x 256 tile a CTA, and 256 x 256 tiles by pairs of CTAs (two-SM MMAs): tails in every dimension, more
    tiles than CTAs, fewer k blocks than stages."""
    ops = _ops()
    x, w, want = _case(M, N, K, M * 3 + N + K)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.gemm_tc5(x, w, out, pair=pair)
    assert _status_clear(ops) == 0, "a bounded wait inside the kernel gave up"
    tol = 2e-3 if out_dtype == torch.float32 else 3e-2
    assert (out.double() - want).abs().max() < tol


@pytest.mark.parametrize("pair", [False, True], ids=["one_cta", "cta_pair"])
@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (200, 104, 136), (512, 3072, 1024), (1030, 1192, 520)])
def test_pipelined_product_with_swiglu_epilogue(M, I, K, pair):
    ops = _ops()
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    gate = (torch.randn(I, K, generator=g) / K ** 0.5).bfloat16()
    up = (torch.randn(I, K, generator=g) / K ** 0.5).bfloat16()
    woven = torch.stack([gate.view(-1, 8, K), up.view(-1, 8, K)], dim=1).reshape(2 * I, K).contiguous().to(DEV)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc5(x, woven, out, gated=True, pair=pair)
    assert _status_clear(ops) == 0
    gg, uu = x.float().cpu() @ gate.float().T, x.float().cpu() @ up.float().T
    assert torch.allclose(out.float().cpu(), gg * torch.sigmoid(gg) * uu, atol=2e-2, rtol=3e-2)


# ------------------------------------------------------------------------------- the weight-streaming kernel

@pytest.mark.parametrize("M", [1, 3, 8, 16, 17, 32, 50, 64, 100, 128])
@pytest.mark.parametrize("N,K", [(16, 32), (100, 72), (384, 96), (1000, 4096), (4104, 1544)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_stream(M, N, K, out_dtype):
    ops = _ops()
    x, w, want = _case(M, N, K, M * 1000 + N)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.gemm_stream(x, w, out)
    assert _status_clear(ops) == 0, "a bounded wait inside the kernel gave up"
    tol = 2e-3 if out_dtype == torch.float32 else 2e-2
    assert (out.double() - want).abs().max() < tol
    # a second call gives the same bits
    out2 = torch.full_like(out, float("nan"))
    ops.gemm_stream(x, w, out2)
    assert _status_clear(ops) == 0
    assert torch.equal(out2, out)
    # a view with a row stride (the q part of a qkv buffer) works too
    big = torch.zeros(M, K + 64, dtype=torch.bfloat16, device=DEV)
    big[:, :K] = x
    out3 = torch.empty_like(out)
    ops.gemm_stream(big[:, :K], w, out3)
    assert torch.equal(out3, out)


@pytest.mark.parametrize("M", [2, 20, 70])
@pytest.mark.parametrize("rows_per_sm", [1, 15, 20, 40, 64, 127, 128, 129, 300])
def test_gemm_stream_ranges_and_chunks(M, rows_per_sm):
    """Ranges of rows_per_sm or one more row a CTA: one chunk, exactly 128 rows, and several chunks of
    unequal height."""
    ops = _ops()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    N, K = sms * rows_per_sm + 5, 200
    most, nchunk, tallest, parts = ops.gemm_stream_plan(M, N, K)
    assert most == rows_per_sm + 1 and tallest == -(-most // nchunk)
    assert (nchunk == (most + 127) // 128 and parts == 1) if most > 64 else (nchunk == 1 and parts > 1)
    x, w, want = _case(M, N, K, M)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_stream(x, w, out)
    assert _status_clear(ops) == 0
    assert (out.double() - want).abs().max() < 2e-3


@pytest.mark.parametrize("M", [1, 8, 13, 32, 50, 128])
@pytest.mark.parametrize("I,K", [(8, 32), (104, 40), (224, 96), (3072, 1024), (12288, 264)])
def test_gemm_stream_gated(M, I, K):
    ops = _ops()
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    gate = (torch.randn(I, K, generator=g) / K ** 0.5).bfloat16()
    up = (torch.randn(I, K, generator=g) / K ** 0.5).bfloat16()
    woven = torch.stack([gate.view(-1, 8, K), up.view(-1, 8, K)], dim=1).reshape(2 * I, K).contiguous().to(DEV)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_stream(x, woven, out, gated=True)
    assert _status_clear(ops) == 0
    gg, uu = x.float().cpu() @ gate.float().T, x.float().cpu() @ up.float().T
    assert torch.allclose(out.float().cpu(), gg * torch.sigmoid(gg) * uu, atol=2e-2, rtol=3e-2)


def test_the_pair_kernel_gives_the_same_bits_again_and_takes_a_view():
    """A second call gives the same bits (the order of the k blocks is fixed); x may be a view with a row stride."""
    ops = _ops()
    M, N, K = 777, 1544, 392
    x, w, want = _case(M, N, K, 11)
    a = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    b = torch.full_like(a, float("nan"))
    ops.gemm_tc5(x, w, a, pair=True)
    ops.gemm_tc5(x, w, b, pair=True)
    assert _status_clear(ops) == 0
    assert torch.equal(a, b) and (a.double() - want).abs().max() < 3e-2
    big = torch.zeros(M, K + 64, dtype=torch.bfloat16, device=DEV)
    big[:, :K] = x
    c = torch.empty_like(a)
    ops.gemm_tc5(big[:, :K], w, c, pair=True)
    assert _status_clear(ops) == 0 and torch.equal(c, a)


def test_gated_linear_takes_the_pair_kernel_for_many_rows():
    """``ops.gated_linear`` with the woven layout: the same numbers whichever kernel the row count selects."""
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    M, I, K = ops.PAIR_MIN_ROWS + 37, 520, 264
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(2 * I, K, generator=g) / K ** 0.5).bfloat16().to(DEV)
    many = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gated_linear(x, w, many, 8)
    assert _status_clear(ops) == 0
    few = torch.empty((100, I), dtype=torch.bfloat16, device=DEV)
    ops.gated_linear(x[:100], w, few, 8)                       # cuBLAS and the SwiGLU kernel
    assert torch.allclose(many[:100].float(), few.float(), atol=2e-2, rtol=3e-2)
    r = (x.float() @ w.float().T).view(M, I // 8, 2, 8)
    want = (torch.nn.functional.silu(r[:, :, 0]) * r[:, :, 1]).reshape(M, I)
    assert torch.allclose(many.float(), want, atol=2e-2, rtol=3e-2)


def test_cluster_kernels_replay_from_a_cuda_graph():
    """The kernels that launch as clusters (the pair product, the sampler) captured into a CUDA graph and replayed
    on new inputs in the same buffers."""
    ops = _ops()
    M, N, K, V = 800, 520, 264, 5000
    x, w, _ = _case(M, N, K, 3)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    logits = torch.empty((6, V), device=DEV)
    temp = torch.tensor([0.0, 1.0, 0.7, 1.2, 0.0, 0.9], device=DEV)
    top_k = torch.tensor([0, 0, 20, 0, 0, 5], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.5, 1.0, 1.0], device=DEV)
    u = torch.tensor([0.1, 0.5, 0.9, 0.3, 0.7, 0.2], device=DEV)
    toks = torch.empty(6, dtype=torch.int32, device=DEV)
    lps = torch.empty(6, device=DEV)
    ops.gemm_tc5(x, w, out, pair=True)                       # compiled and configured before the capture
    ops.sample(logits.normal_(), temp, top_k, top_p, u, toks, lps)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ops.gemm_tc5(x, w, out, pair=True)
        ops.sample(logits, temp, top_k, top_p, u, toks, lps)
    gen = torch.Generator(device=DEV).manual_seed(5)
    for _ in range(3):
        x.copy_(torch.randn(M, K, generator=gen, device=DEV))
        logits.copy_(3 * torch.randn(6, V, generator=gen, device=DEV))
        g.replay()
        torch.cuda.synchronize()
        assert _status_clear(ops) == 0
        assert (out.double() - x.double() @ w.double().T).abs().max() < 3e-2
        want = torch.empty_like(toks)
        ops.sample(logits, temp, top_k, top_p, u, want, None, one_cta=True)
        assert torch.equal(toks, want)
