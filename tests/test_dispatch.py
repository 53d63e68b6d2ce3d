"""The choices the engine makes on the host before it launches anything: how many ways keys are split,
which graph a decode step runs in.  Pure functions, no GPU."""
import pytest


def test_decode_graph_batch_sizes():
    from return_b200.engine.runner import graph_batch_size
    assert [graph_batch_size(m, 64) for m in range(1, 10)] == [1, 2, 3, 4, 5, 6, 7, 8, 12]
    assert [graph_batch_size(m, 64) for m in (12, 13, 16, 17, 24, 25, 33, 48, 49, 64)] == [12, 16, 16, 24, 24, 32, 48, 48, 64, 64]
    assert graph_batch_size(9, 10) == 10 and graph_batch_size(10, 10) == 10          # never beyond max_reside
    sizes = {graph_batch_size(m, 256) for m in range(1, 257)}
    assert len(sizes) <= 20 and all(graph_batch_size(m, 256) >= m for m in range(1, 257))
    # padding stays under half of the step
    assert all(graph_batch_size(m, 256) < 1.5 * m + 1 for m in range(9, 257))


def test_prefill_key_splits():
    """Keys are split only while blocks x heads leave SMs idle and every share keeps enough keys."""
    from return_b200.ext import ops
    assert ops.prefill_splits(256, 8192) == 1 and ops.prefill_splits(100, 8192) == 1
    assert ops.prefill_splits(64, 4096) == 2 and ops.prefill_splits(32, 4096) == 4
    assert ops.prefill_splits(32, 1024) == 2 and ops.prefill_splits(32, 600) == 1 and ops.prefill_splits(2, 100000) == 64
    for ctas in range(1, 300):
        for keys in (100, 700, 5000, 70000):
            s = ops.prefill_splits(ctas, keys)
            assert 1 <= s <= 64 and (s == 1 or (s * ctas <= ops.num_sms() and keys // s >= ops.PREFILL_SPLIT_MIN_KEYS))


def test_decode_key_splits():
    from return_b200.ext import ops
    for base in (1, 8, 64, 296, 512, 2000):
        for keys in (1, 100, 2048, 40000):
            s = ops.decode_splits(base, keys)
            assert 1 <= s <= 64
            assert s == 1 or (keys + s - 1) // s >= 128            # a share keeps at least 128 keys
    assert ops.decode_splits(512, 2048) == 1                      # more CTAs than the GPU holds at once: no split
    assert ops.decode_splits(8, 32768) > ops.decode_splits(8, 2048) >= 2


def test_profile_buckets_know_the_engines_kernels():
    from return_b200 import benchmark
    names = {"void (anonymous namespace)::gemm_skinny_kernel<1, __nv_bfloat16, 0, 2>(...)": "gemm/matmul",
             "nvjet_tst_64x32_64x8_4x1_v_bz_TNT": "gemm/matmul",
             "void (anonymous namespace)::attn_decode_kernel<true>(...)": "decode_attn",
             "(anonymous namespace)::attn_combine_kernel(...)": "decode_attn",
             "attn_prefill_tc5_kernel": "prefill_attn",
             "void add_rmsnorm_vec_kernel<__nv_bfloat16, __nv_bfloat16, 4>(...)": "rmsnorm",
             "void qk_norm_rope_write_vec_kernel<8>(...)": "rope",
             "void swiglu_bf16x8_kernel(...)": "elementwise",
             "void sample_kernel(...)": "softmax/sample", "something_else": "other"}
    for kernel, want in names.items():
        assert benchmark.profile_bucket(kernel) == want, kernel
