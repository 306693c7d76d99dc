"""The host-side plans of the kernel library (no GPU): how keys are cut into slices and K into splits."""
import pytest

from safetyraise_lmengine_b200.kernels.library import KernelLibrary


@pytest.mark.parametrize("n_entries", [1, 2, 3, 8, 17, 64, 300])
@pytest.mark.parametrize("nkv", [1, 2, 8])
@pytest.mark.parametrize("max_kv", [1, 63, 64, 65, 2083, 8192, 40000])
@pytest.mark.parametrize("cap", [8, 32])
def test_attention_split_covers_every_key_in_whole_tiles(n_entries, nkv, max_kv, cap):
    nsplit, chunk = KernelLibrary.attention_split(n_entries, nkv, max_kv, max_slices=cap)
    assert 1 <= nsplit <= cap
    assert chunk > 0 and chunk % 64 == 0
    assert nsplit * chunk >= max_kv                       # every key lies in a slice
    assert (nsplit - 1) * chunk < max(max_kv, 1) + 63     # and no slice is empty
    # within one wave of two blocks per SM, unless a single slice per pair is already more
    assert nsplit == 1 or n_entries * nkv * nsplit <= 296


@pytest.mark.parametrize("M", [1, 8, 9, 16, 17, 32, 33, 64, 65, 128, 129, 300, 512, 1024, 2048, 5000])
@pytest.mark.parametrize("N, K", [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288), (151936, 4096),
                                  (200, 72), (128, 64), (1024, 25600)])
def test_gemm_splits_keeps_its_bounds(M, N, K):
    sp = KernelLibrary.gemm_splits(M, N, K)
    total_kb = (K + 63) // 64
    assert 1 <= sp <= max(1, total_kb)
    if sp > 1:
        assert total_kb // sp >= 4                        # a split keeps at least a few k-blocks
    bn = KernelLibrary.gemm_token_tile(M, N)
    if bn == 256:
        assert sp == 1                                    # pairs of SMs on whole tiles of 256 x 256
    assert KernelLibrary.gemm_token_tile(512, 5120) == 256 and KernelLibrary.gemm_token_tile(512, 4096) == 128
    assert KernelLibrary.gemm_token_tile(2048, 4096) == 256 and KernelLibrary.gemm_token_tile(300, 5120) == 128
    if sp > 8:                                            # beyond a cluster: the partial sums fit the workspace
        tiles = ((N + 127) // 128) * ((M + bn - 1) // bn)
        assert 65536 + sp * tiles * 128 * bn * 4 <= KernelLibrary.GEMM_WS_BYTES


def test_prefill_attention_plan():
    plan = KernelLibrary.prefill_attention_plan
    # a whole prompt of 2,048 tokens, 4 heads per KV head, 8 KV heads: enough blocks of two row tiles, no slices
    assert plan([8192], [2048], 8, 148) == (2, 1, 0)
    # a portion of 512 tokens behind 30,000: 64 blocks of two row tiles; the keys go in slices of whole tiles
    tiles, nsplit, chunk = plan([2048], [30512], 8, 148)
    assert tiles == 2 and nsplit >= 2 and chunk % 128 == 0 and nsplit * chunk >= 30512 > (nsplit - 1) * chunk
    # 152 lone row tiles would need two rounds of the GPU, 80 blocks of two tiles one: two tiles, no slices
    assert plan([2405], [1505], 8, 148) == (2, 1, 0)
    # a handful of rows and keys: nothing to cut
    assert plan([5], [100], 1, 148)[1:] == (1, 0)
    for rows, kv, nkv in (([1, 4000], [9000, 4000], 2), ([300] * 40, [5000] * 40, 8), ([128], [257], 1)):
        tiles, nsplit, chunk = plan(rows, kv, nkv, 148)
        assert tiles in (1, 2) and 1 <= nsplit <= 16
        if nsplit > 1:
            assert tiles == 2 and chunk % 128 == 0 and nsplit * chunk >= max(kv) > (nsplit - 1) * chunk - 128
