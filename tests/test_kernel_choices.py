"""The host-side rules that choose kernels and launch shapes (no GPU needed)."""

import itertools

from llm_runtime_study_b200.ops import attention_bf16, gemm_bf16


def test_projection_kernel_choice_is_always_something_the_library_builds():
    for m, n, k in itertools.product((1, 17, 128, 129, 255, 256, 300, 512, 1000, 2048, 8192),
                                     (8, 264, 4096, 6144, 24576, 151936), (8, 72, 4096, 12288)):
        kernel, width = gemm_bf16.pick_kernel(m, n, k)
        assert kernel in gemm_bf16.KERNELS and width in (0, 128, 256)
        assert width == 256 or kernel == ("splitk" if width == 0 else "persistent")   # split-K chooses its own width
        if kernel == "pair":
            assert m >= gemm_bf16.PAIR_MIN_ROWS
        if kernel == "streamk":
            assert k >= 3072                                   # a K range long enough to share


def test_projection_kernel_choice_at_the_benchmark_shapes():
    layer = ((6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288))
    assert all(gemm_bf16.pick_kernel(2048, n, k) == ("pair", 256) for n, k in layer)
    assert gemm_bf16.pick_kernel(512, 4096, 4096) == ("persistent", 128)
    assert gemm_bf16.pick_kernel(256, 4096, 12288) == ("splitk", 0)
    assert gemm_bf16.pick_kernel(384, 4096, 12288) == ("streamk", 256)


def test_decode_parts_are_bounded_and_use_the_gpu():
    for requests, kv_heads, longest, slots in itertools.product((1, 3, 8, 64, 500), (1, 8), (1, 100, 2048, 32768, 1 << 20), (296, 592)):
        parts = attention_bf16.decode_splits(requests, kv_heads, 1, longest, slots)
        assert 1 <= parts <= 64
        assert parts == 1 or longest // parts >= 64            # a part is never shorter than a few key blocks
    # one long sequence is cut into many parts, a full batch into none
    assert attention_bf16.decode_splits(1, 8, 1, 32768, 296) >= 16
    assert attention_bf16.decode_splits(64, 8, 1, 2048, 592) == 1
    assert attention_bf16.decode_splits(8, 8, 1, 2048, 296) == 4


def test_tile_map_orders_tiles_longest_first():
    table, count = attention_bf16.tile_map([5, 70, 1], 32, "cpu", kv_lens=[300, 70, 900])
    rows = table.t().tolist()                                    # [entry, first token, count]
    assert count == 5 and sorted(r[0] for r in rows) == [0, 1, 1, 1, 2]
    assert rows[0] == [2, 75, 1] and rows[1] == [0, 0, 5]        # 900 keys, then 300, then the 70-token prompt's tiles
    assert [r[2] for r in rows if r[0] == 1] == [6, 32, 32]      # its last tile (6 tokens, 70 keys) before the earlier ones


def test_few_rows_go_to_the_streaming_kernel_unless_the_weights_are_large():
    assert all(gemm_bf16.few_rows_kernel(m, 24576, 4096) == "skinny" for m in (1, 8))
    assert gemm_bf16.few_rows_kernel(1, 5120, 25600) == "splitk" and gemm_bf16.few_rows_kernel(8, 4096, 12288) == "skinny"
    assert gemm_bf16.few_rows_kernel(16, 24576, 4096) == "splitk" and gemm_bf16.few_rows_kernel(9, 51200, 5120) == "splitk"
    assert gemm_bf16.few_rows_kernel(16, 4096, 12288) == "skinny" and gemm_bf16.few_rows_kernel(16, 4096, 4096) == "skinny"


def test_split_k_shape_fills_the_sms_and_keeps_tiles_wide():
    """The width and cluster size the split-K kernel picks by itself (host arithmetic in the library)."""

    shape = gemm_bf16.splitk_shape
    assert shape(64, 4096, 4096) == (128, 4)           # 32 tiles x 4 = 128 CTAs on 148 SMs
    assert shape(16, 24576, 4096) == (192, 1)          # 128 tiles, nothing to share
    assert shape(16, 151936, 4096) == (224, 1)         # 679 tiles: 4.6 rounds of wide tiles, not 10.7 of narrow ones
    assert shape(200, 4096, 12288) == (256, 4)         # two row tiles: 32 wide tiles x 4 rather than 64 narrow ones x 2
    assert shape(8, 24, 64) == (256, 1)                # one K block cannot be shared
    for n, k in ((5120, 25600), (10240, 5120), (1000, 520), (7168, 5120)):
        width, splits = shape(16, n, k)
        assert width % 32 == 0 and 96 <= width <= 256 and splits in (1, 2, 4)
        assert -(-n // width) * splits <= 148 or splits == 1
        assert shape(128, n, k) == (width, splits)     # the choice does not depend on the rows that came along
