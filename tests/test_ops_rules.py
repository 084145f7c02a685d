"""The rules by which the kernel wrappers size their grids and choose a product: pure
functions of the sizes, checked without a GPU."""
import torch

from tiny_llm_infer_b200 import ops


def test_decode_splits_give_enough_blocks_with_enough_keys_each():
    assert ops.decode_splits(8, 8, 4096) == 4            # about a thousand keys per block
    assert ops.decode_splits(1, 8, 4096) == 16           # few rows: at least 128 blocks in all
    assert ops.decode_splits(64, 8, 4096) == 4
    assert ops.decode_splits(1, 1, 100) == 1             # never less than 128 keys a block
    assert ops.decode_splits(1, 1, 1 << 20) == 64        # and never more than 64 blocks a row
    for rows in (1, 3, 8, 64):
        for ctx in (1, 17, 300, 5000):
            s = ops.decode_splits(rows, 2, ctx)
            assert 1 <= s <= 64 and (s == 1 or ctx / s >= 64)


def test_prefill_splits_fill_the_gpu_only_when_runs_stay_long():
    assert ops.prefill_splits(32, 256) == 1 and ops.prefill_splits(32, 1024) == 2
    assert ops.prefill_splits(32, 4096) == 4 and ops.prefill_splits(16, 8192) == 8
    assert ops.prefill_splits(64, 4096) == 2 and ops.prefill_splits(128, 65536) == 1
    for blocks in (1, 3, 40, 200):
        for ctx in (64, 1000, 40000):
            s = ops.prefill_splits(blocks, ctx)
            assert s in (1, 2, 4, 8) and (s == 1 or (blocks * s <= ops.SM_COUNT and -(-ctx // 64) // s >= 8))


def test_the_tcgen05_product_is_chosen_where_its_tiles_fill_the_gpu():
    bf = torch.bfloat16
    assert ops.tcgen05_pays(2048, 4096, 4096, bf) and ops.tcgen05_pays(2048, 12288, 4096, bf, col_tile=128)
    assert not ops.tcgen05_pays(2048, 6144, 4096, bf)            # 8 x 24 tiles: a ragged second round
    assert not ops.tcgen05_pays(64, 4096, 4096, bf) and not ops.tcgen05_pays(2048, 4096, 4096, torch.float32)
    assert not ops.tcgen05_pays(2048, 4096, 4100, bf)            # K no multiple of 8
