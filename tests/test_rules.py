"""Host-side rules of the kernels' launches: how many splits a decoding attention takes, how many slices of K the
tcgen05 product takes, and how a mixed step's sequences are divided between the two attention kernels.  No GPU."""
from types import SimpleNamespace

import pytest


@pytest.fixture()
def ops(monkeypatch):
    from rust_mlx_b200.kernels import ops as module
    monkeypatch.setattr(module, "_SM_COUNT", 148)
    return module


def test_decoding_attention_splits(ops):
    # batch size -> splits at 8 kv heads for contexts of 256, 2,048, 8,192, 32,768 and 131,072 tokens
    want = {1: [2, 8, 8, 32, 32], 2: [2, 8, 8, 8, 8], 3: [2, 8, 8, 8, 8], 4: [2, 4, 4, 4, 4], 6: [2, 4, 4, 4, 4],
            8: [2, 4, 4, 4, 4], 12: [2, 2, 2, 2, 2], 16: [2, 2, 2, 2, 2], 32: [1, 1, 1, 1, 1], 64: [1, 1, 1, 1, 1]}
    for batch, row in want.items():
        assert [ops.flash_splits(batch, 8, ctx) for ctx in (256, 2048, 8192, 32768, 131072)] == row, batch
    assert ops.flash_splits(1, 8, 100) == 1          # under four key tiles there is nothing to share
    for batch in range(1, 200):
        for ctx in (64, 1000, 5000, 70000):
            s = ops.flash_splits(batch, 8, ctx)
            assert s >= 1 and s <= max(1, -(-ctx // 64) // 2)   # every split has at least two key tiles


def test_slices_of_k_of_the_tcgen05_product(ops):
    assert ops.tcgen05_splits(8, 4096, 12288) == 6     # the down projection: 192 blocks of 32 k-blocks
    assert ops.tcgen05_splits(8, 4096, 4096) == 4      # the output projection: 128 blocks
    assert ops.tcgen05_splits(8, 6144, 4096) == 3
    assert ops.tcgen05_splits(8, 24576, 4096) == 1     # enough tiles
    assert ops.tcgen05_splits(8, 151936, 4096) == 1
    assert ops.tcgen05_splits(1, 128, 64) == 1         # one k-block cannot be sliced
    for n in (128, 1000, 4096, 20000):
        for k in (64, 520, 4096, 30000):
            s = ops.tcgen05_splits(8, n, k)
            assert 1 <= s <= 8 and (s == 1 or -(-k // 64) // s >= 4)


def batch_of(counts, lens):
    starts = [0]
    for c in counts:
        starts.append(starts[-1] + c)
    return SimpleNamespace(n_seqs=len(counts), q_start_host=starts, seq_lens_host=lens, q_start=list(starts),
                           positions=None, status=None, per_step={})


def test_mixed_steps_divide_into_decoded_tokens_and_portions(ops):
    b = batch_of([1, 1, 1, 512, 40], [900, 30, 2000, 700, 40])
    short, long_ = ops._short_and_long(b, 4)
    assert (short.first, short.last, long_.first, long_.last) == (0, 3, 3, 5)
    assert short.max_q_len == 1 and short.max_seq_len == 2000 and long_.max_q_len == 512 and long_.max_seq_len == 700
    assert short.q_start_host == [0, 1, 2, 3] and long_.q_start_host == [3, 515, 555]
    assert ops._short_and_long(b, 4) is b.per_step[("short_and_long", 4)]        # once per step
    # the short run may be the batch's tail; with 4 query heads per kv head up to 4 tokens are "short"
    b = batch_of([300, 4, 2], [300, 50, 60])
    short, long_ = ops._short_and_long(b, 4)
    assert (short.first, short.last, long_.first, long_.last) == (1, 3, 0, 1)
    # all of one kind, or short ones in the middle: one launch for all
    assert ops._short_and_long(batch_of([1, 1], [5, 6]), 4) is None
    assert ops._short_and_long(batch_of([64, 70], [64, 70]), 4) is None
    assert ops._short_and_long(batch_of([64, 1, 70], [64, 9, 70]), 4) is None
    # with 16 query heads per kv head only single tokens are short
    short, long_ = ops._short_and_long(batch_of([1, 2, 200], [5, 6, 200]), 16)
    assert (short.first, short.last, long_.first, long_.last) == (0, 1, 1, 3)


def test_division_of_prompt_attention(ops):
    # (tiles a block, runs of keys) at 8 kv heads, 4 query heads each (32 tokens a tile)
    assert ops.tcgen05_attention_shape([2048], 8, 4, 2048) == (2, 1)       # 256 blocks: enough
    assert ops.tcgen05_attention_shape([512], 8, 4, 3072) == (2, 2)        # 64 blocks, 48 key tiles: two runs
    assert ops.tcgen05_attention_shape([256], 8, 4, 3072) == (2, 4)
    assert ops.tcgen05_attention_shape([512], 8, 4, 1024) == (1, 1)        # too few keys to share: one tile a block
    assert ops.tcgen05_attention_shape([512], 8, 4, 8192) == (2, 2)
    assert ops.tcgen05_attention_shape([64], 8, 4, 65536) == (2, 8)
    assert ops.tcgen05_attention_shape([40, 40, 40], 2, 16, 40) == (1, 1)
    assert ops.tcgen05_attention_shape([1024], 8, 4, 5120) == (2, 1)       # 128 blocks of two tiles: about one an SM
    assert ops.tcgen05_attention_shape([64], 8, 4, 1064) == (1, 4)         # few keys and few tiles: short runs, one tile a block
    assert ops.tcgen05_attention_shape([128, 128, 128, 128], 8, 4, 1128) == (1, 1)
