"""The host-side work list of the attention kernels: every visible key of every single-token request lies in
exactly one work item, items are whole tiles, a step fills one wave of blocks where it can, and portions are
cut into query tiles that cover them exactly."""

from types import SimpleNamespace

import numpy as np
import pytest

from tokasaurus_b200.parts.attention import DECODE_BLOCK_SLOTS, MIN_SPLIT_KEYS, plan_attention, split_keys_evenly


@pytest.mark.parametrize("spans", [[1], [2053] * 8, [2053] * 16, [2053] * 32, [2053] * 64, [17, 40000, 300, 64, 65],
                                   [100000] + [100] * 63, [128] * 500])
@pytest.mark.parametrize("blocks_per_item", [1, 8, 16])
def test_split_covers_every_key_once(spans, blocks_per_item):
    span = np.asarray(spans, dtype=np.int64)
    n, size = split_keys_evenly(span, blocks_per_item)
    assert n.shape == span.shape and (n >= 1).all()
    assert (size % 64 == 0).all() and (size >= 64).all()
    assert ((n - 1) * size < span).all() and (n * size >= span).all()  # no empty item, none missing
    # a request is cut only down to the floor, and one long request among short ones is still cut
    assert (size[n > 1] >= MIN_SPLIT_KEYS).all()
    slots = DECODE_BLOCK_SLOTS // blocks_per_item
    if span.max() > 4 * span.sum() / max(1, slots) and span.max() > 4 * MIN_SPLIT_KEYS:
        assert n[np.argmax(span)] > 1


def test_one_wave_where_the_batch_allows():
    for batch, want_items in ((8, 72), (16, 64), (32, 64), (64, 64)):  # a wave of 148 SMs x 4 blocks, 8 blocks an item
        n, _ = split_keys_evenly(np.full((batch,), 2053, dtype=np.int64), 8)
        assert int(n.sum()) == want_items, batch


@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("query_tile", [64, 128])
def test_plan_items_and_tiles(window, query_tile):
    q_len = np.asarray([1, 1, 70, 2, 130, 1, 128], dtype=np.int32)
    kv_len = np.asarray([1, 777, 70, 259, 400, 256, 128], dtype=np.int32)
    plan = plan_attention(SimpleNamespace(seq_q_len=q_len, seq_kv_len=kv_len), window, query_tile=query_tile)
    n_items, n_dec, n_tiles = (int(x) for x in plan["counts"][:3])
    items = plan["items"][: 3 * n_items].reshape(-1, 3)
    dec = plan["dec_seqs"][:n_dec]
    assert list(dec) == [0, 1, 5]
    start = plan["dec_item_start"][: n_dec + 1]
    for e, s in enumerate(dec):
        mine = items[start[e]:start[e + 1]]
        assert (mine[:, 0] == s).all() and (plan["item_entry"][start[e]:start[e + 1]] == e).all()
        span = min(int(kv_len[s]), window) if window else int(kv_len[s])
        covered = np.zeros(span, dtype=np.int32)
        for _, first, count in mine:
            covered[first:min(span, first + count)] += 1
        assert (covered == 1).all()
    tiles = plan["tiles"][: 2 * n_tiles].reshape(-1, 2)
    for s in (2, 3, 4, 6):
        firsts = sorted(int(q0) for r, q0 in tiles if r == s)
        assert firsts == list(range(0, int(q_len[s]), query_tile))
    # the tiles that reach the furthest come first
    reach = [int(kv_len[r] - q_len[r] + q0) for r, q0 in tiles]
    assert reach == sorted(reach, reverse=True)


def test_item_count_stays_under_the_bound_of_the_graphs():
    """CUDA graphs of decode steps size the work list for a batch size alone; no mix of contexts may need more."""
    from tokasaurus_b200.parts.attention import PagedAttention
    from tokasaurus_b200.parts.rope import NoPositionEncoding

    rng = np.random.default_rng(0)
    for nh, nkv in ((32, 8), (4, 4), (64, 1)):
        mixer = PagedAttention(nh * 16, nh, nkv, 16, NoPositionEncoding(), "q", "k", "v", "o")
        for _ in range(300):
            r = int(rng.integers(1, 130))
            kind = int(rng.integers(0, 3))
            span = rng.integers(1, [200, 5000, 200000][kind], size=r).astype(np.int64)
            n, _ = split_keys_evenly(span, mixer._blocks_per_item())
            assert int(n.sum()) <= mixer.plan_capacity(r)["items"], (nh, nkv, r, kind)


def test_plan_says_whether_some_item_is_longer_than_three_tiles():
    """counts[5] picks the split-key kernel's variant (tiles by TMA or not); it must follow the items' sizes."""
    from types import SimpleNamespace

    def flag(kv):
        host = SimpleNamespace(seq_q_len=np.ones(len(kv), dtype=np.int32), seq_kv_len=np.asarray(kv, dtype=np.int32))
        plan = plan_attention(host, None)
        sizes = plan["items"].reshape(-1, 3)[: int(plan["counts"][0]), 2]
        assert int(plan["counts"][5]) == int(sizes.max() > 192)
        return int(plan["counts"][5])

    assert flag([2048]) == 0           # one request: cut into items of 128 keys
    assert flag([100, 7]) == 0
    assert flag([2048] * 8) == 1       # items of 384 keys
    assert flag([50, 40000]) == 1


def test_few_query_tiles_ask_for_one_head_a_block():
    """counts[7]: a step whose portions make so few 128-query tiles that blocks of two heads would leave SMs without
    work (one 512-token portion: 4 tiles x 16 pairs on 148 SMs) asks the portions' kernel for a block a head."""
    def counts(q_lens, head_blocks):
        host = SimpleNamespace(seq_q_len=np.asarray(q_lens, dtype=np.int32),
                               seq_kv_len=np.asarray([q + 1000 for q in q_lens], dtype=np.int32))
        return plan_attention(host, None, query_tile=128, head_blocks=head_blocks)["counts"]
    assert counts([512], 148 // 32)[2] == 4 and counts([512], 148 // 32)[7] == 1
    assert counts([513], 148 // 32)[7] == 0       # five tiles of 32 heads are more than the SMs
    assert counts([1, 1, 300], 148 // 32)[7] == 1  # decoding requests make no tiles
    assert counts([1, 1], 148 // 32)[7] == 0       # no tiles at all
    assert counts([512], 0)[7] == 0                # a planner that was given no device
