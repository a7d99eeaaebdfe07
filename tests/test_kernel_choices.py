"""How many CTAs share the keys of a query tile (prefill) or of a (token, kv head) (decode): the
host-side choices of ``prism_b200.ops``, which need no GPU."""

import random

import numpy as np

import pytest

from prism_b200 import ops

B200 = 148        # SMs of the device the measured thresholds come from; the tests size the grids for it by hand


def test_prefill_splits_choice():
    """Splits only when the query tiles leave the GPU idle and the keys are many."""
    assert ops.prefill_splits(1, 2048, 28, 2048, None, sms=B200) == 1          # 448 CTAs already
    assert ops.prefill_splits(1, 128, 28, 640, None, sms=B200) == 1            # 10 key tiles: not worth a merge
    assert ops.prefill_splits(1, 128, 28, 2048 + 128, None, sms=B200) == 2     # few CTAs: worth it from 2,048 keys
    assert ops.prefill_splits(1, 512, 28, 2048 + 512, None, sms=B200) == 1
    n = ops.prefill_splits(1, 128, 28, 32768 + 128, None, sms=B200)
    assert 2 <= n <= 16 and 28 * n <= 2 * B200
    assert ops.prefill_splits(1, 128, 28, 32768 + 128, 512, sms=B200) == 1     # a window of 512 keys: few tiles
    assert ops.prefill_splits(4, 256, 28, 32768, None, sms=B200) == 1


def test_decode_splits_choice():
    """As many splits as fill one wave; a batch that fills the GPU unevenly gets a few splits once the
    contexts are long enough to pay for the merge."""
    assert ops.decode_splits(8, 4, 2100, None, sms=B200) == 9                  # 288 CTAs for 296 places
    assert ops.decode_splits(1, 4, 2100, None, sms=B200) == 11                 # three 64-key tiles each at least
    assert ops.decode_splits(1, 4, 500, None, sms=B200) == 3
    assert ops.decode_splits(1, 4, 100, None, sms=B200) == 1
    assert ops.decode_splits(1, 4, 32768, None, sms=B200) == 64                # never more than 64
    assert ops.decode_splits(64, 4, 2100, None, sms=B200) == 1                 # short contexts: no merge
    assert ops.decode_splits(64, 4, 8192, None, sms=B200) == 1
    assert ops.decode_splits(64, 4, 32768, None, sms=B200) == 4                # 256 CTAs would be 2 + 1 per SM
    assert ops.decode_splits(74, 4, 32768, None, sms=B200) == 1                # 296 CTAs: even already
    assert ops.decode_splits(64, 4, 32768, 512, sms=B200) == 1                 # a window of 512 keys is a short context
    assert ops.decode_splits(64, 4, 32768, None, balance=False, sms=B200) == 1     # a captured graph knows a bound only
    assert ops.decode_splits(8, 4, 32768, None, balance=False, sms=B200) == 9


def test_grids_follow_the_device():
    """The SM count is the device's, not a constant: other counts give other grids, and without a
    device the count must be given."""
    assert ops.decode_splits(8, 4, 2100, None, sms=132) == 8         # 256 CTAs for 264 places
    assert ops.decode_splits(8, 4, 2100, None, sms=64) == 4
    assert ops.tc_ksplit(4608, 3584, sms=148) == 4 and ops.tc_ksplit(4608, 3584, sms=80) == 2
    assert ops.tc_ksplit(3584, 18944, sms=148) == 5 and ops.tc_ksplit(152064, 3584, sms=148) == 1
    # a few tokens and a long K: half as many CTAs again (two fit on an SM), 32 k-blocks each at least
    assert ops.tc_ksplit(3584, 18944, sms=148, M=8) == 7 and ops.tc_ksplit(3584, 18944, sms=148, M=32) == 5
    assert ops.tc_ksplit(4608, 3584, sms=148, M=8) == 4 and ops.tc_ksplit(5120, 13824, sms=148, M=1) == 5
    # few tokens: rounded to the nearest count, not down (two CTAs fit on an SM); many tokens: never more CTAs than SMs
    assert ops.tc_ksplit(7168, 5120, sms=148, M=8) == 3 and ops.tc_ksplit(7168, 5120, sms=148, M=32) == 2
    assert ops.tc_ksplit(5120, 5120, sms=148, M=1) == 4 and ops.tc_ksplit(3584, 3584, sms=148, M=16) == 5
    assert ops.prefill_splits(1, 128, 28, 32768 + 128, None, sms=64) < ops.prefill_splits(1, 128, 28, 32768 + 128, None, sms=148)
    import torch
    if not torch.cuda.is_available():
        with pytest.raises(ops.KernelError, match="sms="):
            ops.decode_splits(8, 4, 2100, None)


def test_prefill_kernel_choice():
    """64 tokens and more: the tcgen05 kernel; fewer: the mma.sync kernel, unless the cache is long."""
    assert ops.prefill_on_tc(64, 64, None) and ops.prefill_on_tc(2048, 2048, None)
    assert not ops.prefill_on_tc(63, 1000, None)
    assert ops.prefill_on_tc(5, 6000, None)                          # a prompt's last few tokens behind the rest
    assert not ops.prefill_on_tc(5, 6000, 512)                       # a window keeps the keys few


def test_decoders_leave_a_mixed_step_for_the_decode_kernel():
    assert not ops.decoders_apart(0, 0, None)
    assert not ops.decoders_apart(3, 2000, None)                     # a few short ones stay with the portions
    assert ops.decoders_apart(ops.MIXED_SPLIT_MIN, 100, None)
    assert ops.decoders_apart(1, 6001, None)                         # one long context is enough
    assert not ops.decoders_apart(1, 6001, 512)


def test_decode_plan_reproduces_the_measured_choices_for_equal_contexts():
    """Equal contexts of 2,100 keys on 148 SMs with 4 kv heads: the plan gives every request the number of CTAs
    that was measured best for its batch size."""
    for batch, want in [(1, 11), (8, 9), (16, 4), (24, 3), (32, 2), (40, 1), (48, 1), (56, 1), (64, 1)]:
        target, cap = ops.decode_plan_for([2099] * batch, 4, None, sms=148)
        assert cap == want, (batch, cap)
        assert ops.decode_used_splits(ops.decode_tiles(2099, None), target, 64) == want
    # many long contexts of one length: the number of CTAs each that fills whole waves, about two of them
    for batch, want in [(24, 3), (32, 4), (40, 5), (48, 3), (64, 2)]:
        for keys in (8192, 16384, 32768):
            assert ops.decode_plan_for([keys - 1] * batch, 4, None, sms=148)[1] == want, (batch, keys)
    assert ops.decode_plan_for([8191] * 8, 4, None, sms=148)[1] == 9          # a few requests: one wave as before
    assert ops.decode_plan_for([4095] * 48, 4, None, sms=148)[1] == 1         # shorter contexts: as before


def test_decode_plan_shares_a_ragged_batch_by_context():
    """One long context among short ones: the long one gets CTAs in proportion, the short ones a single CTA,
    all CTAs together fit in one wave, and no CTA gets fewer than the least number of tiles."""
    sms = 148
    rng = random.Random(3)
    for _ in range(200):
        batch = rng.choice([1, 2, 5, 8, 17, 32, 64])
        nkv = rng.choice([1, 2, 4, 8])
        window = rng.choice([None, None, 300, 4096])
        pos = [rng.choice([0, 5, 63, 64, 700, 5000, 40000]) + rng.randrange(64) for _ in range(batch)]
        target, cap = ops.decode_plan_for(pos, nkv, window, sms=sms)
        used = [ops.decode_used_splits(ops.decode_tiles(p, window), target, cap) for p in pos]
        assert max(used) == cap >= 1
        if batch * nkv <= 2 * sms:                    # one CTA each fits at once: then the plan fills one wave,
            n = sum(used) * nkv                       # or two where many CTAs are short and end early
            assert n <= 2 * sms or (n <= 4 * sms and sum(ops.decode_tiles(p, window) for p in pos) / sum(used)
                                    < 0.75 * max(ops.decode_tiles(p, window) / u for p, u in zip(pos, used)) * 2)
        for p, u in zip(pos, used):
            t = ops.decode_tiles(p, window)
            assert u == 1 or t // u >= ops.DECODE_MIN_TILES
    # 64 requests of 128 to 4,096 keys: one wave would leave CTAs of 2 to 58 tiles; two waves of at most 21
    rng = random.Random(0)
    ragged = [4096] + [rng.randint(128, 4096) for _ in range(63)]
    target, cap = ops.decode_plan_for(ragged, 4, None, sms=sms)
    used = [ops.decode_used_splits(ops.decode_tiles(p, None), target, cap) for p in ragged]
    assert 2 * sms < sum(used) * 4 <= 4 * sms and max(ops.decode_tiles(p, None) / u for p, u in zip(ragged, used)) < 22
    target, cap = ops.decode_plan_for([16383] + [499] * 31, 4, None, sms=sms)
    assert cap > 16 and ops.decode_used_splits(ops.decode_tiles(499, None), target, cap) == 1
    # a window bounds what a token sees
    assert ops.decode_tiles(40000, 128) <= 3 and ops.decode_tiles(10, 128) == 1 and ops.decode_tiles(64, None) == 2
    # a descriptor without a plan holds 0: the least number of tiles per CTA decides
    assert ops.decode_used_splits(33, 0, 64) == 11 and ops.decode_used_splits(33, 0, 4) == 4


def test_decode_work_items_cover_every_request_once():
    """The items of a step: consecutive per request, split numbers 0 .. used - 1, no CTA without a tile, and the
    counts that ``decode_plan_for`` gives (less where fewer CTAs leave each the same number of tiles)."""
    rng = random.Random(5)
    for _ in range(100):
        batch = rng.choice([1, 3, 8, 33, 64])
        nkv = rng.choice([1, 4, 8])
        window = rng.choice([None, 200, 5000])
        pos = [rng.choice([0, 63, 64, 900, 7000, 33000]) + rng.randrange(64) for _ in range(batch)]
        items, starts, most = ops.decode_work_items(pos, nkv, window, sms=148)
        target, cap = ops.decode_plan_for(pos, nkv, window, sms=148)
        used_of, first_of = starts >> 16, starts & 0xffff
        assert items.dtype.name == starts.dtype.name == "int32" and items.shape == (used_of.sum(), 4)
        assert len(starts) == batch and sorted(first_of.tolist()) == (np.cumsum(sorted_used(items, batch)) - sorted_used(items, batch)).tolist()
        longest = []
        for b, p in enumerate(pos):
            mine = items[first_of[b]:first_of[b] + used_of[b]]
            used = len(mine)
            tiles = ops.decode_tiles(p, window)
            assert 1 <= used <= ops.decode_used_splits(tiles, target, cap) and used <= most
            assert mine[:, 0].tolist() == [b] * used and mine[:, 3].tolist() == [b] * used
            assert mine[:, 2].tolist() == [p] * used
            assert (mine[:, 1] & 0xffff).tolist() == list(range(used)) and (mine[:, 1] >> 16).tolist() == [used] * used
            per = -(-tiles // used)
            assert (used - 1) * per < tiles                   # the last CTA has a tile
            assert -(-tiles // ops.decode_used_splits(tiles, target, cap)) == per     # and none has more than planned
            longest.append((first_of[b], per))
        assert most == used_of.max()
        in_order = [per for _, per in sorted(longest)]
        assert in_order == sorted(in_order, reverse=True)     # the longest CTAs come first


def sorted_used(items, batch):
    """The requests' item counts in the order in which their items lie."""
    seen, out = set(), []
    for tok, word in zip(items[:, 0].tolist(), items[:, 1].tolist()):
        if tok not in seen:
            seen.add(tok)
            out.append(word >> 16)
    return np.array(out)


def test_decode_work_items_remembered_between_steps_are_the_same():
    """The caller's memo saves the planning while no request's tile count changes; the result is the same."""
    rng = random.Random(9)
    for _ in range(10):
        batch, window = rng.choice([1, 5, 33]), rng.choice([None, 300])
        start = [rng.randint(0, 5000) for _ in range(batch)]
        memo, reused = {}, 0
        for step in range(150):
            pos = [p + step for p in start]
            before = memo.get("key")
            a = ops.decode_work_items(pos, 4, window, sms=148, memo=memo)
            reused += memo.get("key") == before
            b = ops.decode_work_items(pos, 4, window, sms=148)
            assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]) and a[2] == b[2]
        assert batch > 1 or reused >= 140
