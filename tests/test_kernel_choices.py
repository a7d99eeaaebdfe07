"""How many CTAs share the keys of a query tile (prefill) or of a (token, kv head) (decode): the
host-side choices of ``prism_b200.ops``, which need no GPU."""

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
