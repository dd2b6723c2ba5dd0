"""kapyb_gather_signal / kapyb_gather_wait on one GPU: the flag words live in
pinned host memory, so the test decides who signals.  A wait that nobody
answers runs into its time limit, reports KAPYB_TIMEOUT through kapyb_check and
leaves the context usable; no kernel here waits for another kernel of the same
GPU (a signal is always stream-ordered before the wait that needs it)."""
import pytest
import torch

from util import normal

pytestmark = pytest.mark.gpu


def pinned_words(n=64):
    t = torch.zeros(n, dtype=torch.int32).pin_memory()
    return t


def test_signal_then_wait(handle):
    flags = pinned_words()
    for seq in (1, 2, 3):
        handle.gather_signal([flags.data_ptr()], 0, seq)
        handle.gather_wait(flags.data_ptr(), 1, seq, limit_ms=500)
        handle.check()
        assert int(flags[0]) == seq
    # already past the awaited number: returns at once
    handle.gather_wait(flags.data_ptr(), 1, 2, limit_ms=50)
    handle.check()


def test_three_ranks_emulated(handle):
    """Three flag arrays stand for three ranks; each 'rank' signals into all of
    them, after which every array satisfies a wait on all three words."""
    arrays = [pinned_words() for _ in range(3)]
    ptrs = [a.data_ptr() for a in arrays]
    for r in range(3):
        handle.gather_signal(ptrs, r, 7)
    for r in range(3):
        handle.gather_wait(ptrs[r], 3, 7, limit_ms=500)
    handle.check()
    for a in arrays:
        assert a[:3].tolist() == [7, 7, 7] and int(a[3]) == 0


def test_sequence_numbers_wrap(handle):
    flags = pinned_words()
    handle.gather_signal([flags.data_ptr()], 0, 0xFFFFFFFF)
    handle.gather_wait(flags.data_ptr(), 1, 0xFFFFFFFF, limit_ms=500)
    handle.gather_signal([flags.data_ptr()], 0, 0x100000001)      # wraps to 1
    handle.gather_wait(flags.data_ptr(), 1, 1, limit_ms=500)
    handle.check()
    # 0xFFFFFFFF is "behind" 1 on the wrapped number line: that wait is satisfied too
    handle.gather_wait(flags.data_ptr(), 1, 0xFFFFFFFF, limit_ms=50)
    handle.check()


def test_unanswered_wait_times_out_and_recovers(handle, pkg):
    flags = pinned_words()
    A, B = normal((256, 256), 1).cuda(), normal((256, 256), 2).cuda()
    want = handle.matmul(A, B)
    handle.check()
    handle.gather_signal([flags.data_ptr()], 0, 1)          # word 0 is there, word 1 never comes
    handle.gather_wait(flags.data_ptr(), 2, 1, limit_ms=50)
    with pytest.raises(pkg.KapybTimeout):
        handle.check()
    # the context is intact: status cleared, kernels run, results are the same bits
    handle.check()
    assert torch.equal(handle.matmul(A, B), want)
    handle.check()
    # and once the missing word arrives (written by the host here) the wait passes
    flags[1] = 1
    handle.gather_wait(flags.data_ptr(), 2, 1, limit_ms=500)
    handle.check()


def test_argument_checks(handle):
    flags = pinned_words()
    with pytest.raises(ValueError, match="ranks"):
        handle.gather_signal([flags.data_ptr()], 3, 1)
    with pytest.raises(ValueError, match="flag array"):
        handle.gather_wait(0, 1, 1)
    with pytest.raises(ValueError, match="1..64"):
        handle.gather_wait(flags.data_ptr(), 65, 1)
