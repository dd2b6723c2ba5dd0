"""Failure detection without a GPU fault: a pipeline whose producer never
signals makes every other role's bounded wait run out; the kernel tears down,
the host sees KAPYB_TIMEOUT, and the context stays usable."""
import pytest
import torch

from util import normal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("path", ["1cta:128", "2cta:256", "2cta:512"])
def test_starved_pipeline_times_out_cleanly(handle, pkg, path):
    A, B = normal((512, 256), 1).cuda(), normal((256, 1024), 2).cuda()
    want = handle.matmul(A, B)
    handle.check()
    # debug bit 16: the TMA producer neither loads nor arrives; waits give up after 50 ms
    handle.set_matmul_path(path + ":d16:w50")
    try:
        handle.matmul(A, B)
        with pytest.raises(pkg.KapybTimeout):
            handle.check()
    finally:
        handle.set_matmul_path("auto")
    # the status word was cleared and the device is fine: same call, same bits
    again = handle.matmul(A, B)
    handle.check()
    assert torch.equal(again, want)
