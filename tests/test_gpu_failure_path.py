"""The failure path of the bounded waits, taken on purpose in the allowed form: a self-test kernel of the
library waits on a barrier nobody arrives on, its wait runs out after a short limit and it returns with a
code in the status word.  Nothing faults, traps or hangs; the device stays usable.

Checked here: the code arrives, launches queued behind a failure do nothing (the word is sticky),
``check_status`` raises ``KernelStatusError`` and clears the word, and the next call is correct again."""
import pytest
import torch

import kernelfuser_b200 as kf
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_wait_runs_out_status_is_reported_and_cleared():
    dev = torch.device("cuda")
    xs = kf.make_inputs(2, 300, 8, 2, 128, seed=5)
    dx = [x.to(dev) for x in xs]
    want = orc.oracle_fp32(*xs, True)
    kf.check_status()  # starts clean

    kf.selftest_wait_timeout(100_000)  # ~50 microseconds of polling, then the kernel gives up
    torch.cuda.synchronize()
    assert int(kf.status_word(dev).item()) == 901

    # every attention kernel drains without touching its output while the word is set
    for variant in (0, 1, 2, 3, 5):
        out = torch.full(dx[0].shape, float("nan"), dtype=dx[0].dtype, device=dev)
        kf.optimized_attention(*dx, causal=True, out=out, variant=variant)
        torch.cuda.synchronize()
        assert torch.isnan(out).all(), variant

    with pytest.raises(kf.KernelStatusError, match="901"):
        kf.check_status()
    assert int(kf.status_word(dev).item()) == 0
    kf.check_status()  # cleared: does not raise again

    for variant in (0, 3):
        out = kf.optimized_attention(*dx, causal=True, variant=variant)
        torch.cuda.synchronize()
        kf.check_status()
        assert orc.within_tolerance(orc.metric(out.cpu(), want)), variant


def test_first_failure_wins():
    dev = torch.device("cuda")
    st = kf.status_word(dev)
    st.fill_(7)
    kf.selftest_wait_timeout(10_000)
    torch.cuda.synchronize()
    assert int(st.item()) == 7  # an earlier code is not overwritten
    with pytest.raises(kf.KernelStatusError, match="7"):
        kf.check_status()
