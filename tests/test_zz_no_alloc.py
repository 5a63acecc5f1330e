"""GPU test of the allocation-free entry point ``kf_optimized_attention_static``.

That entry point serves callers that cannot allocate device memory at the
point of the call (the host framework owns the device heap, cudaMalloc is
off-limits there, or the request path must stay out of the allocator): the
prepared-K scratch is a fixed 32 MiB array inside the library instead of a
tensor allocated per call.  Its result must equal the regular entry points'
(``kf_prepare_rows`` + ``kf_attention_fwd``) on back-to-back calls that share
the array, and sizes beyond the array must be refused on the host.

This file sorts last on purpose so a run that stops at the first failure has
already exercised everything else.
"""
import pytest
import torch

import kernelfuser_b200 as kf
from kernelfuser_b200 import _lib
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _dev(xs):
    return [x.cuda() for x in xs]


def test_static_scratch_matches_regular_entry_point_twice_in_a_row():
    # two different problems back to back: the second is smaller, so stale
    # rows of the first call stay in the shared array beside it
    cases = [dict(b=2, s=517, hq=8, hkv=2, d=128, dtype=torch.bfloat16, seed=31, causal=True),
             dict(b=1, s=200, hq=4, hkv=4, d=256, dtype=torch.float16, seed=32, causal=False)]
    for c in cases:
        xs = kf.make_inputs(c["b"], c["s"], c["hq"], c["hkv"], c["d"], dtype=c["dtype"], theta=1e4, seed=c["seed"])
        dx = _dev(xs)
        want = kf.optimized_attention(*dx, causal=c["causal"])
        out = torch.full_like(dx[0], float("nan"))
        kf.status_word(out.device)  # the caller's status word exists before the call
        count = lambda: torch.cuda.memory_stats()["allocation.all.allocated"]  # allocations so far (monotonic)
        before = count()
        got = kf.optimized_attention_static(*dx, out, causal=c["causal"])
        assert count() == before  # the call requested no device memory from torch's allocator
        torch.cuda.synchronize()
        kf.check_status()
        assert got.data_ptr() == out.data_ptr()
        # same kernels on the same data: identical up to the tolerance the parity tests use
        m = orc.metric(got.cpu(), want.cpu())
        assert orc.within_tolerance(m), (c, m)
        assert m["max_abs"] == 0.0, (c, m)
        # and it is right in absolute terms, not merely consistent
        assert orc.within_tolerance(orc.metric(got.cpu(), orc.oracle_fp32(*xs, c["causal"])))


def test_sizes_beyond_the_builtin_scratch_are_refused():
    lib = _lib.load()
    limit = lib.kf_static_scratch_bytes()
    assert limit == 32 << 20
    b, hkv, s, d = 5, 8, 4096, 128  # B*Hkv*S*D*2 = 40 MiB > 32 MiB
    assert 2 * b * hkv * s * d > limit
    q = torch.empty(1, 8, 8, 128, dtype=torch.bfloat16, device="cuda")  # never read: the call is refused first
    st = kf.status_word(q.device)
    strides = [8 * s * d, s * d, d]
    rc = lib.kf_optimized_attention_static(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(),
                                           None, None, q.data_ptr(), b, 8, hkv, s, d, 0, 1, 1, 1e-6, 0.1,
                                           *(strides * 4), st.data_ptr(), None)
    assert rc == -1
    assert b"built-in scratch" in lib.kf_last_error()
    torch.cuda.synchronize()
    kf.check_status()
