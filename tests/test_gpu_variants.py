"""Every attention kernel variant (baseline, pipelined, persistent, one tile per CTA) against the
FP32 oracle on the same inputs; the default (automatic) choice is covered by
tests/test_gpu_attention.py."""
import pytest
import torch

import kernelfuser_b200 as kf
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", [1, 2, 3, 5])
@pytest.mark.parametrize("s,hq,hkv,causal,dtype", [
    (517, 8, 2, True, torch.bfloat16),    # even GQA group: two heads per CTA, ragged tail
    (390, 6, 2, True, torch.float16),     # odd group size: two query blocks of one head per CTA
    (129, 3, 3, False, torch.bfloat16),   # G = 1, second tile of the last pair is empty
    (64, 4, 4, True, torch.bfloat16),     # a single sub-block
])
def test_variant_matches_oracle(variant, s, hq, hkv, causal, dtype):
    # one seed for all variants: every kernel sees the same rows, so a difference
    # between variants is a difference between kernels, not between inputs
    xs = kf.make_inputs(3, s, hq, hkv, 128, dtype=dtype, seed=41)
    ref = orc.oracle_fp32(*xs, causal)
    out = kf.optimized_attention(*[x.cuda() for x in xs], causal=causal, variant=variant)
    torch.cuda.synchronize()
    kf.check_status()
    m = orc.metric(out.cpu(), ref)
    assert orc.within_tolerance(m), (variant, s, hq, hkv, m)


def test_many_items_per_persistent_cta():
    # more work items than SMs, so every CTA of the persistent kernel walks several items
    xs = kf.make_inputs(6, 700, 16, 4, 128, seed=77)
    ref = orc.oracle_fp32(*xs, True)
    dx = [x.cuda() for x in xs]
    outs = [kf.optimized_attention(*dx, causal=True, variant=v) for v in (3, 1)]
    torch.cuda.synchronize()
    kf.check_status()
    for o in outs:
        assert orc.within_tolerance(orc.metric(o.cpu(), ref))


def test_d128_only_variants_reject_d256():
    xs = [x.cuda() for x in kf.make_inputs(1, 64, 2, 1, 256, seed=1)]
    for variant in (5,):
        with pytest.raises(ValueError):
            kf.optimized_attention(*xs, causal=True, variant=variant)


@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("s,hq,hkv,causal,dtype", [
    (517, 4, 2, True, torch.bfloat16),
    (200, 3, 1, False, torch.float16),
    (64, 2, 2, True, torch.bfloat16),
])
def test_d256_variants_match_oracle(variant, s, hq, hkv, causal, dtype):
    xs = kf.make_inputs(2, s, hq, hkv, 256, dtype=dtype, theta=1e4, seed=61)
    ref = orc.oracle_fp32(*xs, causal)
    out = kf.optimized_attention(*[x.cuda() for x in xs], causal=causal, variant=variant)
    torch.cuda.synchronize()
    kf.check_status()
    m = orc.metric(out.cpu(), ref)
    assert orc.within_tolerance(m), (variant, s, hq, hkv, m)


def test_persistent_kernels_reuse_their_counter_slots():
    # The persistent kernels take work from counters in the library image, 64 slots used in turn and reset by
    # the last CTA of each launch: run more launches than slots, on two streams, both head dims, and compare
    # every result with the first one of its kind.
    xs128 = [x.cuda() for x in kf.make_inputs(2, 640, 8, 2, 128, seed=5)]
    xs256 = [x.cuda() for x in kf.make_inputs(1, 512, 4, 2, 256, theta=1e4, seed=6)]
    ref128 = kf.optimized_attention(*xs128, causal=True, variant=3)
    ref256 = kf.optimized_attention(*xs256, causal=True, variant=3)
    torch.cuda.synchronize()
    kf.check_status()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    outs = []
    for i in range(100):
        xs, ref = (xs128, ref128) if i % 3 else (xs256, ref256)
        if i % 2:
            with torch.cuda.stream(side):
                outs.append((kf.optimized_attention(*xs, causal=True, variant=3), ref))
        else:
            outs.append((kf.optimized_attention(*xs, causal=True, variant=3), ref))
    torch.cuda.synchronize()
    kf.check_status()
    for out, ref in outs:
        assert torch.equal(out, ref)
