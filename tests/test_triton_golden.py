"""Outputs of the reference's REAL compiled arm as golden vectors.

``tests/golden/triton_arm_b200.npz`` was written by ``oracle/triton_arm.py
--golden`` on a B200: prepared K and the operator's output of the reference's
Triton kernels (``launch_attention``, src/e1_rope_publication_v1.py:661-677)
on small seeded cases.  Inputs are regenerated here from the seed.

CPU tests pin the oracle's emulation of the arm's rounding contract to these
vectors; the GPU tests hold the CUDA path to them: prepared K equal except for
last-place effects of the summation order, and an error against the FP32
oracle no worse than the recorded arm's own.
"""
import numpy as np
import pytest
import torch

import kernelfuser_b200 as kf
from conftest import GOLDEN
from oracle import oracle as orc

CASES = ["g128_hf", "g128_legacy", "g128_norope", "g128_long", "g256_hf"]
# Elements that may differ from the recorded prepared K: the row's sum of squares is added up in a
# different order, which moves the inverse RMS by one fp32 place and flips a rounding now and then
# (observed on million-element tensors: CPU emulation <= 1.5e-5, CUDA kernel <= 3e-6 of the elements; on
# these small fixtures one such row is 26 of 40 960 elements = 6.3e-4).
KN_MISMATCH = 1e-3


def load(name):
    z = np.load(GOLDEN / "triton_arm_b200.npz")
    b, s, hq, hkv, d, theta, rope, hf = (int(x) for x in z[name + "_cfg"])
    xs = kf.make_inputs(b, s, hq, hkv, d, dtype=torch.bfloat16, theta=float(theta), seed=0, rope=bool(rope))
    kn = torch.from_numpy(z[name + "_kn"].copy()).view(torch.bfloat16)
    out = torch.from_numpy(z[name + "_out"].copy()).view(torch.bfloat16)
    return xs, kn, out, "hf" if hf else "legacy"


@pytest.mark.parametrize("name", CASES)
def test_emulated_rows_equal_the_real_arm(name):
    xs, kn, _, style = load(name)
    got = orc.emulate_rows(xs[1], xs[4], xs[5], xs[6], hf_norm=(style == "hf"))
    assert float((got != kn).float().mean()) <= KN_MISMATCH


@pytest.mark.parametrize("name", CASES)
def test_emulated_operator_equals_the_real_arm(name):
    xs, _, out, style = load(name)
    got = orc.emulate_optimized_attention(*xs, causal=True, norm_style=style)
    d = (got.float() - out.float()).abs()
    # fp32 accumulation order inside the matrix products differs, and one prepared K row that differs in a
    # few places moves every output behind it a little: one-place differences (observed: 0.06-0.23 % of the
    # elements, 6.7 % on the case with such a row), and the same error against the FP32 oracle
    assert float((d > 0).float().mean()) <= 0.1 and float(d.max()) <= 2.0 ** -7
    want = orc.oracle_fp32(*xs, True)
    mine, arm = orc.metric(got, want), orc.metric(out, want)
    assert abs(mine["mean_abs"] - arm["mean_abs"]) <= 0.005 * arm["mean_abs"], (mine, arm)


def test_uncontracted_spelling_is_not_what_the_arm_computes():
    # r(r(y*c) - r(p*s)), the literal reading of the source, differs from the arm in >10 % of the elements
    xs, kn, _, _ = load("g128_long")
    q, k, v, gq, gk, cos, sin = xs
    r = lambda t: t.to(torch.bfloat16).float()
    kf32 = k.float()
    inv = torch.rsqrt(kf32.square().sum(-1, keepdim=True) / 128 + 1e-6)
    y = r(r(kf32 * inv) * gk.float())
    p = torch.cat([y[..., 64:], y[..., :64]], -1)
    pr, ro = r(y * cos.float()), r(p * sin.float())
    lit = torch.cat([r(pr[..., :64] - ro[..., :64]), r(pr[..., 64:] + ro[..., 64:])], -1).to(torch.bfloat16)
    assert float((lit != kn).float().mean()) > 0.1


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_cuda_prepared_k_equals_the_real_arm(name):
    xs, kn, _, style = load(name)
    dev = torch.device("cuda")
    got = kf.prepare_rows(xs[1].to(dev), xs[4].to(dev), None if xs[5] is None else xs[5].to(dev),
                          None if xs[6] is None else xs[6].to(dev), norm_style=style).cpu()
    torch.cuda.synchronize()
    assert float((got != kn).float().mean()) <= KN_MISMATCH


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("mode", ["query", "unfused"])
def test_cuda_error_no_worse_than_the_real_arm(name, mode):
    xs, _, out, style = load(name)
    dev = torch.device("cuda")
    got = kf.optimized_attention(*[None if x is None else x.to(dev) for x in xs], causal=True, mode=mode,
                                 norm_style=style).cpu()
    torch.cuda.synchronize()
    kf.check_status()
    want = orc.oracle_fp32(*xs, True)
    mine, arm = orc.metric(got, want), orc.metric(out, want)
    assert mine["pass"], mine
    # the arm's own error, plus one output place at |o| < 0.25 and 3 % for the different block size
    assert mine["max_abs"] <= arm["max_abs"] + 2.0 ** -10, (mine, arm)
    assert mine["mean_abs"] <= 1.03 * arm["mean_abs"], (mine, arm)
    assert mine["relative_l2"] <= 1.03 * arm["relative_l2"], (mine, arm)
