"""CPU tests of the oracle against the golden vectors produced by the
reference's own ``oracle_fp32`` (see tests/golden/make_golden.py)."""
import hashlib
import json

import numpy as np
import pytest
import torch

from conftest import GOLDEN, SMALL_GOLDEN, load_golden
from kernelfuser_b200.inputs import WORKLOADS, make_inputs, make_workload_inputs, rope_tables
from oracle import oracle as orc


@pytest.mark.parametrize("name", SMALL_GOLDEN)
@pytest.mark.parametrize("causal", [False, True])
def test_oracle_matches_reference_golden(name, causal):
    meta, t = load_golden(name)
    want = t["out_causal" if causal else "out_full"]
    for fn in (orc.oracle_fp32, orc.oracle_fp32_explicit):
        got = fn(t["q"], t["k"], t["v"], t["gq"], t["gk"], t.get("cos"), t.get("sin"), causal)
        assert got.shape == want.shape
        assert torch.allclose(got, want, atol=2e-5, rtol=1e-5), (name, fn.__name__, (got - want).abs().max())


@pytest.mark.parametrize("causal", [False, True])
def test_factored_emulation_against_the_reference_golden(causal):
    # the factored no-RoPE form is the same operator as the no-RoPE oracle the reference stored;
    # its CPU emulation must meet the tolerance the kernels are held to
    meta, t = load_golden("norope_s33_d128_bf16")
    want = t["out_causal" if causal else "out_full"]
    got = orc.emulate_factored_attention(t["q"], t["k"], t["v"], t["gq"], t["gk"], causal=causal)
    assert orc.within_tolerance(orc.metric(got, want))


def test_golden_inputs_regenerate_from_seed():
    # the stored inputs are what the seeded generator produces today
    for name in SMALL_GOLDEN:
        meta, t = load_golden(name)
        xs = make_inputs(meta["B"], meta["S"], meta["Hq"], meta["Hkv"], meta["D"],
                         dtype=getattr(torch, meta["dtype"]), theta=meta["theta"], seed=meta["seed"],
                         rope=meta["rope"])
        for key, x in zip(("q", "k", "v", "gq", "gk", "cos", "sin"), xs):
            if x is None:
                continue
            assert torch.equal(x.view(torch.int16), t[key].view(torch.int16)), (name, key)


def test_c1_known_answer():
    z = np.load(GOLDEN / "c1_fp32_seed0.npz")
    meta = json.loads(bytes(z["meta"]).decode())
    xs = make_workload_inputs(WORKLOADS["C1"], seed=0)
    for key, x in zip(("q", "k", "v", "gq", "gk", "cos", "sin"), xs):
        digest = hashlib.sha256(x.contiguous().numpy().tobytes()).hexdigest()
        assert digest == meta["input_sha256"][key], key
    for fn in (orc.oracle_fp32, orc.oracle_fp32_explicit):
        o = fn(*xs, True).flatten()
        sample = o[torch.arange(0, o.numel(), meta["sample_stride"])]
        assert torch.allclose(sample, torch.from_numpy(z["sample"]), atol=2e-5, rtol=1e-5)
        assert abs(float(o.double().sum()) - meta["out_sum"]) < 1e-2
        assert abs(float(o.double().abs().sum()) - meta["out_abs_sum"]) < 1e-1 + 1e-6 * meta["out_abs_sum"]


def test_rope_tables_layout():
    cos, sin = rope_tables(torch.arange(7), 128, 1e6, torch.bfloat16)
    assert cos.shape == (7, 128) and torch.equal(cos[:, :64], cos[:, 64:]) and torch.equal(sin[:, :64], sin[:, 64:])
    assert torch.all(cos[0] == 1) and torch.all(sin[0] == 0)


def test_gqa_mapping():
    x = torch.arange(2 * 3 * 1 * 1, dtype=torch.float32).reshape(2, 3, 1, 1)
    y = orc.expand(x, 6)
    assert y.shape[1] == 6
    for h in range(6):
        assert torch.equal(y[:, h], x[:, h // 2])


def test_causal_single_token_is_v():
    q, k, v, gq, gk, cos, sin = make_inputs(2, 1, 4, 2, 128, seed=5)
    o = orc.oracle_fp32(q, k, v, gq, gk, cos, sin, True)
    assert torch.allclose(o, orc.expand(v.float(), 4), atol=1e-6)


@pytest.mark.parametrize("dtype,d,theta", [(torch.bfloat16, 128, 1e6), (torch.float16, 128, 1e6),
                                           (torch.bfloat16, 256, 1e4)])
@pytest.mark.parametrize("causal", [False, True])
def test_emulated_compiled_arm_passes_gate(dtype, d, theta, causal):
    # the rounding-contract emulation of the reference's compiled arm meets the
    # reference gate and the build's max-abs / mean-abs tolerance
    xs = make_inputs(1, 200, 4, 2, d, dtype=dtype, theta=theta, seed=1701)
    ref = orc.oracle_fp32(*xs, causal)
    for style in ("hf", "legacy"):
        got = orc.emulate_optimized_attention(*xs, causal=causal, norm_style=style)
        m = orc.metric(got, ref)
        assert orc.within_tolerance(m), (style, m)


def test_emulated_rows_close_to_fp32():
    q, k, v, gq, gk, cos, sin = make_inputs(1, 50, 2, 2, 128, seed=3)
    y = orc.emulate_rows(k, gk, cos, sin).float()
    want = orc.rope_fp32(orc.rmsnorm_fp32(k, gk), cos, sin)
    assert (y - want).abs().max() < 0.06 and (y - want).abs().mean() < 5e-3


def test_metric_thresholds():
    y = torch.ones(4, 4)
    assert orc.metric(y.clone(), y)["pass"]
    assert not orc.metric(y + 0.06, y)["pass"]
    bad = y.clone(); bad[0, 0] = float("nan")
    m = orc.metric(bad, y)
    assert not m["pass"] and not m["finite"]
    assert orc.attention_flops(16, 32, 4096, 128, True) == pytest.approx(2.199e12, rel=1e-3)
