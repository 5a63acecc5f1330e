"""GPU parity of ``optimized_attention`` (CUDA path through the C ABI) against
the FP32 oracle: golden fixtures from the reference, the named configurations,
tails, GQA ratios, modes and norm styles.

Tolerance (bf16 and fp16): max-abs <= 2e-2 and mean-abs <= 2e-3 against the
FP32 oracle, plus the reference's own gate (allclose atol=rtol=0.025 and
relative-L2 <= 0.025, src/e1_rope_publication_v1.py:287-293), and an error no
worse than that of the reference's compiled arm: its CPU emulation
(``oracle.emulate_optimized_attention``, pinned to outputs of the real Triton
kernels by tests/test_triton_golden.py) must not be beaten by more than 3 % in
mean-abs / one output place in max-abs.  Where the arm's own max-abs error on an
input exceeds 2e-2 (seed 1701 at GQA 4: 0.02097 on an early row), the bound is the
arm's error: the CUDA path reproduces the arm's rounding points and cannot do
better on that element.
"""
import pytest
import torch

import kernelfuser_b200 as kf
from conftest import SMALL_GOLDEN, load_golden
from kernelfuser_b200.inputs import WORKLOADS
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def to_dev(xs):
    return [None if x is None else x.to(DEV) for x in xs]


def run(xs, **kw):
    out = kf.optimized_attention(*to_dev(xs), **kw)
    torch.cuda.synchronize()
    kf.check_status()
    return out.cpu()


def check(out, ref, label, emu=None):
    m = orc.metric(out, ref)
    if emu is None:
        assert orc.within_tolerance(m), (label, m)
        return m
    me = orc.metric(emu, ref)
    assert m["pass"] and m["mean_abs"] <= orc.MEAN_ABS_TOL, (label, m)
    assert m["max_abs"] <= max(orc.MAX_ABS_TOL, me["max_abs"]), (label, m, me)
    assert m["max_abs"] <= me["max_abs"] + 2.0 ** -8, (label, m, me)
    assert m["mean_abs"] <= 1.03 * me["mean_abs"], (label, m, me)
    return m


@pytest.mark.parametrize("name", SMALL_GOLDEN)
@pytest.mark.parametrize("causal", [False, True])
def test_matches_reference_golden(name, causal):
    meta, t = load_golden(name)
    xs = [t["q"], t["k"], t["v"], t["gq"], t["gk"], t.get("cos"), t.get("sin")]
    style = "hf" if meta["rope"] else "legacy"  # as the reference's API check pairs them
    for mode in ("query", "unfused"):
        out = run(xs, causal=causal, mode=mode, norm_style=style)
        emu = orc.emulate_optimized_attention(*xs, causal=causal, norm_style=style)
        check(out, t["out_causal" if causal else "out_full"], (name, causal, mode), emu)


@pytest.mark.parametrize("s", [1, 33, 129, 1000, 1025])
@pytest.mark.parametrize("causal", [False, True])
def test_sequence_tails(s, causal):
    xs = kf.make_inputs(2, s, 8, 2, 128, seed=4909)
    ref = orc.oracle_fp32(*xs, causal)
    out = run(xs, causal=causal)
    assert out.shape == ref.shape
    check(out, ref, ("tail", s, causal))


@pytest.mark.parametrize("hq,hkv", [(8, 8), (8, 4), (8, 2), (8, 1)])
def test_gqa_ratios(hq, hkv):
    xs = kf.make_inputs(2, 300, hq, hkv, 128, seed=1701)
    ref = orc.oracle_fp32(*xs, True)
    check(run(xs, causal=True), ref, ("gqa", hq, hkv), orc.emulate_optimized_attention(*xs, causal=True))


@pytest.mark.parametrize("seed", [0, 1701, 2803, 3907])
def test_c2_config(seed):
    w = WORKLOADS["C2"]
    xs = kf.make_workload_inputs(w, seed=seed)
    ref = orc.oracle_fp32(*xs, True)
    emu = orc.emulate_optimized_attention(*xs, causal=True) if seed == 0 else None
    check(run(xs, causal=True), ref, ("C2", seed), emu)


def test_c1_shape_in_bf16():
    # C1's shape and seed (the CPU known-answer case), inputs cast to bf16
    w = WORKLOADS["C1"]
    xs = kf.make_workload_inputs(w, seed=0, dtype=torch.bfloat16)
    ref = orc.oracle_fp32(*xs, True)
    check(run(xs, causal=True), ref, "C1-bf16", orc.emulate_optimized_attention(*xs, causal=True))


def test_c3_config_fp16_tail():
    w = WORKLOADS["C3"]
    xs = kf.make_workload_inputs(w, seed=0)
    ref = orc.oracle_fp32(*xs, True)
    m = check(run(xs, causal=True), ref, "C3")
    assert m["max_abs"] < 5e-3  # fp16 carries three more mantissa bits than bf16


def test_d256_theta1e4():
    xs = kf.make_inputs(2, 1024, 4, 2, 256, theta=1e4, seed=0)
    ref = orc.oracle_fp32(*xs, True)
    check(run(xs, causal=True), ref, "D256", orc.emulate_optimized_attention(*xs, causal=True))


def test_positions_theta_and_scale_eps_extensions():
    q, k, v, gq, gk, cos, sin = kf.make_inputs(1, 200, 4, 2, 128, theta=1e6, seed=3)
    ref = orc.oracle_fp32(q, k, v, gq, gk, cos, sin, True, scale=0.05, eps=1e-5)
    out = kf.optimized_attention(*to_dev([q, k, v, gq, gk]), causal=True, positions=torch.arange(200),
                                 theta=1e6, scale=0.05, eps=1e-5)
    torch.cuda.synchronize()
    check(out.cpu(), ref, "extensions")


def test_arm_adapter_accepts_model_style_views():
    # [B,S,H,D] projections viewed as [B,H,S,D], [B,S,D] tables, explicit scale
    b, s, hq, hkv, d = 2, 150, 4, 2, 128
    q, k, v, gq, gk, cos, sin = kf.make_inputs(b, s, hq, hkv, d, seed=21)
    ref = orc.oracle_fp32(q, k, v, gq, gk, cos, sin, True, scale=1 / 16.0)
    qd = q.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    kd = k.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    vd = v.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    assert not qd.is_contiguous()
    out = kf.fused(qd, kd, vd, gq.to(DEV), gk.to(DEV), cos.to(DEV)[None].expand(b, s, d),
                   sin.to(DEV)[None].expand(b, s, d), True, 1e-6, 1 / 16.0, "qwen3")
    torch.cuda.synchronize()
    kf.check_status()
    check(out.cpu(), ref, "arm adapter")


def test_arm_adapter_writes_the_projection_layout():
    # [B,S,H,D] projections in, [B,S,Hq*D] out: no layout copy on either side of the operator
    b, s, hq, hkv, d = 2, 333, 8, 2, 128
    q, k, v, gq, gk, cos, sin = kf.make_inputs(b, s, hq, hkv, d, seed=23)
    ref = orc.oracle_fp32(q, k, v, gq, gk, cos, sin, True)
    views = [t.transpose(1, 2).contiguous().to(DEV).transpose(1, 2) for t in (q, k, v)]
    small = to_dev([gq, gk, cos, sin])
    flat = kf.fused(*views, *small, True, out_layout="bshd")
    plain = kf.fused(*views, *small, True)
    torch.cuda.synchronize()
    kf.check_status()
    assert flat.shape == (b, s, hq * d) and flat.is_contiguous()
    as_bhsd = flat.view(b, s, hq, d).transpose(1, 2)
    check(as_bhsd.contiguous().cpu(), ref, "bshd output")
    assert torch.equal(as_bhsd.contiguous().view(torch.int16), plain.view(torch.int16))
    with pytest.raises(ValueError):
        kf.fused(*views, *small, True, out_layout="sbhd")


def test_output_fully_written_and_deterministic():
    xs = to_dev(kf.make_inputs(2, 333, 8, 2, 128, seed=8))
    out1 = torch.full_like(xs[0], float("nan"))
    out2 = torch.full_like(xs[0], float("nan"))
    kf.optimized_attention(*xs, causal=True, out=out1)
    kf.optimized_attention(*xs, causal=True, out=out2)
    torch.cuda.synchronize()
    kf.check_status()
    assert torch.isfinite(out1).all()
    assert torch.equal(out1.view(torch.int16), out2.view(torch.int16))


def test_head_sharded_views_match_full():
    # rank-style head slices passed as strided views give the same result as the full call
    from kernelfuser_b200.shard import head_shard, shard_inputs
    xs = to_dev(kf.make_inputs(2, 260, 8, 4, 128, seed=13))
    full = kf.optimized_attention(*xs, causal=True)
    parts = []
    for r in range(2):
        sh = head_shard(8, 4, r, 2)
        qs, ks, vs = shard_inputs(xs[0], xs[1], xs[2], sh, contiguous=True)
        parts.append(kf.optimized_attention(qs, ks, vs, *xs[3:], causal=True))
    torch.cuda.synchronize()
    kf.check_status()
    assert torch.equal(torch.cat(parts, 1).view(torch.int16), full.view(torch.int16))


def test_cuda_graph_capture_replay():
    xs = to_dev(kf.make_inputs(1, 256, 8, 2, 128, seed=5))
    eager = kf.optimized_attention(*xs, causal=True)
    torch.cuda.synchronize()
    out = torch.empty_like(xs[0]); kn = torch.empty_like(xs[1])
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        kf.optimized_attention(*xs, causal=True, out=out, kn=kn)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    kf.check_status()
    assert torch.equal(out.view(torch.int16), eager.view(torch.int16))


def test_host_buffer_entry_point_matches_device_path():
    # pinned host tensors in, pinned host tensor out; ragged last chunk (B = 5, chunks of 2)
    xs = kf.make_inputs(5, 260, 8, 2, 128, seed=17)
    want = kf.optimized_attention(*to_dev(xs), causal=True)
    got = kf.optimized_attention_host(*xs, causal=True, chunk_batch=2)
    again = kf.optimized_attention_host(*xs, causal=True, chunk_batch=2)  # staging buffers are reused
    torch.cuda.synchronize()
    kf.check_status()
    assert got.is_pinned() and not got.is_cuda
    assert torch.equal(got.view(torch.int16), want.cpu().view(torch.int16))
    assert torch.equal(again.view(torch.int16), got.view(torch.int16))
    with pytest.raises(ValueError):
        kf.optimized_attention_host(*to_dev(xs), causal=True)
