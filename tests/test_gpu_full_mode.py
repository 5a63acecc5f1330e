"""`launch_attention` in its three modes (the reference's launcher, src/e1_rope_publication_v1.py:661-677):
'full' (one launch, K normalised and rotated per tile inside the loop), 'query' and 'unfused', against the FP32
oracle and against one another on the same inputs."""
import pytest
import torch

import kernelfuser_b200 as kf
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _run(mode, dx, causal, **kw):
    q, k = dx[0], dx[1]
    out = torch.empty_like(q)
    scratch = {}
    if mode != "full":
        scratch["kn"] = torch.empty_like(k)
    if mode == "unfused":
        scratch["qn"] = torch.empty_like(q)
    kf.launch_attention(tuple(dx), out, causal=causal, mode=mode, **scratch, **kw)
    torch.cuda.synchronize()
    kf.check_status()
    return out


@pytest.mark.parametrize("b,s,hq,hkv,d,causal,dtype,theta", [
    (2, 300, 8, 2, 128, True, torch.bfloat16, 1e6),    # ragged tail, GQA 4
    (1, 128, 32, 8, 128, True, torch.bfloat16, 1e6),   # the CPU-runnable configuration's shape
    (3, 129, 3, 3, 128, False, torch.float16, 1e6),    # one key past a block, not causal, G = 1
    (2, 200, 4, 2, 256, True, torch.bfloat16, 1e4),    # head dim 256
    (1, 64, 2, 1, 256, False, torch.float16, 1e4),
])
def test_full_mode_matches_oracle_and_query_mode(b, s, hq, hkv, d, causal, dtype, theta):
    xs = kf.make_inputs(b, s, hq, hkv, d, dtype=dtype, theta=theta, seed=2803)
    ref = orc.oracle_fp32(*xs, causal)
    dx = [x.cuda() for x in xs]
    full = _run("full", dx, causal)
    assert orc.within_tolerance(orc.metric(full.cpu(), ref))
    # the same kernel fed with a prepared K: identical rounding points, identical loop -> identical bits
    base = kf.optimized_attention(*dx, causal=causal, variant=1)
    torch.cuda.synchronize()
    assert torch.equal(full, base)
    for mode in ("query", "unfused"):
        assert orc.within_tolerance(orc.metric(_run(mode, dx, causal).cpu(), ref)), mode


@pytest.mark.parametrize("kw,style,rope", [
    (dict(hf_norm=False), "legacy", True),
    (dict(rope=False), "hf", False),
    (dict(rope=False, hf_norm=False), "legacy", False),
])
def test_full_mode_norm_style_and_no_rope(kw, style, rope):
    xs = kf.make_inputs(2, 260, 4, 2, 128, seed=3907)
    q, k, v, gq, gk, cos, sin = xs
    ref = orc.oracle_fp32(q, k, v, gq, gk, cos if rope else None, sin if rope else None, True)
    dx = [x.cuda() for x in xs]
    full = _run("full", dx, True, **kw)
    assert orc.within_tolerance(orc.metric(full.cpu(), ref))
    base = kf.optimized_attention(dx[0], dx[1], dx[2], dx[3], dx[4], dx[5] if rope else None, dx[6] if rope else None,
                                  causal=True, norm_style=style, variant=1)
    torch.cuda.synchronize()
    assert torch.equal(full, base)


def test_full_mode_on_head_strided_views():
    # q/k/v as a model produces them: [B, S, H, D] storage viewed as [B, H, S, D]
    xs = kf.make_inputs(2, 192, 4, 2, 128, seed=1701)
    dx = [x.cuda() for x in xs]
    strided = [t.transpose(1, 2).contiguous().transpose(1, 2) for t in dx[:3]] + dx[3:]
    a = _run("full", dx, True)
    b = _run("full", strided, True)
    assert torch.equal(a, b)
