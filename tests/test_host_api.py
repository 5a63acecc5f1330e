"""CPU tests of the boundary: the C-ABI library loads and exports what the
header declares, argument errors are rejected on the host before any launch,
and ``optimized_attention`` raises ``ValueError`` for the same misuse as the
reference (src/e1_rope_publication_v1.py:695-719;
src/e4_model_shapes_publication_v2.py:276-283)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

import kernelfuser_b200 as kf
from kernelfuser_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "kf_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kf_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert {"kf_version", "kf_last_error", "kf_prepare_rows", "kf_attention_fwd"} <= set(names)
    for n in names:
        assert hasattr(lib, n), n
    assert lib.kf_version() >= 100


def test_c_abi_rejects_bad_arguments_before_launch():
    lib = _lib.load()
    buf = (ctypes.c_char * 4096)()
    p = (ctypes.addressof(buf) + 15) & ~15
    # bad head dim
    rc = lib.kf_prepare_rows(p, p, p, None, None, 1, 1, 8, 64, 0, 1, 1e-6, 0, 0, 64, 0, 0, 64, None)
    assert rc == -1 and b"head dim" in lib.kf_last_error()
    # only one table
    rc = lib.kf_prepare_rows(p, p, p, p, None, 1, 1, 8, 128, 0, 1, 1e-6, 0, 0, 128, 0, 0, 128, None)
    assert rc == -1
    # misaligned pointer
    rc = lib.kf_prepare_rows(p + 2, p, p, None, None, 1, 1, 8, 128, 0, 1, 1e-6, 0, 0, 128, 0, 0, 128, None)
    assert rc == -2
    # stride not a multiple of 8 elements
    rc = lib.kf_prepare_rows(p, p, p, None, None, 1, 1, 8, 128, 0, 1, 1e-6, 0, 0, 132, 0, 0, 128, None)
    assert rc == -2
    # bad dtype / bad GQA ratio / null status on the attention entry point
    args = [p] * 7
    st = [1024 * 128, 128 * 8, 128]
    rc = lib.kf_attention_fwd(*args, 1, 4, 2, 8, 128, 7, 1, 1, 1, 1e-6, 0.1, *(st * 4), p, 0, None)
    assert rc == -1
    rc = lib.kf_attention_fwd(*args, 1, 4, 3, 8, 128, 0, 1, 1, 1, 1e-6, 0.1, *(st * 4), p, 0, None)
    assert rc == -1 and b"multiple" in lib.kf_last_error()
    rc = lib.kf_attention_fwd(*args, 1, 4, 2, 8, 128, 0, 1, 1, 1, 1e-6, 0.1, *(st * 4), None, 0, None)
    assert rc == -1
    rc = lib.kf_attention_fwd(*args, 1, 4, 2, 8, 128, 0, 1, 1, 1, 1e-6, -1.0, *(st * 4), p, 0, None)
    assert rc == -1
    # expanded (broadcast) views: a zero stride over a batch or head dimension larger than 1 is refused,
    # for any of q / kn / v / out and for the row-prepare input; a size-1 dimension may carry stride 0
    for which in range(4):
        for dim in (0, 1):
            strides = [list(st) for _ in range(4)]
            strides[which][dim] = 0
            flat = [x for t in strides for x in t]
            rc = lib.kf_attention_fwd(*args, 2, 4, 2, 8, 128, 0, 1, 1, 1, 1e-6, 0.1, *flat, p, 0, None)
            assert rc == -2 and b"size 1" in lib.kf_last_error(), (which, dim)
    rc = lib.kf_prepare_rows(p, p, p, None, None, 2, 1, 8, 128, 0, 1, 1e-6, 0, 0, 128, 1024, 0, 128, None)
    assert rc == -2
    rc = lib.kf_selftest_wait_timeout(None, 1000, None)
    assert rc == -1
    rc = lib.kf_selftest_wait_timeout(p, 0, None)
    assert rc == -1
    # the one-launch form: both weights are required, and the same stride rule holds
    rc = lib.kf_attention_full(p, p, p, p, None, None, None, p, 1, 4, 2, 8, 128, 0, 1, 1, 1e-6, 0.1, *(st * 4), p, None)
    assert rc == -1 and b"gamma" in lib.kf_last_error()
    rc = lib.kf_attention_full(p, p, p, p, p, None, None, p, 2, 4, 2, 8, 128, 0, 1, 1, 1e-6, 0.1,
                               0, st[1], st[2], *(st * 3), p, None)
    assert rc == -2 and b"size 1" in lib.kf_last_error()


def test_expanded_views_are_refused_by_the_adapters():
    # the strides are inspected on the host before any CUDA call
    q, k, v, gq, gk, cos, sin = _inputs()
    ke = k[:, :1].expand(-1, 2, -1, -1)  # stride 0 over two KV heads
    for fn in (lambda: kf.fused(q, ke, v, gq, gk, cos, sin, True), lambda: kf.factored_attention(q, ke, v, gq, gk)):
        with pytest.raises(ValueError, match="expanded"):
            fn()


def test_library_is_rebuilt_when_sources_change(tmp_path, monkeypatch):
    from kernelfuser_b200 import build
    assert not build.stale()  # the loaded library matches the tree
    monkeypatch.setattr(build, "STAMP", tmp_path / "missing.srchash")
    assert build.stale()
    (tmp_path / "missing.srchash").write_text("0" * 64)
    assert build.stale()


def _inputs(**kw):
    return kf.make_inputs(1, 33, 4, 2, 128, **kw)


@pytest.mark.parametrize("kwargs", [{"mode": "bad"}, {"bn": 31}, {"norm_style": "bad"}, {"mode": "full"}])
def test_invalid_kwargs_raise_value_error(kwargs):
    with pytest.raises(ValueError):
        kf.optimized_attention(*_inputs(), **kwargs)


def test_misuse_raises_value_error():
    q, k, v, gq, gk, cos, sin = _inputs()
    with pytest.raises(ValueError, match="both rotary"):
        kf.optimized_attention(q, k, v, gq, gk, cos, None)
    with pytest.raises(ValueError, match="forward-only"):
        kf.optimized_attention(q.float().requires_grad_(), k, v, gq, gk, cos, sin)
    with pytest.raises(ValueError, match="Expected Q"):
        kf.optimized_attention(q[0], k, v, gq, gk, cos, sin)
    with pytest.raises(ValueError, match="Expected Q"):
        kf.optimized_attention(q, k, v[:, :1], gq, gk, cos, sin)
    with pytest.raises(ValueError, match="valid GQA"):
        kf.optimized_attention(q[:, :3], k, v, gq, gk, cos, sin)
    with pytest.raises(ValueError, match="valid GQA"):
        kf.optimized_attention(q[..., :64], k[..., :64], v[..., :64], gq[:64], gk[:64], cos[:, :64], sin[:, :64])
    with pytest.raises(ValueError, match="gamma"):
        kf.optimized_attention(q, k, v, gq[:64], gk, cos, sin)
    with pytest.raises(ValueError, match="gamma"):
        kf.optimized_attention(q, k, v, gq, gk, cos[:5], sin[:5])
    # CPU tensors are not accepted: there is no CPU path
    with pytest.raises(ValueError, match="CUDA"):
        kf.optimized_attention(q, k, v, gq, gk, cos, sin)
    with pytest.raises(ValueError, match="positions"):
        kf.optimized_attention(q, k, v, gq, gk, positions=torch.arange(33))
    with pytest.raises(ValueError, match="positions"):
        kf.optimized_attention(q, k, v, gq, gk, cos, sin, positions=torch.arange(33), theta=1e6)
    # the factored form: CPU tensors, mismatched scratch
    with pytest.raises(ValueError, match="CUDA"):
        kf.factored_attention(q, k, v, gq, gk, causal=True)
    with pytest.raises(ValueError, match="Expected Q"):
        kf.factored_attention(q, k[:, :, :5], v, gq, gk)
    # the reference's launcher: its two errors, and CPU tensors
    with pytest.raises(ValueError, match="Invalid fusion mode"):
        kf.launch_attention((q, k, v, gq, gk, cos, sin), torch.empty_like(q), mode="key")
    with pytest.raises(ValueError, match="CUDA"):
        kf.launch_attention((q, k, v, gq, gk, cos, sin), torch.empty_like(q), mode="full")
    with pytest.raises(ValueError, match="Missing scratch"):
        kf.launch_attention((q, k, v, gq, gk, cos, sin), torch.empty_like(q), mode="query")
    with pytest.raises(ValueError, match="Missing scratch"):
        kf.launch_attention((q, k, v, gq, gk, cos, sin), torch.empty_like(q), mode="unfused", kn=torch.empty_like(k))
    # the arm adapter: unknown output layout, and CPU tensors
    with pytest.raises(ValueError, match="out_layout"):
        kf.fused(q, k, v, gq, gk, cos, sin, True, out_layout="sbhd")
    with pytest.raises(ValueError, match="CUDA"):
        kf.fused(q, k, v, gq, gk, cos, sin, True, out_layout="bshd")


def test_no_cpu_fallback_in_product():
    # the product package never imports the oracle
    for f in (ROOT / "kernelfuser_b200").glob("*.py"):
        assert "oracle" not in f.read_text(), f
