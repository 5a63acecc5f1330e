"""Operator API: ``optimized_attention`` and the runner-arm adapter ``fused``.

Mirrors the reference's public operator
(``optimized_attention``, src/e1_rope_publication_v1.py:680-726): the same
positional/keyword signature, the same ``ValueError`` for every misuse it
rejects (:695-719, with "compute capability 9" replaced by "10" and the dtype
widened to bf16 or fp16), the same allocation pattern (``out`` and the
prepared-K scratch via ``torch.empty_like``), two asynchronous launches on the
current stream and no host synchronisation.  Keyword-only extensions whose
defaults reproduce the reference: ``positions``/``theta`` (build the rotary
tables as ``make_inputs`` does, :180-183), ``eps``, ``scale``, ``out``, ``kn``.

The kernels live in libkf_b200.so (hand-written CUDA for sm_100a) and are
reached through ctypes; there is no fallback path.
"""
from __future__ import annotations

import os

import torch

from . import _lib
from .inputs import rope_tables

_DTYPES = {torch.bfloat16: _lib.KF_BF16, torch.float16: _lib.KF_FP16}
_status = {}  # device index -> int32[1] status word


def _default_variant() -> int:
    """Kernel variant used when a call does not name one (0 = automatic);
    the environment variable KF_B200_ATTN_VARIANT overrides it for experiments."""
    return int(os.environ.get("KF_B200_ATTN_VARIANT", "0"))


class KernelStatusError(RuntimeError):
    """A kernel gave up on a bounded wait and reported a status code."""


def status_word(device: torch.device) -> torch.Tensor:
    """The per-device int32 status word the kernels report into (0 = ok)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device=None) -> None:
    """Synchronise and raise if any kernel reported a failure on ``device``."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(dev)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise KernelStatusError(f"kernel reported status {code} (a bounded wait expired)")


def selftest_wait_timeout(limit_clocks: int = 100_000, device=None) -> None:
    """Run the library's self-test of the failure path (``kf_selftest_wait_timeout``): one warp waits on a
    barrier nobody arrives on and gives up after ``limit_clocks`` SM clocks, leaving code 901 in the
    device's status word.  The next ``check_status()`` raises ``KernelStatusError`` and clears the word;
    until then every attention launch on the device returns without doing anything."""
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        st = status_word(dev)
        _call(lib.kf_selftest_wait_timeout(st.data_ptr(), int(limit_clocks), torch.cuda.current_stream().cuda_stream))


def _strides3(t: torch.Tensor):
    return t.stride(0), t.stride(1), t.stride(2)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _call(rc: int) -> None:
    if rc != 0:
        msg = _lib.last_error()
        if rc in (-1, -2, -4):
            raise ValueError(msg)
        raise RuntimeError(f"libkf_b200 error {rc}: {msg}")


def prepare_rows(x, gamma, cos=None, sin=None, *, norm_style="hf", eps=1e-6, out=None):
    """RMSNorm + gamma + split-half RoPE of every row of ``x`` [B,H,S,D]
    (position = row index).  The reference's ``prepare_attention``
    (src/e1_rope_publication_v1.py:652-658) for one tensor."""
    lib = _lib.load()
    b, h, s, d = x.shape
    y = torch.empty_like(x) if out is None else out
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        _call(lib.kf_prepare_rows(_ptr(x), _ptr(y), _ptr(gamma), _ptr(cos), _ptr(sin), b, h, s, d,
                                  _DTYPES[x.dtype], int(norm_style == "hf"), float(eps),
                                  *_strides3(x), *_strides3(y), stream))
    return y


def attention_forward(q, kn, v, gq, cos, sin, out, *, causal, norm_style="hf", fuse_q=True, eps=1e-6,
                      scale=None, variant=0):
    """Launch the attention kernel on prepared K (``kn``); see kf_attention_fwd."""
    lib = _lib.load()
    b, hq, s, d = q.shape
    hkv = kn.shape[1]
    sc = float(d ** -0.5 if scale is None else scale)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        st = status_word(q.device)
        _call(lib.kf_attention_fwd(_ptr(q), _ptr(kn), _ptr(v), _ptr(gq), _ptr(cos), _ptr(sin), _ptr(out),
                                   b, hq, hkv, s, d, _DTYPES[q.dtype], int(bool(causal)),
                                   int(norm_style == "hf"), int(bool(fuse_q)), float(eps), sc,
                                   *_strides3(q), *_strides3(kn), *_strides3(v), *_strides3(out),
                                   st.data_ptr(), int(variant) if variant else _default_variant(), stream))
    return out


def _check_strided(q, k, v):
    """Layout rules for the entry points that read strided q/k/v in place (head-transposed views of
    [B,S,H,D] projections): contiguous head dimension, 16-byte aligned strides, no expanded dimension."""
    for t in (q, k, v):
        if t.ndim != 4:
            continue  # reported by the shape checks
        if t.stride(3) != 1 or any(st % 8 for st in t.stride()[:3]):
            raise ValueError("q/k/v need a contiguous head dimension and 16-byte aligned strides")
        if any(st == 0 and n > 1 for st, n in zip(t.stride()[:3], t.shape[:3])):
            raise ValueError("q/k/v must not be expanded (stride 0 over a dimension larger than 1)")


def _validate(q, k, v, gq, gk, cos, sin, mode, bn, norm_style, require_contiguous=True):
    # Same predicates, in the same order, as the reference (:695-719).
    if mode not in ("query", "unfused") or bn not in (64, 128):
        raise ValueError("Expected query/unfused mode and BN=64/128")
    if norm_style not in ("hf", "legacy"):
        raise ValueError("Expected hf or legacy norm_style")
    if (cos is None) != (sin is None):
        raise ValueError("Provide both rotary tables or neither")
    rotary = cos is not None
    tensors = (q, k, v, gq, gk) + ((cos, sin) if rotary else ())
    if any(t.requires_grad for t in tensors):
        raise ValueError("This API is forward-only")
    if q.ndim != 4 or k.ndim != 4 or k.shape != v.shape:
        raise ValueError("Expected Q [B,Hq,S,D] and K/V [B,Hkv,S,D]")
    b, h, s, d = q.shape
    if (d not in (128, 256) or min(b, h, s) < 1 or k.shape[0] != b or
            tuple(k.shape[2:]) != (s, d) or k.shape[1] < 1 or h % k.shape[1]):
        raise ValueError("Expected D=128/256, matching batch/sequence and valid GQA")
    if tuple(gq.shape) != (d,) or tuple(gk.shape) != (d,) or (
            rotary and (tuple(cos.shape) != (s, d) or tuple(sin.shape) != (s, d))):
        raise ValueError("Expected gamma [D] and optional rotary tables [S,D]")
    if (q.dtype not in _DTYPES or
            any(not t.is_cuda or t.device != q.device or t.dtype != q.dtype for t in tensors) or
            (require_contiguous and any(not t.is_contiguous() for t in tensors))):
        raise ValueError("Inputs must be contiguous BF16 (or FP16) on one CUDA device")
    if torch.cuda.get_device_capability(q.device)[0] != 10:
        raise ValueError("This implementation is written for SM100/Blackwell")
    return rotary


def optimized_attention(q, k, v, gq, gk, cos=None, sin=None, *, causal=False,
                        mode="query", bn=128, gather=False, norm_style="hf",
                        positions=None, theta=None, eps=1e-6, scale=None, out=None, kn=None,
                        variant=0):
    """Forward attention with per-head Q/K RMSNorm and optional split-half RoPE.

    ``mode='query'`` prepares K once, then fuses Q normalisation and rotation
    into the attention prologue (no normalised-Q tensor is written);
    ``mode='unfused'`` prepares both Q and K first.  Pass both ``cos`` and
    ``sin`` [S, D] to enable RoPE, or ``positions`` [S] with ``theta`` to have
    the tables built here.  ``norm_style='hf'`` rounds the normalised
    activation before the gamma multiply; ``'legacy'`` rounds once after the
    fp32 product.  ``bn`` and ``gather`` are accepted and validated for
    compatibility with the reference signature
    (src/e1_rope_publication_v1.py:680-681); they select Triton tiling details
    there and do not change the result.  ``out`` / ``kn`` let a caller supply
    preallocated output and prepared-K scratch.
    """
    if positions is not None or theta is not None:
        if positions is None or theta is None or cos is not None or sin is not None:
            raise ValueError("Provide positions together with theta, and no tables")
        cos, sin = rope_tables(positions.to(q.device), q.shape[-1], float(theta), q.dtype)
    _validate(q, k, v, gq, gk, cos, sin, mode, bn, norm_style)
    if not (eps > 0):
        raise ValueError("eps must be positive")
    out = torch.empty_like(q) if out is None else out
    kn = torch.empty_like(k) if kn is None else kn
    if out.shape != q.shape or out.dtype != q.dtype or kn.shape != k.shape or kn.dtype != k.dtype:
        raise ValueError("out / kn must match q / k in shape and dtype")
    with torch.cuda.device(q.device):
        if mode == "unfused":
            prepare_rows(k, gk, cos, sin, norm_style=norm_style, eps=eps, out=kn)
            qn = prepare_rows(q, gq, cos, sin, norm_style=norm_style, eps=eps)
            attention_forward(qn, kn, v, gq, cos, sin, out, causal=causal, norm_style=norm_style,
                              fuse_q=False, eps=eps, scale=scale, variant=variant)
        else:
            # one C call for both launches
            b, hq, s, d = q.shape
            sc = float(d ** -0.5 if scale is None else scale)
            _call(_lib.load().kf_optimized_attention(
                _ptr(q), _ptr(k), _ptr(v), _ptr(gq), _ptr(gk), _ptr(cos), _ptr(sin), _ptr(kn), _ptr(out),
                b, hq, k.shape[1], s, d, _DTYPES[q.dtype], int(bool(causal)), int(norm_style == "hf"), float(eps), sc,
                *_strides3(q), *_strides3(k), *_strides3(v), *_strides3(kn), *_strides3(out),
                status_word(q.device).data_ptr(), int(variant) if variant else _default_variant(),
                torch.cuda.current_stream().cuda_stream))
    return out


def attention_full(q, k, v, gq, gk, cos, sin, out, *, causal, norm_style="hf", eps=1e-6, scale=None):
    """One launch on the RAW q and k: the kernel transforms every K tile in its loop (see kf_attention_full)."""
    lib = _lib.load()
    b, hq, s, d = q.shape
    sc = float(d ** -0.5 if scale is None else scale)
    with torch.cuda.device(q.device):
        _call(lib.kf_attention_full(_ptr(q), _ptr(k), _ptr(v), _ptr(gq), _ptr(gk), _ptr(cos), _ptr(sin), _ptr(out),
                                    b, hq, k.shape[1], s, d, _DTYPES[q.dtype], int(bool(causal)),
                                    int(norm_style == "hf"), float(eps), sc,
                                    *_strides3(q), *_strides3(k), *_strides3(v), *_strides3(out),
                                    status_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream))
    return out


def launch_attention(inputs, out, *, causal=False, mode="query", bm=64, bn=64, warps=4, stages=1, gather=True,
                     rope=True, hf_norm=True, qn=None, kn=None):
    """The reference's launcher (src/e1_rope_publication_v1.py:661-677) with its signature and errors: full fusion
    (``mode='full'``: one launch, K transformed per tile, no scratch), query-only fusion (``'query'``: K prepared
    into ``kn``, Q transformed in the attention prologue) or the two-kernel unfused control (``'unfused'``: Q into
    ``qn`` and K into ``kn`` first).  ``inputs`` = ``(q, k, v, gq, gk, cos, sin)``; ``rope=False`` ignores the tables;
    ``bm``, ``bn``, ``warps``, ``stages`` and ``gather`` tune the Triton kernels there and do not change the
    result, so they are accepted and ignored.  Like the reference's launcher it checks the mode and the scratch
    buffers only (plus: the tensors must be on a GPU); shapes and dtypes are what ``optimized_attention`` checks."""
    if mode not in ("full", "query", "unfused"):
        raise ValueError("Invalid fusion mode")
    q, k, v, gq, gk, cos, sin = inputs
    if not rope:
        cos = sin = None
    if mode != "full" and (kn is None or (mode == "unfused" and qn is None)):
        raise ValueError("Missing scratch buffers")
    if not all(t.is_cuda for t in (q, k, v, gq, gk, out)):
        raise ValueError("Expected CUDA tensors")  # there is no CPU path
    style = "hf" if hf_norm else "legacy"
    if mode == "full":
        _check_strided(q, k, v)
        return attention_full(q, k, v, gq, gk, cos, sin, out, causal=causal, norm_style=style)
    if mode == "unfused":
        prepare_rows(k, gk, cos, sin, norm_style=style, out=kn)
        prepare_rows(q, gq, cos, sin, norm_style=style, out=qn)
        return attention_forward(qn, kn, v, gq, cos, sin, out, causal=causal, norm_style=style, fuse_q=False)
    # both launches in one C call (the attention kernel then starts as a dependent of the prepare)
    b, hq, s, d = q.shape
    with torch.cuda.device(q.device):
        _call(_lib.load().kf_optimized_attention(
            _ptr(q), _ptr(k), _ptr(v), _ptr(gq), _ptr(gk), _ptr(cos), _ptr(sin), _ptr(kn), _ptr(out),
            b, hq, k.shape[1], s, d, _DTYPES[q.dtype], int(bool(causal)), int(bool(hf_norm)), 1e-6, float(d ** -0.5),
            *_strides3(q), *_strides3(k), *_strides3(v), *_strides3(kn), *_strides3(out),
            status_word(q.device).data_ptr(), _default_variant(), torch.cuda.current_stream().cuda_stream))
    return out


def fused(q, k, v, gq, gk, cos, sin, causal, eps=1e-6, scale=None, norm_style="qwen3", *, out_layout="bhsd"):
    """Runner-arm adapter with the signature of the reference's arms
    (``fused``/``separate``/``vendor``/``compiled_fn``,
    src/e1_rope_publication_v1.py:185-225).  Accepts [S,D], [B,S,D] or
    [B,1,S,D] tables (the first broadcast slice is used, :192-200), an
    explicit ``scale``/``eps``, and head-transposed (non-contiguous) q/k/v
    views as produced by a model's ``view(...).transpose(1, 2)``, so the
    projections' [B,S,H,D] outputs are read in place.

    ``out_layout='bshd'`` (keyword-only extension) makes the kernel write the
    result where the model's output projection wants it: the returned tensor
    is contiguous [B, S, Hq*D], i.e. the ``transpose(1, 2).reshape(B, S, -1)``
    that follows the attention call in a decoder layer
    (src/e2_qwen3_rope_prefill.py:159) costs no copy."""
    if out_layout not in ("bhsd", "bshd"):
        raise ValueError("out_layout must be 'bhsd' or 'bshd'")
    if cos is not None:
        if cos.ndim == 4: cos = cos[:, 0]
        if sin.ndim == 4: sin = sin[:, 0]
        if cos.ndim == 3: cos = cos[0]
        if sin.ndim == 3: sin = sin[0]
        cos = cos.to(q.dtype).contiguous()
        sin = sin.to(q.dtype).contiguous()
    style = "legacy" if norm_style == "legacy" else "hf"
    _check_strided(q, k, v)
    _validate(q, k, v, gq.contiguous(), gk.contiguous(), cos, sin, "query", 128, style, require_contiguous=False)
    b, hq, s, d = q.shape
    if out_layout == "bshd":
        flat = torch.empty((b, s, hq * d), dtype=q.dtype, device=q.device)
        out = flat.view(b, s, hq, d).transpose(1, 2)  # [B,Hq,S,D] view with row stride Hq*D
    else:
        flat = out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    kn = torch.empty(k.shape, dtype=k.dtype, device=k.device)
    gq, gk = gq.contiguous(), gk.contiguous()
    sc = float(d ** -0.5 if scale is None else scale)
    with torch.cuda.device(q.device):
        # both launches in one C call (the attention kernel then starts as a dependent of the prepare)
        _call(_lib.load().kf_optimized_attention(
            _ptr(q), _ptr(k), _ptr(v), _ptr(gq), _ptr(gk), _ptr(cos), _ptr(sin), _ptr(kn), _ptr(out),
            b, hq, k.shape[1], s, d, _DTYPES[q.dtype], int(bool(causal)), int(style == "hf"), float(eps), sc,
            *_strides3(q), *_strides3(k), *_strides3(v), *_strides3(kn), *_strides3(out),
            status_word(q.device).data_ptr(), _default_variant(), torch.cuda.current_stream().cuda_stream))
    return flat


def factored_attention(q, k, v, gq, gk, *, causal=False, eps=1e-6, scale=None, out=None, kn=None, variant=0):
    """No-RoPE attention in the reference's FACTORED form (``launch_factored_attention``,
    src/e1_qk_publication_v3.py:638-650): the query weight is folded into the prepared keys,
    ``KN = r(k * inv_rms(k) * gk * gq)``, the raw ``q`` feeds Q K^T and every query row's scores
    are scaled by ``inv_rms(q_row) * scale * log2(e)``.  Mathematically the same operator as
    ``optimized_attention`` without tables, with fewer roundings on the Q side and no rounded
    Q at all; opt-in because the rounding points differ.  The reference's FP32 ``INV``
    tensor does not exist here: the inverse RMS is computed in the attention prologue."""
    lib = _lib.load()
    gq, gk = gq.contiguous(), gk.contiguous()
    _check_strided(q, k, v)
    _validate(q, k, v, gq, gk, None, None, "query", 128, "legacy", require_contiguous=False)
    if not (eps > 0):
        raise ValueError("eps must be positive")
    out = torch.empty(q.shape, dtype=q.dtype, device=q.device) if out is None else out
    kn = torch.empty(k.shape, dtype=k.dtype, device=k.device) if kn is None else kn
    if out.shape != q.shape or out.dtype != q.dtype or kn.shape != k.shape or kn.dtype != k.dtype:
        raise ValueError("out / kn must match q / k in shape and dtype")
    b, hq, s, d = q.shape
    sc = float(d ** -0.5 if scale is None else scale)
    with torch.cuda.device(q.device):
        st = status_word(q.device)
        stream = torch.cuda.current_stream().cuda_stream
        _call(lib.kf_factored_attention(
            _ptr(q), _ptr(k), _ptr(v), _ptr(gq), _ptr(gk), _ptr(kn), _ptr(out),
            b, hq, k.shape[1], s, d, _DTYPES[q.dtype], int(bool(causal)), float(eps), sc,
            *_strides3(q), *_strides3(k), *_strides3(v), *_strides3(kn), *_strides3(out),
            st.data_ptr(), int(variant), stream))
    return out


def optimized_attention_static(q, k, v, gq, gk, cos, sin, out, *, causal=False, norm_style="hf",
                               eps=1e-6, scale=None):
    """The whole operator through ``kf_optimized_attention_static``: the
    prepared K goes to a fixed 32 MiB array inside the library instead of a
    freshly allocated tensor, so this call allocates nothing (``out`` is the
    caller's).  Meant for callers that cannot allocate device memory where
    they call from (a host framework that owns the device heap, a section
    where cudaMalloc is off-limits, a request path that must stay out of the
    allocator).  ``B*Hkv*S*D*2`` bytes must fit in the array (``ValueError``
    otherwise).  All calls on a device share that array: do not let two of
    them overlap on the GPU.  The first call on a device looks up the array's
    address and should be made outside any stream capture."""
    lib = _lib.load()
    _validate(q, k, v, gq, gk, cos, sin, "query", 128, norm_style)
    if out.shape != q.shape or out.dtype != q.dtype or out.device != q.device or not out.is_contiguous():
        raise ValueError("out must match q in shape, dtype and device and be contiguous")
    b, hq, s, d = q.shape
    sc = float(d ** -0.5 if scale is None else scale)
    with torch.cuda.device(q.device):
        st = status_word(q.device)
        stream = torch.cuda.current_stream().cuda_stream
        _call(lib.kf_optimized_attention_static(
            _ptr(q), _ptr(k), _ptr(v), _ptr(gq), _ptr(gk), _ptr(cos), _ptr(sin), _ptr(out),
            b, hq, k.shape[1], s, d, _DTYPES[q.dtype], int(bool(causal)), int(norm_style == "hf"),
            float(eps), sc, *_strides3(q), *_strides3(k), *_strides3(v), *_strides3(out),
            st.data_ptr(), stream))
    return out


# --------------------------------------------------------------------------
# Host-buffer entry point: batch-chunked, copy/compute overlapped
# --------------------------------------------------------------------------
class _HostPipeline:
    """Device staging buffers, streams and events for one (device, chunk shape, dtype)."""

    def __init__(self, device, qshape, kshape, dtype):
        self.key = (device, tuple(qshape), tuple(kshape), dtype)
        mk = lambda shape: [torch.empty(shape, dtype=dtype, device=device) for _ in range(2)]
        self.q, self.k, self.v = mk(qshape), mk(kshape), mk(kshape)
        self.kn, self.o = mk(kshape), mk(qshape)
        self.h2d = torch.cuda.Stream(device=device)
        self.d2h = torch.cuda.Stream(device=device)
        self.compute = torch.cuda.Stream(device=device)


_pipelines = {}          # insertion-ordered: least recently used first
_MAX_PIPELINES = 4       # staging-buffer sets kept; older ones are dropped (their device memory is freed)


def release_host_pipelines() -> None:
    """Drop the cached device staging buffers of ``optimized_attention_host``."""
    _pipelines.clear()


def optimized_attention_host(q, k, v, gq, gk, cos=None, sin=None, *, causal=False, norm_style="hf",
                             eps=1e-6, scale=None, out=None, device=None, chunk_batch=None):
    """``optimized_attention`` for HOST tensors: q/k/v (and the returned output) live in CPU
    memory, pinned for full copy speed.  The batch is cut into chunks and three streams overlap
    the host-to-device copy of chunk i+1, the kernels of chunk i and the device-to-host copy of
    chunk i-1 (PCIe is full duplex), with two sets of device staging buffers that are kept and
    reused across calls.  Same semantics and errors as ``optimized_attention``; gamma vectors
    and rotary tables may be CPU or device tensors.  Returns the output as a pinned CPU tensor
    ([B, Hq, S, D]) after synchronising the copies."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("optimized_attention_host takes host tensors; use optimized_attention for device tensors")
    if q.ndim != 4 or k.ndim != 4 or k.shape != v.shape or q.shape[0] != k.shape[0]:
        raise ValueError("Expected Q [B,Hq,S,D] and K/V [B,Hkv,S,D]")
    b = q.shape[0]
    cb = chunk_batch or max(1, b // 8)
    q, k, v = (t if t.is_pinned() else t.contiguous().pin_memory() for t in (q, k, v))
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    small = [None if t is None else t.to(dev, non_blocking=True) for t in (gq, gk, cos, sin)]
    qshape, kshape = (cb,) + tuple(q.shape[1:]), (cb,) + tuple(k.shape[1:])
    key = (dev, qshape, kshape, q.dtype)
    pl = _pipelines.pop(key, None)
    if pl is None:
        pl = _HostPipeline(dev, qshape, kshape, q.dtype)
    _pipelines[key] = pl  # most recently used last
    while len(_pipelines) > _MAX_PIPELINES:
        _pipelines.pop(next(iter(_pipelines)))
    cur = torch.cuda.current_stream(dev)
    for st in (pl.h2d, pl.compute, pl.d2h):
        st.wait_stream(cur)  # the small tensors above, and any earlier use of the staging buffers
    n_chunks = (b + cb - 1) // cb
    ev_comp = [None] * n_chunks
    ev_d2h = [None] * n_chunks
    for c in range(n_chunks):
        lo, hi = c * cb, min((c + 1) * cb, b)
        n, sl = hi - lo, c & 1
        with torch.cuda.stream(pl.h2d):
            if c >= 2:
                pl.h2d.wait_event(ev_comp[c - 2])  # the kernels that read this buffer set are done
            pl.q[sl][:n].copy_(q[lo:hi], non_blocking=True)
            pl.k[sl][:n].copy_(k[lo:hi], non_blocking=True)
            pl.v[sl][:n].copy_(v[lo:hi], non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(pl.h2d)
        with torch.cuda.stream(pl.compute):
            pl.compute.wait_event(ev_in)
            if c >= 2:
                pl.compute.wait_event(ev_d2h[c - 2])  # the output buffer has been copied out
            optimized_attention(pl.q[sl][:n], pl.k[sl][:n], pl.v[sl][:n], *small, causal=causal,
                                norm_style=norm_style, eps=eps, scale=scale, out=pl.o[sl][:n], kn=pl.kn[sl][:n])
            ev_comp[c] = torch.cuda.Event()
            ev_comp[c].record(pl.compute)
        with torch.cuda.stream(pl.d2h):
            pl.d2h.wait_event(ev_comp[c])
            out[lo:hi].copy_(pl.o[sl][:n], non_blocking=True)
            ev_d2h[c] = torch.cuda.Event()
            ev_d2h[c].record(pl.d2h)
    cur.wait_stream(pl.d2h)
    cur.wait_stream(pl.compute)
    cur.wait_stream(pl.h2d)
    cur.synchronize()
    return out
