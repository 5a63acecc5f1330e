"""Algorithmic work and roofline denominators for the attention path."""
from __future__ import annotations

import json
from pathlib import Path

# Fallback denominators (an earlier measurement on the same GPU pool), used
# only when no measured-peaks file is present.
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def attention_flops(b, hq, s, d, causal=True) -> float:
    """4*B*Hq*S^2*D for dense attention (QK^T and PV), half when causal."""
    f = 4.0 * b * hq * s * s * d
    return f / 2 if causal else f


def prepare_bytes(b, h, s, d, elem_bytes=2) -> float:
    """One read of x and one write of y; tables and gamma excluded."""
    return 2.0 * b * h * s * d * elem_bytes


def load_peaks(repo_root=None) -> dict:
    """Measured peaks if the file is present, else the stated fallback."""
    root = Path(repo_root) if repo_root else Path(__file__).resolve().parent.parent
    p = root / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            m = json.loads(p.read_text())
            return {"source": "measured", "hbm_gbs": float(m["hbm_gbs"]),
                    "bf16_tflops": float(m["bf16_tflops"]),
                    "bf16_tflops_sustained": float(m.get("bf16_tflops_sustained", m["bf16_tflops"]))}
        except Exception:
            pass
    return {"source": "fallback", "hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
            "bf16_tflops_sustained": 1400.0}
