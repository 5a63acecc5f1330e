"""Generate the golden fixtures in this directory from the reference itself.

Run in a container that has the reference checkout (CPU is enough):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's ``src/e1_rope_publication_v1.py`` and evaluates its
``oracle_fp32`` (and ``refinement_oracle`` for the no-RoPE case) on seeded
inputs made by ``kernelfuser_b200.inputs.make_inputs``.  Small cases store the
inputs (16-bit patterns) and the full fp32 outputs; the C1 known-answer case
(B=1, S=128, Hq=32, Hkv=8, D=128, fp32, seed 0) stores a checksum of the
inputs and a strided sample of the outputs.  The reference is only needed to
regenerate the fixtures, never to run the tests.
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from kernelfuser_b200.inputs import WORKLOADS, make_inputs, make_workload_inputs  # noqa: E402

SMALL_CASES = {
    # name: (B, S, Hq, Hkv, D, dtype, theta, rope, seed)
    "rope_s33_d128_bf16": (1, 33, 4, 2, 128, "bfloat16", 1e6, True, 9909),
    "rope_s129_d256_bf16": (1, 129, 2, 1, 256, "bfloat16", 1e4, True, 4909),
    "norope_s33_d128_bf16": (1, 33, 4, 2, 128, "bfloat16", 1e6, False, 9909),
    "rope_s40_d128_fp16": (2, 40, 4, 4, 128, "float16", 1e6, True, 1701),
}


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def main(ref_root: str) -> None:
    sys.path.insert(0, str(Path(ref_root) / "src"))
    import e1_rope_publication_v1 as ref  # the reference module, unmodified

    torch.set_num_threads(1)  # fixed reduction order for the stored outputs
    for name, (b, s, hq, hkv, d, dt, theta, rope, seed) in SMALL_CASES.items():
        dtype = getattr(torch, dt)
        q, k, v, gq, gk, cos, sin = make_inputs(b, s, hq, hkv, d, dtype=dtype, theta=theta,
                                                seed=seed, rope=rope)
        arrays = {"q": bits16(q), "k": bits16(k), "v": bits16(v), "gq": bits16(gq), "gk": bits16(gk)}
        if rope:
            arrays["cos"] = bits16(cos)
            arrays["sin"] = bits16(sin)
        for causal in (False, True):
            if rope:
                o = ref.oracle_fp32(q, k, v, gq, gk, cos, sin, causal)
            else:
                o = ref.refinement_oracle((q, k, v, gq, gk, q, k), causal, False)
            arrays["out_causal" if causal else "out_full"] = o.numpy().astype(np.float32)
        meta = dict(B=b, S=s, Hq=hq, Hkv=hkv, D=d, dtype=dt, theta=theta, rope=rope, seed=seed)
        arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
        np.savez_compressed(HERE / f"{name}.npz", **arrays)
        print("wrote", name)

    # C1: the CPU known-answer configuration, fp32 inputs from seed 0.
    w = WORKLOADS["C1"]
    xs = make_workload_inputs(w, seed=0)
    o = ref.oracle_fp32(*xs, True)
    flat = o.flatten()
    idx = torch.arange(0, flat.numel(), 97)
    c1 = {
        "workload": "C1", "seed": 0, "causal": True,
        "input_sha256": {n: sha(t) for n, t in zip(("q", "k", "v", "gq", "gk", "cos", "sin"), xs)},
        "sample_stride": 97,
        "out_sum": float(flat.double().sum()),
        "out_abs_sum": float(flat.double().abs().sum()),
    }
    np.savez_compressed(HERE / "c1_fp32_seed0.npz",
                        sample=flat[idx].numpy().astype(np.float32),
                        meta=np.frombuffer(json.dumps(c1).encode(), dtype=np.uint8))
    print("wrote c1_fp32_seed0")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
