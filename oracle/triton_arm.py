"""Run the reference's compiled (Triton) arm next to the CUDA path on one GPU.

TEST INFRASTRUCTURE ONLY (a checker, like the rest of this folder).  It needs
an untouched copy of the reference's ``src`` folder under ``baseline/_ref/src``
(git-ignored) and a GPU; it imports ``launch_attention``
(src/e1_rope_publication_v1.py:661-677, kernels :586-649) from there and calls
it exactly as ``optimized_attention`` does (:722-725: mode, bm=64, bn=128,
gather=False, preallocated ``kn``), skipping only the capability gate of :716.

For every case it records
  * the error of the Triton arm and of the CUDA path against the FP32 oracle
    (max-abs, mean-abs, relative L2) on identical seeded inputs,
  * how far the CPU emulation of the arm's rounding contract
    (``oracle.emulate_rows`` / ``emulate_optimized_attention``) is from the
    real arm,
  * per-call device time of both by the reference's graph-replay protocol
    (src/fusion_harness.py:32-79).

    python oracle/triton_arm.py [--out OUT/triton_arm.json] [--quick]
    python oracle/triton_arm.py --golden OUT/triton_arm_b200.npz
    python oracle/triton_arm.py --fusion-table OUT/fusion_table.json [--with-full]

The second form writes the fixture ``tests/golden/triton_arm_b200.npz`` is a copy
of: prepared K and outputs of the real arm on small seeded cases (inputs are
regenerated from the seed by the tests), which pin ``emulate_rows`` /
``emulate_optimized_attention`` and bound the CUDA path's error.
"""
from __future__ import annotations

import argparse
import tempfile
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
REF_SRC = ROOT / "baseline" / "_ref" / "src"

CASES = [
    # name, B, S, Hq, Hkv, D, theta, oracle batches, emulate, time
    ("C1_bf16", 1, 128, 32, 8, 128, 1e6, 1, True, True),
    ("C2", 1, 2048, 32, 8, 128, 1e6, 1, True, True),
    ("C3_bf16", 4, 1000, 32, 8, 128, 1e6, 4, False, True),
    ("D256_s1024", 1, 1024, 16, 8, 256, 1e4, 1, True, True),
    ("C4", 16, 4096, 32, 8, 128, 1e6, 1, False, True),
    ("C5", 8, 8192, 16, 8, 256, 1e4, 0, False, True),
]


def load_reference():
    if not (REF_SRC / "e1_rope_publication_v1.py").exists():
        raise SystemExit(f"{REF_SRC} is missing: copy the reference's src folder there first")
    sys.path.insert(0, str(REF_SRC))
    import e1_rope_publication_v1 as ref  # noqa: E402
    return ref


def run_case(ref, orc, kf, paired, case, quick=False):
    name, b, s, hq, hkv, d, theta, nb_oracle, emulate, do_time = case
    dt = torch.bfloat16  # the reference arm computes in bf16 only (`_rows` casts to tl.bfloat16)
    xs = kf.make_inputs(b, s, hq, hkv, d, dtype=dt, theta=theta, seed=0)
    q, k, v, gq, gk, cos, sin = [x.cuda() for x in xs]
    rec = {"case": name, "shape": {"B": b, "S": s, "Hq": hq, "Hkv": hkv, "D": d}, "dtype": "bf16"}

    # ---- the reference arm (two Triton launches) and the CUDA path, same inputs
    t_out, t_kn = torch.empty_like(q), torch.empty_like(k)
    inputs = (q, k, v, gq, gk, cos, sin)

    def triton_call():
        ref.launch_attention(inputs, t_out, causal=True, mode="query", bm=64, bn=128, gather=False,
                             rope=True, hf_norm=True, qn=None, kn=t_kn)

    c_out, c_kn = torch.empty_like(q), torch.empty_like(k)

    def cuda_call():
        kf.optimized_attention(q, k, v, gq, gk, cos, sin, causal=True, out=c_out, kn=c_kn)

    try:
        triton_call()
        torch.cuda.synchronize()
        rec["triton_ran"] = True
    except Exception as e:  # compile or launch failure: record it and go on with the CUDA path only
        rec["triton_ran"] = False
        rec["triton_error"] = f"{type(e).__name__}: {str(e).splitlines()[0][:300]}"
    cuda_call()
    torch.cuda.synchronize()
    kf.check_status()

    # ---- errors against the FP32 oracle (CPU, the first `nb_oracle` batches)
    if nb_oracle > 0:
        sl = slice(0, nb_oracle)
        want = orc.oracle_fp32(xs[0][sl], xs[1][sl], xs[2][sl], xs[3], xs[4], xs[5], xs[6], True)
        rec["cuda_vs_oracle"] = orc.metric(c_out[sl].cpu(), want)
        if rec["triton_ran"]:
            rec["triton_vs_oracle"] = orc.metric(t_out[sl].cpu(), want)
    if rec["triton_ran"]:
        diff = (c_out.float() - t_out.float()).abs()
        rec["cuda_vs_triton"] = {"max_abs": float(diff.max()), "mean_abs": float(diff.mean())}
        # prepared K: the CUDA kernel and the CPU emulation of `_rows` against the real kernel
        kd = (c_kn.float() - t_kn.float()).abs()
        rec["kn_cuda_vs_triton"] = {"max_abs": float(kd.max()), "mismatch_frac": float((kd > 0).float().mean())}
        if emulate:
            e_kn = orc.emulate_rows(xs[1], xs[4], xs[5], xs[6], hf_norm=True)
            ed = (e_kn.float() - t_kn.cpu().float()).abs()
            rec["kn_emulation_vs_triton"] = {"max_abs": float(ed.max()),
                                             "mismatch_frac": float((ed > 0).float().mean())}
            e_out = orc.emulate_optimized_attention(*xs, causal=True)
            od = (e_out.float() - t_out.cpu().float()).abs()
            rec["out_emulation_vs_triton"] = {"max_abs": float(od.max()), "mean_abs": float(od.mean())}
            if nb_oracle > 0:
                rec["emulation_vs_oracle"] = orc.metric(e_out[sl], want)

    # ---- device time, reference protocol (graphs of back-to-back calls, fresh captures per round)
    if do_time:
        fns = {"cuda": cuda_call}
        if rec["triton_ran"]:
            fns["triton"] = triton_call
        big = b * hq * s * s > (1 << 32)
        t = paired(fns, rounds=2 if quick else 5, samples=3 if quick else 7, replays=5 if big else 20)
        fl = orc.attention_flops(b, hq, s, d, True)
        for arm in fns:
            t[arm]["tflops"] = fl / (t[arm]["median_us"] * 1e-6) / 1e12
        rec["time"] = t
    return rec


# name, B, S, Hq, Hkv, D, theta, rope, hf_norm   (inputs: make_inputs(..., seed=0), bf16)
GOLDEN_CASES = [
    ("g128_hf", 1, 160, 4, 2, 128, 1e6, True, True),
    ("g128_legacy", 1, 160, 4, 2, 128, 1e6, True, False),
    ("g128_norope", 1, 160, 4, 2, 128, 1e6, False, True),
    ("g128_long", 1, 640, 2, 1, 128, 1e6, True, True),
    ("g256_hf", 1, 96, 2, 1, 256, 1e4, True, True),
]


def write_golden(ref, kf, path):
    import numpy as np
    out = {}
    for name, b, s, hq, hkv, d, theta, rope, hf in GOLDEN_CASES:
        xs = kf.make_inputs(b, s, hq, hkv, d, dtype=torch.bfloat16, theta=theta, seed=0)
        q, k, v, gq, gk, cos, sin = [x.cuda() for x in xs]
        o, kn = torch.empty_like(q), torch.empty_like(k)
        tabs = (cos, sin) if rope else (q, k)  # placeholders, as the reference passes them (:720)
        ref.launch_attention((q, k, v, gq, gk) + tabs, o, causal=True, mode="query", bm=64, bn=128,
                             gather=False, rope=rope, hf_norm=hf, qn=None, kn=kn)
        torch.cuda.synchronize()
        out[name + "_kn"] = kn.view(torch.int16).cpu().numpy()
        out[name + "_out"] = o.view(torch.int16).cpu().numpy()
        out[name + "_cfg"] = np.array([b, s, hq, hkv, d, int(theta), int(rope), int(hf)], dtype=np.int64)
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {sorted(out)}")


# Query fusion against the equally scheduled two-kernel control, the comparison the reference publishes for
# Hopper (results/RESULTS.md:61-65; arms at src/e1_rope_publication_v1.py:214-225): both modes of the CUDA
# path and of the reference's Triton arm, same protocol.   name, B, S, Hq, Hkv, D, theta
FUSION_SHAPES = [("B1_S128", 1, 128, 32, 8, 128, 1e6), ("B8_S128", 8, 128, 32, 8, 128, 1e6),
                 ("B32_S128", 32, 128, 32, 8, 128, 1e6), ("B1_S512", 1, 512, 32, 8, 128, 1e6),
                 ("B8_S512", 8, 512, 32, 8, 128, 1e6), ("B32_S512", 32, 512, 32, 8, 128, 1e6),
                 ("C2", 1, 2048, 32, 8, 128, 1e6), ("C4", 16, 4096, 32, 8, 128, 1e6),
                 ("C5", 8, 8192, 16, 8, 256, 1e4)]


def fusion_table(ref, kf, paired, path, with_full=False):
    rows = []
    for name, b, s, hq, hkv, d, theta in FUSION_SHAPES:
        xs = kf.make_inputs(b, s, hq, hkv, d, dtype=torch.bfloat16, theta=theta, seed=0)
        q, k, v, gq, gk, cos, sin = [x.cuda() for x in xs]
        out, kn, qn = torch.empty_like(q), torch.empty_like(k), torch.empty_like(q)
        inputs = (q, k, v, gq, gk, cos, sin)
        fns = {
            "cuda_query": lambda: kf.optimized_attention(q, k, v, gq, gk, cos, sin, causal=True, out=out, kn=kn),
            "cuda_unfused": lambda: kf.optimized_attention(q, k, v, gq, gk, cos, sin, causal=True, mode="unfused",
                                                           out=out, kn=kn),
            "triton_query": lambda: ref.launch_attention(inputs, out, causal=True, mode="query", bm=64, bn=128,
                                                         gather=False, qn=None, kn=kn),
            "triton_unfused": lambda: ref.launch_attention(inputs, out, causal=True, mode="unfused", bm=64, bn=128,
                                                           gather=False, qn=qn, kn=kn),
        }
        if with_full:
            # full fusion, one launch (the reference's tuned tiling for that mode: BM=32, BN=64, `:834`)
            fns["cuda_full"] = lambda: kf.launch_attention(inputs, out, causal=True, mode="full")
            fns["triton_full"] = lambda: ref.launch_attention(inputs, out, causal=True, mode="full", bm=32, bn=64,
                                                              gather=False)
        big = b * hq * s * s > (1 << 32)
        t = paired(fns, rounds=3, samples=5, replays=5 if big else 20)
        kf.check_status()
        row = {"shape": name, "B": b, "S": s, "Hq": hq, "Hkv": hkv, "D": d}
        for arm in fns:
            row[arm + "_us"] = t[arm]["median_us"]
        row["cuda_fusion_gain"] = row["cuda_unfused_us"] / row["cuda_query_us"]
        row["triton_fusion_gain"] = row["triton_unfused_us"] / row["triton_query_us"]
        rows.append(row)
        print(json.dumps(row), flush=True)
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    Path(path).write_text(json.dumps(rows, indent=1) + "\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--fusion-table", default="", help="write the fused-vs-unfused timing table to this JSON file")
    ap.add_argument("--with-full", action="store_true", help="add the one-launch full-fusion arms to the table")
    ap.add_argument("--golden", default="")
    ap.add_argument("--out", default=str(Path(tempfile.gettempdir()) / "triton_arm.json"))
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--cases", default="")
    args = ap.parse_args()
    import kernelfuser_b200 as kf
    from kernelfuser_b200.timing import paired
    from oracle import oracle as orc
    ref = load_reference()
    import triton
    if args.golden:
        write_golden(ref, kf, args.golden)
        return
    if args.fusion_table:
        fusion_table(ref, kf, paired, args.fusion_table, with_full=args.with_full)
        return
    want = set(filter(None, args.cases.split(",")))
    recs = []
    for case in CASES:
        if want and case[0] not in want:
            continue
        rec = run_case(ref, orc, kf, paired, case, quick=args.quick)
        recs.append(rec)
        print(json.dumps(rec), flush=True)
    Path(args.out).parent.mkdir(parents=True, exist_ok=True)
    Path(args.out).write_text(json.dumps({"triton": triton.__version__, "torch": torch.__version__,
                                          "gpu": torch.cuda.get_device_name(0), "cases": recs}, indent=1) + "\n")


if __name__ == "__main__":
    main()
