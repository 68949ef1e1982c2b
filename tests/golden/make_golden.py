"""Regenerates tests/golden/sampler_golden.npz from the REFERENCE sampler itself (qp::Sampler of
src/sampler.cpp compiled into oracle/_ref/ by oracle/Makefile).  Run where the reference sources are present:

    python tests/golden/make_golden.py

The reference has no sampler test or golden vector of its own, so these fixtures (outputs of the reference
code on seeded inputs, inputs included for the small cases) are what pins the CPU restatement and, through
it, the CUDA path.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import Ref, make_params  # noqa: E402
from qpack_b200 import synth  # noqa: E402

MAX_OUT = 64


def small_cases():
    """Ragged / tiny / tie-heavy rows with mixed parameters: inputs are stored with the outputs."""
    rng = np.random.default_rng(20240601)
    cases = []
    for V in (1, 2, 3, 5, 31, 32, 33, 255, 1023, 1024, 1025, 3075, 3076, 4099):
        for variant in range(3):
            B = 3
            x = (rng.standard_normal((B, V)) * 2.5).astype(np.float32)
            if variant == 1:
                x = np.round(x)  # heavy ties, signed zeros
                x[x == 0] = np.where(rng.random(np.count_nonzero(x == 0)) < 0.5, 0.0, -0.0)
            H = [0, 7, 80][variant]
            hist = rng.integers(-3, V + 3, size=(B, max(H, 1))).astype(np.int32)
            if H:
                for r in range(B):
                    top = np.argsort(-x[r], kind="stable")[: min(V, 6)]
                    hist[r, : min(H, 3)] = rng.choice(top, min(H, 3))
            hl = np.array([H, H // 2, max(H - 1, 0)], np.int32)
            p = make_params(
                B,
                temperature=rng.choice([0.0, 0.6, 1.0, 1.4], B).astype(np.float32),
                top_k=rng.choice([0, 1, 4, 40, 300], B).astype(np.int32),
                top_p=rng.choice([0.5, 0.9, 0.97, 1.0], B).astype(np.float32),
                min_p=rng.choice([0.0, 0.05, 0.2], B).astype(np.float32),
                repeat_penalty=rng.choice([1.0, 1.1, 1.3, 0.9], B).astype(np.float32),
                repeat_last_n=rng.choice([0, 4, 64, -1], B).astype(np.int32),
                seed=rng.integers(1, 1 << 60, B).astype(np.uint64),
            )
            cases.append((x, hist, hl, p))
    return cases


def main():
    out = {}
    # 1. small cases, inputs stored
    for i, (x, hist, hl, p) in enumerate(small_cases()):
        V = x.shape[1]
        r = Ref.sample_rows(p, x, hist, hl, max_out=min(V, MAX_OUT))
        out[f"small{i}_logits"] = x
        out[f"small{i}_hist"] = hist
        out[f"small{i}_hist_len"] = hl
        out[f"small{i}_params"] = p
        out[f"small{i}_ids"] = r["ids"]
        out[f"small{i}_count"] = r["count"]
        out[f"small{i}_dist_ids"] = r["dist_ids"]
        out[f"small{i}_dist_p"] = r["dist_p"]
    out["n_small"] = np.int32(i + 1)
    # 2. the reference micro-benchmark's row (bench/sampler_bench.cpp:6-9), seed 42: distribution and 8 draws
    x, h = synth.sampler_bench_row()
    k = 0
    for T in (0.0, 0.7):
        for rp in (1.0, 1.1):
            s = Ref(make_params(1, temperature=T, repeat_penalty=rp, seed=42))
            ids, pr = s.dist(x[0], h[0])
            out[f"sb{k}_params"] = make_params(1, temperature=T, repeat_penalty=rp, seed=42)
            out[f"sb{k}_dist_ids"] = ids
            out[f"sb{k}_dist_p"] = pr
            out[f"sb{k}_draws"] = np.array([s.sample(x[0], h[0]) for _ in range(8)], np.int32)
            k += 1
    # 3. the single-row loop (config 1): 48 successive draws of one sampler, history growing
    params, hist0 = synth.single_row_loop()
    s = Ref(params)
    hist = list(hist0)
    ids, counts, sums = [], [], []
    for step in range(48):
        lg = synth.single_row_step(step)
        d_ids, d_p = s.dist(lg[0], np.array(hist, np.int32))
        t = s.draw(d_ids, d_p)
        ids.append(t)
        counts.append(len(d_ids))
        sums.append(float(lg.astype(np.float64).sum()))
        hist.append(t)
    out["loop_ids"] = np.array(ids, np.int32)
    out["loop_counts"] = np.array(counts, np.int32)
    out["loop_logit_sums"] = np.array(sums, np.float64)  # guards against drift of the input generator
    # 4. first rows of the batched configurations at full vocabulary (inputs regenerated from their seeds)
    for name, wl in (("serving", synth.serving_batch(rows=8)), ("mixed", synth.mixed_batch(rows=16)),
                     ("sharded", synth.sharded_batch(rows=8)), ("llama3", synth.llama3_batch(rows=4))):
        r = Ref.sample_rows(wl.params, wl.logits, wl.history, wl.hist_len, max_out=MAX_OUT, threads=4)
        out[f"{name}_ids"] = r["ids"]
        out[f"{name}_count"] = r["count"]
        out[f"{name}_dist_ids"] = r["dist_ids"]
        out[f"{name}_dist_p"] = r["dist_p"]
        out[f"{name}_logit_sums"] = wl.logits.astype(np.float64).sum(axis=1)
    path = os.path.join(ROOT, "tests", "golden", "sampler_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
