"""Lockstep batch of 32 sessions, model level, tolerance class.  Beyond 16 rows the batched linears run
on the tensor cores with a summation order of their own, so their results are not bit-equal to the
exact-order GEMV (which is what the reference would compute for every row).  This test runs the same 32
sessions of the full 36+4-layer all-INT4 model through both ticks and compares, after the first decode
tick (identical inputs on both sides: teacher forcing by construction):
  - per layer, the K and V rows the tick appended to the bf16 cache (functions of that layer's input
    hidden state): max-abs difference and cosine per session;
  - the sampled semantic token and the nine greedy codebook codes of that frame."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))

# What the tensor-core tick achieves against the exact-order tick on a random-init checkpoint, with margin.
# Measured (36 layers, 22 comparable sessions): cosine 0.999999 at layer 0, 0.99988 at layer 5, 0.99947 at
# layer 35; max-abs / layer max 0.003 -> 0.031.  The linears themselves differ from the exact GEMV by at most
# one bf16 rounding step per output (tests/test_skinny_gpu.py); over 36 residual layers of an untrained
# network those flips accumulate.  So the tighter class asked of hidden states (2e-2 max-abs, cosine
# 0.9999) holds for the first layers only, and the batch path is reported in this looser class; batches of
# up to 16 rows stay on the exact-order kernel and are bit-equal to the reference.
MAX_REL, MIN_COS, MIN_SEM_AGREE = 5e-2, 0.999, 0.8
TIGHT_ABS, TIGHT_COS = 2e-2, 0.9999


def _run(path, out):
    r = subprocess.run([sys.executable, os.path.join(HERE, "batch32_worker.py"), path, out], capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    return np.load(out)


def test_batch32_tensor_core_tick_against_exact_order_tick(tmp_path):
    tc = _run("tc", str(tmp_path / "tc.npz"))
    ex = _run("exact", str(tmp_path / "exact.npz"))
    assert int(tc["graph"]) == 1 and int(ex["graph"]) == 1
    assert int(tc["kernels"]) < int(ex["kernels"]), "the two runs must have taken different linears"
    # Frame 0 is sampled from the prefill state, but its nine codebook codes already come from the batched
    # fast-AR linears, and a flipped greedy arg-max there changes what frame 1 is fed.  Teacher forcing
    # therefore holds for the sessions whose frame 0 is identical on both paths: those are compared.
    same0 = (tc["codes"][0] == ex["codes"][0]).all(axis=1)
    assert np.array_equal(tc["codes"][0][:, 0], ex["codes"][0][:, 0]), "the semantic token of frame 0 involves no batched linear"
    n_tf = int(same0.sum())
    print(f"{n_tf} of 32 sessions have an identical frame 0 (the others flipped a greedy fast-AR arg-max on near-tied random-weight logits)")
    assert n_tf >= 8, "too few sessions left to compare"
    a, b = tc["rows"].astype(np.float64)[same0], ex["rows"].astype(np.float64)[same0]  # [session][layer][16 planes][128]
    assert a.shape == b.shape == (n_tf, 36, 16, 128)
    worst_abs, worst_cos = 0.0, 1.0
    per_layer = []
    for layer in range(36):
        x, y = a[:, layer].reshape(n_tf, -1), b[:, layer].reshape(n_tf, -1)
        d = np.abs(x - y).max()
        scale = np.abs(y).max()
        cos = ((x * y).sum(1) / (np.linalg.norm(x, axis=1) * np.linalg.norm(y, axis=1))).min()
        per_layer.append((layer, d, d / scale, cos))
        worst_abs, worst_cos = max(worst_abs, d / max(scale, 1.0)), min(worst_cos, cos)
    print("layer: max-abs, max-abs / layer max, min cosine over the compared sessions")
    for layer, d, rel, cos in per_layer:
        print(f"  {layer:2d}: {d:.4f} {rel:.5f} {cos:.6f}")
    same_sem = float((tc["codes"][1][same0, 0] == ex["codes"][1][same0, 0]).mean())
    same_all = float((tc["codes"][1][same0] == ex["codes"][1][same0]).mean())
    later = [round(float((tc["codes"][f][same0] == ex["codes"][f][same0]).mean()), 3) for f in range(2, tc["codes"].shape[0])]
    print(f"frame 1 (identical inputs): semantic token equal for {same_sem:.3f} of the compared sessions, all ten codes {same_all:.3f}; "
          f"free-running frames after it: {later}")
    tight = [layer for layer, d, rel, cos in per_layer if d <= TIGHT_ABS and cos >= TIGHT_COS]
    print(f"layers within 2e-2 max-abs and cosine 0.9999: {tight}")
    assert 0 in tight, "the first layer sees one batched linear only: it must be within the tight class"
    assert worst_cos >= MIN_COS, f"cosine {worst_cos}"
    assert worst_abs <= MAX_REL, f"max-abs relative to max(1, layer max) {worst_abs}"
    assert same_sem >= MIN_SEM_AGREE, f"teacher-forced semantic arg-max agreement {same_sem}"
