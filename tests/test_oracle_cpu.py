"""CPU tests: the oracle (oracle/s2p_oracle.c) pinned against golden vectors that
were produced by the reference's own Python and C code (tests/golden/make_golden.py),
plus the size-independent properties the reference states for its quantisers and GEMVs."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

from oracle import oracle_api as oa

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden")


def quant_g(orc, w_bits, N, K, G=32, mse=1):
    q = np.empty((N, K), np.int8); sc = np.empty((N, K // G), np.uint16)
    orc.s2po_quant_g(oa.ptr(q), oa.ptr(sc), oa.ptr(w_bits), N, K, G, 7, mse)
    return q, sc


def test_bf16_f16_conversions_match_numpy(oracle):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(5000).astype(np.float32) * s for s in (1e-6, 1e-3, 1.0, 300.0, 7e4)])
    x = np.concatenate([x, np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 5.96e-8, 2.98e-8, 6.1e-5], np.float32)])
    got_h = np.array([oracle.s2po_f2h(float(v)) for v in x], np.uint16)
    with np.errstate(over="ignore"):
        want_h = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got_h, want_h)
    back = np.array([oracle.s2po_h2f(int(h)) for h in want_h], np.float32)
    assert np.array_equal(back.view(np.uint32), want_h.view(np.float16).astype(np.float32).view(np.uint32))
    got_b = np.array([oracle.s2po_f2bf(float(v)) for v in x], np.uint16)
    assert np.array_equal(got_b, oa.f32_to_bf16(x))


def test_quantisers_against_reference_python(oracle):
    """Dequantised INT4-g32 (MSE search) and INT8 weights vs the reference's torch port
    (tools/qat_fastar.py:47-70,104-117).  The torch port divides by the scale where the CUDA
    kernel multiplies by 1.0f/scale and sums the error in another order (it says so itself),
    so a handful of groups may pick a neighbouring clip candidate: >= 99.5 % of groups must
    agree exactly, and no element may move by more than one quantisation step."""
    g = np.load(os.path.join(GOLD, "quantisers.npz"))
    for name in ("a", "b"):
        w = g[f"w_{name}"]; N, K = w.shape
        q, sc = quant_g(oracle, w, N, K)
        scf = np.array([oracle.s2po_h2f(int(h)) for h in sc.ravel()], np.float32).reshape(sc.shape)
        deq = q.astype(np.float32).reshape(N, K // 32, 32) * scf[:, :, None]
        want = g[f"int4_deq_{name}"].reshape(N, K // 32, 32)
        zero = (oa.bf16_to_f32(w).reshape(N, K // 32, 32) == 0).all(-1)
        same = (deq == want).all(-1) | zero
        assert same.mean() >= 0.995, same.mean()
        assert np.max(np.abs(deq - want) - scf[:, :, None]) <= 1e-9
        # INT8 per channel: scale = amax/127, q = rint(w * (1/scale)) vs torch's round(w / scale)
        q8 = np.empty((N, K), np.int8); s8 = np.empty(N, np.float32)
        oracle.s2po_quant_int8(oa.ptr(q8), oa.ptr(s8), oa.ptr(w), N, K)
        deq8 = q8.astype(np.float32) * s8[:, None]
        want8 = g[f"int8_deq_{name}"]
        assert (deq8 == want8).mean() >= 0.999
        assert np.max(np.abs(deq8 - want8) - s8[:, None]) <= 1e-9
        assert s8[3] == 1.0 and not q8[3].any()  # all-zero row: unit scale, zero codes


def test_quantiser_properties(oracle):
    rng = np.random.default_rng(1)
    N, K = 16, 1024
    w = oa.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    q, sc = quant_g(oracle, w, N, K)
    assert q.min() >= -7 and q.max() <= 7
    pk = np.empty((N, K // 2), np.uint8); oracle.s2po_pack(oa.ptr(pk), oa.ptr(q), N * K // 2)
    back = np.empty((N, K), np.int8); oracle.s2po_unpack(oa.ptr(back), oa.ptr(pk), N * K // 2)
    assert np.array_equal(back, q)                       # pack -> unpack round trip
    assert np.array_equal(pk & 0xF, q[:, 0::2] & 0xF)    # low nibble = even column
    d1 = np.empty((N, K), np.uint16); d2 = np.empty((N, K), np.uint16)
    oracle.s2po_dequant_g(oa.ptr(d1), oa.ptr(q), oa.ptr(sc), N, K, 32)
    oracle.s2po_dequant_p(oa.ptr(d2), oa.ptr(pk), oa.ptr(sc), N, K, 32)
    assert np.array_equal(d1, d2)                        # packed == container dequant
    # MSE search never does worse than plain absmax rounding
    q0, sc0 = quant_g(oracle, w, N, K, mse=0)
    wf = oa.bf16_to_f32(w)
    err = lambda qq, ss: ((wf - qq.astype(np.float32) * np.repeat(ss.view(np.float16).astype(np.float32), 32, axis=1)) ** 2).sum()
    assert err(q, sc) <= err(q0, sc0) * (1 + 1e-6)
    # quantising the dequantised tensor reproduces the INT8 codes (idempotence on the grid)
    q8 = np.empty((N, K), np.int8); s8 = np.empty(N, np.float32)
    oracle.s2po_quant_int8(oa.ptr(q8), oa.ptr(s8), oa.ptr(w), N, K)
    assert np.abs(q8).max(axis=1).min() == 127           # the absmax element maps to +-127


def test_gemv_packed_equals_container_and_linearity(oracle):
    """The reference's invariants (include/s2pro/gemm.h:128-132): packed and int8-container
    GEMVs are bit-identical; batched rows equal single-row calls."""
    rng = np.random.default_rng(2)
    N, K, M = 40, 1536, 5
    w = oa.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    x = oa.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    q, sc = quant_g(oracle, w, N, K)
    pk = np.empty((N, K // 2), np.uint8); oracle.s2po_pack(oa.ptr(pk), oa.ptr(q), N * K // 2)
    y1 = np.empty((M, N), np.uint16); y2 = np.empty((M, N), np.uint16)
    oracle.s2po_gemv_g(oa.ptr(y1), oa.ptr(x), oa.ptr(q), oa.ptr(sc), M, N, K, 32)
    oracle.s2po_gemv_p(oa.ptr(y2), oa.ptr(x), oa.ptr(pk), oa.ptr(sc), M, N, K, 32)
    assert np.array_equal(y1, y2)
    for m in range(M):
        y = np.empty((1, N), np.uint16)
        oracle.s2po_gemv_p(oa.ptr(y), oa.ptr(np.ascontiguousarray(x[m:m + 1])), oa.ptr(pk), oa.ptr(sc), 1, N, K, 32)
        assert np.array_equal(y[0], y2[m])
    # against a float64 dot product of the dequantised weights: bf16 output tolerance
    deq = q.astype(np.float64) * np.repeat(sc.view(np.float16).astype(np.float64), 32, axis=1)
    ref = oa.bf16_to_f32(x).astype(np.float64) @ deq.T
    got = oa.bf16_to_f32(y2).astype(np.float64)
    assert np.max(np.abs(got - ref)) <= 2 ** -7 * np.max(np.abs(ref)) + 1e-3
    # empty K tail is not a thing (K % 512 == 0 is a precondition); M = 1, N = 1 edge
    y = np.empty((1, 1), np.uint16)
    oracle.s2po_gemv_p(oa.ptr(y), oa.ptr(np.ascontiguousarray(x[:1])), oa.ptr(pk[:1]), oa.ptr(sc[:1]), 1, 1, K, 32)
    assert y[0, 0] == y2[0, 0]


def test_sampler_against_reference_host_sampler(oracle):
    """Token sequences of the reference's src/slowar/sampling.c (greedy, seeded, seeded+hot,
    with a forced EOS frame) must be reproduced exactly."""
    g = np.load(os.path.join(GOLD, "sampler.npz"))
    logits = g["smp_logits"]
    for tag, temp, seed in (("greedy", 0.0, 0), ("seeded", 0.8, 42), ("seeded_hot", 1.3, 7)):
        sp = C.create_string_buffer(oracle.s2po_sampler_size())
        oracle.s2po_sampler_init(sp, temp, 0.8, 1.1, 16, seed, 0)
        for t in range(logits.shape[0]):
            sem, eos = C.c_int32(0), C.c_int32(0)
            tok = oracle.s2po_sample(sp, oa.ptr(logits[t]), int(logits[t, 4096]), 4096, 151678, 151645, C.byref(sem), C.byref(eos))
            assert (tok, sem.value, eos.value) == (int(g[f"smp_{tag}_tok"][t]), int(g[f"smp_{tag}_sem"][t]), int(g[f"smp_{tag}_eos"][t])), (tag, t)
        assert g[f"smp_{tag}_eos"][7] == 1  # the EOS frame is in the fixture


def test_sampler_against_rebuilt_reference_if_present(oracle):
    """Same check live against oracle/_ref/libs2pref_sampling.so when it exists here."""
    p = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libs2pref_sampling.so")
    if not os.path.exists(p):
        pytest.skip("reference sampler not built on this machine")
    lib = C.CDLL(p)
    lib.s2ps_sample.restype = C.c_int64

    class Cfg(C.Structure):
        _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("repetition_penalty", C.c_float),
                    ("repetition_window", C.c_int), ("seed", C.c_uint64)]
    rng = np.random.default_rng(9)
    for temp, seed, window in ((0.0, 0, 16), (0.7, 123, 4), (1.0, 99, 64)):
        ref_sp = C.create_string_buffer(1024)
        lib.s2ps_sampler_init(ref_sp, C.byref(Cfg(temp, 0.9, 1.3, window, seed)), C.c_uint64(0))
        sp = C.create_string_buffer(oracle.s2po_sampler_size())
        oracle.s2po_sampler_init(sp, temp, 0.9, 1.3, window, seed, 0)
        for t in range(80):
            lg = oa.f32_to_bf16((rng.standard_normal(4097) * 3).astype(np.float32))
            s1, e1, s2, e2 = C.c_int32(0), C.c_int(0), C.c_int32(0), C.c_int32(0)
            t1 = lib.s2ps_sample(ref_sp, oa.ptr(lg), C.c_uint16(int(lg[4096])), C.byref(s1), C.byref(e1))
            t2 = oracle.s2po_sample(sp, oa.ptr(lg), int(lg[4096]), 4096, 151678, 151645, C.byref(s2), C.byref(e2))
            assert (t1, s1.value, e1.value) == (t2, s2.value, e2.value), (temp, seed, t)


def test_fast_ar_against_reference_torch_model(oracle):
    """The oracle's fast-AR frame (bf16 weights, reduced width) vs the greedy codes and
    teacher-forced logits of the reference's torch FastAR (tools/qat_fastar.py:180-232).
    Tolerance: the torch model runs f32 activations, the oracle rounds activations to bf16
    like the CUDA path: logits within 0.15 max-abs and cosine >= 0.999; codes equal wherever
    the torch top-2 margin exceeds that bound."""
    sys.path.insert(0, GOLD)
    from fastar_inputs import DIMS, make_inputs
    g = np.load(os.path.join(GOLD, "fastar.npz"))
    tensors, hidden, sem = make_inputs()
    m = oracle.s2po_model_new(DIMS["dim"], DIMS["q_heads"], DIMS["kv_heads"], DIMS["ffn"], 4096, 0, DIMS["layers"], 4096, 10,
                              0, 4095, 0, 0, 0, 0, 0, 64)
    b = lambda t: oa.f32_to_bf16(t.numpy())
    for i in range(DIMS["layers"]):
        p = f"audio_decoder.layers.{i}"
        for which, key in ((0, "attention.wqkv"), (1, "attention.wo"), (2, "feed_forward.w1"), (3, "feed_forward.w3"),
                           (4, "feed_forward.w2"), (5, "attention_norm"), (6, "ffn_norm")):
            a = b(tensors[f"{p}.{key}.weight"])
            oracle.s2po_model_set_layer(m, 1, i, which, oa.ptr(a))
    for which, key in ((2, "norm"), (3, "output"), (5, "embeddings")):
        a = b(tensors[f"audio_decoder.{key}.weight"])
        oracle.s2po_model_set_global(m, which, oa.ptr(a))
    hid = b(hidden)
    agree = total = 0
    for r in range(DIMS["rows"]):
        codes = np.zeros(9, np.int32); logits = np.zeros((9, 4096), np.float32)
        oracle.s2po_fast_frame(m, oa.ptr(np.ascontiguousarray(hid[r])), int(sem[r]), oa.ptr(codes), oa.ptr(logits))
        want = g["fa_codes"][r]
        if r < 2:
            ref = g["fa_logits"][r].astype(np.float32)
            # compare step by step only while the trajectories coincide (teacher forcing follows torch's codes)
            for step in range(9):
                cos = float(np.dot(logits[step], ref[step]) / (np.linalg.norm(logits[step]) * np.linalg.norm(ref[step])))
                assert cos >= 0.999, (r, step, cos)
                assert np.max(np.abs(logits[step] - ref[step])) <= 0.15
                if codes[step] != want[step]:
                    break
        for step in range(9):
            total += 1
            if codes[step] == want[step]:
                agree += 1
            else:
                break
    oracle.s2po_model_free(m)
    assert agree >= 0.9 * total, (agree, total)
