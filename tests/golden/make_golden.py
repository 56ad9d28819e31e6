#!/usr/bin/env python
"""Generates tests/golden/*.npz by IMPORTING the reference's own Python code
(tools/qat_fastar.py: its bit-faithful port of the g32 quantiser, its INT8
reference linear and its torch fast-AR model) and the reference's host sampler
(src/slowar/sampling.c, compiled by oracle/Makefile into oracle/_ref).  Run where
the reference checkout is available (S2P_REFERENCE points at it); the outputs are
committed so that the tests need neither.

    python tests/golden/make_golden.py
"""
import ctypes as C
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("S2P_REFERENCE") or os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference"))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)
from oracle import oracle_api  # noqa: E402


def load_ref_module():
    spec = importlib.util.spec_from_file_location("qat_fastar", os.path.join(REF, "tools", "qat_fastar.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bf16_round(t):
    return t.to(torch.bfloat16).float()


def golden_quantisers(q):
    """Dequantised g32 INT4 weights and INT8 reference weights of seeded matrices."""
    out = {}
    g = torch.Generator().manual_seed(1234)
    for name, (N, K) in {"a": (64, 512), "b": (24, 1024)}.items():
        w = bf16_round(torch.randn(N, K, generator=g) * 0.02)
        w[3] = 0.0  # an all-zero row: the quantiser writes zeros and a unit scale
        w[5, :32] = 0.0
        out[f"w_{name}"] = oracle_api.f32_to_bf16(w.numpy())
        out[f"int4_deq_{name}"] = q.fake_quant_g32(w).numpy().astype(np.float32)
        out[f"int8_deq_{name}"] = q.Int8Linear(w).weight.numpy().astype(np.float32)
    return out


def golden_fastar(q):
    """Greedy 9-step fast-AR decode of the reference's torch model at reduced width
    (its module constants are patched: the arithmetic is unchanged).  Only the outputs
    are stored; the seeded inputs are rebuilt by tests/golden/fastar_inputs.py."""
    from fastar_inputs import DIMS, make_inputs
    q.DIM, q.N_HEAD, q.N_KV, q.HEAD_DIM, q.FFN, q.VOCAB = DIMS["dim"], DIMS["q_heads"], DIMS["kv_heads"], 128, DIMS["ffn"], 4096
    tensors, hidden, sem = make_inputs()
    model = q.FastAR(tensors, q.RefLinear, 1e-6, 1e6)
    with torch.no_grad():
        codes = model.greedy(hidden, sem)
        logits = model.forward_seq(hidden, sem, codes[:, :8])  # teacher-forced along the greedy trajectory
    return {"fa_codes": codes.numpy().astype(np.int32), "fa_logits": logits[:2].numpy().astype(np.float16)}


def golden_sampler():
    """Token sequences of the reference's host sampler (sampling.c) on seeded logits."""
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libs2pref_sampling.so"))

    class Cfg(C.Structure):
        _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("repetition_penalty", C.c_float),
                    ("repetition_window", C.c_int), ("seed", C.c_uint64)]
    lib.s2ps_sample.restype = C.c_int64
    out = {}
    rng = np.random.default_rng(5)
    steps = 40
    logits = oracle_api.f32_to_bf16((rng.standard_normal((steps, 4097)) * 2.0).astype(np.float32))
    logits[7, 4096] = oracle_api.f32_to_bf16(np.array([30.0], np.float32))[0]  # forces an EOS frame
    out["smp_logits"] = logits
    for tag, temp, seed in (("greedy", 0.0, 0), ("seeded", 0.8, 42), ("seeded_hot", 1.3, 7)):
        sp = C.create_string_buffer(1024)
        cfg = Cfg(temp, 0.8, 1.1, 16, seed)
        lib.s2ps_sampler_init(sp, C.byref(cfg), C.c_uint64(0))
        toks, sems, eoss = [], [], []
        for t in range(steps):
            sem, eos = C.c_int32(0), C.c_int(0)
            tok = lib.s2ps_sample(sp, logits[t].ctypes.data_as(C.c_void_p), C.c_uint16(int(logits[t, 4096])),
                                  C.byref(sem), C.byref(eos))
            toks.append(tok); sems.append(sem.value); eoss.append(eos.value)
        out[f"smp_{tag}_tok"] = np.array(toks, np.int64)
        out[f"smp_{tag}_sem"] = np.array(sems, np.int32)
        out[f"smp_{tag}_eos"] = np.array(eoss, np.int32)
    return out


def main():
    q = load_ref_module()
    np.savez_compressed(os.path.join(HERE, "quantisers.npz"), **golden_quantisers(q))
    np.savez_compressed(os.path.join(HERE, "sampler.npz"), **golden_sampler())
    np.savez_compressed(os.path.join(HERE, "fastar.npz"), **golden_fastar(q))
    for f in ("quantisers.npz", "sampler.npz", "fastar.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")


if __name__ == "__main__":
    main()
