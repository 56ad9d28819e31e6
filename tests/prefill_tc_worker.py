"""Child process of tests/test_prefill_tc_gpu.py: the same prompt prefilled twice into fresh sessions of one
model, once through dequantise + cuBLAS (the default, bit-identical to the reference) and once with
S2P_PREFILL_TC=1 (tensor cores straight from the quantised weights), KV cache compared plane by plane.
Usage: prefill_tc_worker.py MODE N_SLOW TOKENS    (MODE: int8 | int4)"""
import ctypes as C
import importlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    mode, n_slow, n_tok = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    os.environ.update({"S2P_INT8": "1", "S2P_QCACHE": "0", "S2P_KV8": "0", "S2P_SCRATCH_ROWS": "1024"})
    if mode == "int4":
        os.environ.update({"S2P_INT4": "1", "S2P_INT4_ALL": "1"})
    import torch
    capi = importlib.import_module("s2pro-native_b200.capi")
    synth = importlib.import_module("s2pro-native_b200.synth")
    ckpt = os.environ.get("S2P_TEST_CKPT_DIR", "/dev/shm") + f"/s2p_synth_l{n_slow}"
    synth.write_checkpoint(ckpt, n_slow=n_slow, seed=0 if n_slow == 2 else 1, generator="auto")
    L = capi.load_library()
    opts = capi.ModelOpts(capi.GEMM_INT8, 2048, 2)
    m = C.c_void_p()
    assert L.s2p_model_load(ckpt.encode(), C.byref(opts), C.byref(m)) == 0
    ids = synth.random_prompt(n_tok, 11)
    out = {}
    for tc in (0, 1):
        os.environ["S2P_PREFILL_TC"] = str(tc)
        cfg = L.s2p_sampling_defaults()
        cfg.temperature = 0.0
        s = C.c_void_p()
        assert L.s2p_session_create(m, C.byref(cfg), C.byref(s)) == 0
        # two slices, so that a slice starting inside the cache is covered as well
        cut = n_tok * 2 // 3
        for a, b in ((0, cut), (cut, n_tok)):
            rc = L.s2p_session_prefill(s, ids[a:b].ctypes.data_as(C.c_void_p), None, b - a, None, 0)
            assert rc == 0, rc
        nb = L.s2p_session_kv_bytes(m, n_tok)
        kv = torch.empty(nb, dtype=torch.uint8, device="cuda")
        assert L.s2p_session_kv_save(s, n_tok, C.c_void_p(kv.data_ptr())) == 0
        frames = []
        codes = (C.c_int32 * 10)()
        eos = C.c_int(0)
        for _ in range(4):
            assert L.s2p_session_next_frame(s, codes, C.byref(eos)) == 0
            frames.append(list(codes))
            if eos.value:
                break
        out[tc] = (kv.view(torch.bfloat16).float(), frames)
        L.s2p_session_destroy(s)
    a, b = out[0][0], out[1][0]
    cos = float(torch.nn.functional.cosine_similarity(a, b, dim=0))
    rel = float((a - b).abs().max() / a.abs().max())
    same = float((a == b).float().mean())
    print("RESULT " + json.dumps({"kv_cosine": cos, "kv_max_rel": rel, "kv_equal_share": same, "finite": bool(torch.isfinite(b).all()),
                                  "frames_default": out[0][1], "frames_tc": out[1][1]}))
    L.s2p_model_free(m)


if __name__ == "__main__":
    main()
