"""Child process of the sidecar tests: load the 2-layer all-INT4 checkpoint through one library with the
prequantised-weight sidecar enabled in a given directory, decode a few greedy frames, print them.
One process per load: the reference reads its S2P_* switches once.
Usage: qcache_worker.py mine|ref SIDECAR_DIR"""
import ctypes as C
import importlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    which, qdir = sys.argv[1], sys.argv[2]
    os.environ.update({"S2P_INT8": "1", "S2P_INT4": "1", "S2P_INT4_ALL": "1", "S2P_QCACHE": "1", "S2P_QCACHE_DIR": qdir})
    capi = importlib.import_module("s2pro-native_b200.capi")
    synth = importlib.import_module("s2pro-native_b200.synth")
    ckpt = os.environ.get("S2P_TEST_CKPT_DIR", "/dev/shm") + "/s2p_synth_l2"
    synth.write_checkpoint(ckpt, n_slow=2, seed=0, generator="auto")
    if which == "mine":
        L = capi.load_library()
    else:
        L = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libs2pref_l2.so"))
        capi.bind(L, capi.PROTOTYPES, strict=False)
    opts = capi.ModelOpts(capi.GEMM_INT8, 512, 1)
    m = C.c_void_p()
    capi.check(L.s2p_model_load(ckpt.encode(), C.byref(opts), C.byref(m)), "load")
    cfg = L.s2p_sampling_defaults()
    cfg.temperature = 0.0
    s = C.c_void_p()
    capi.check(L.s2p_session_create(m, C.byref(cfg), C.byref(s)), "session")
    ids = synth.random_prompt(32, 11)
    capi.check(L.s2p_session_prefill(s, ids.ctypes.data_as(C.c_void_p), None, len(ids), None, 0), "prefill")
    codes = (C.c_int32 * 10)()
    eos = C.c_int(0)
    frames = []
    for _ in range(6):
        capi.check(L.s2p_session_next_frame(s, codes, C.byref(eos)), "frame")
        frames.append(list(codes))
    L.s2p_session_destroy(s)
    L.s2p_model_free(m)
    print("RESULT " + json.dumps({"frames": frames}))


if __name__ == "__main__":
    main()
