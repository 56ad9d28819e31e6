"""Child process of the lockstep-batch tolerance test: 32 sessions of the full model through the
tensor-core batched tick and through the exact-order tick (S2P_NO_TC=1), one process per path
(the switch is read when the tick's graph is captured).

Prints one JSON object: per layer, the K and V rows the first decode tick appended for every session
(bf16 KV cache, so they are the layer's own values: K after qk-norm and RoPE, V raw - both are
functions of that layer's input hidden state), and the codes of the first frames.
Usage: batch32_worker.py PATH OUT.npz     (PATH: tc | exact)"""
import ctypes as C
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    path, out = sys.argv[1], sys.argv[2]
    n_sess, prompt_len, frames = 32, 40, 6
    os.environ.update({"S2P_INT8": "1", "S2P_INT4": "1", "S2P_INT4_ALL": "1", "S2P_QCACHE": "0", "S2P_KV8": "0"})
    os.environ["S2P_NO_TC"] = "1" if path == "exact" else "0"
    import torch
    capi = importlib.import_module("s2pro-native_b200.capi")
    synth = importlib.import_module("s2pro-native_b200.synth")
    ckpt = os.environ.get("S2P_TEST_CKPT_DIR", "/dev/shm") + "/s2p_synth_l36"
    synth.write_checkpoint(ckpt, n_slow=36, seed=1, generator="auto")
    L = capi.load_library()
    opts = capi.ModelOpts(capi.GEMM_INT8, 256, n_sess)
    m = C.c_void_p()
    capi.check(L.s2p_model_load(ckpt.encode(), C.byref(opts), C.byref(m)), "load")
    sess = []
    for i in range(n_sess):
        cfg = L.s2p_sampling_defaults()
        cfg.temperature = 0.0  # greedy: the two paths differ only through their arithmetic
        s = C.c_void_p()
        capi.check(L.s2p_session_create(m, C.byref(cfg), C.byref(s)), "session")
        ids = synth.random_prompt(prompt_len, 300 + i)
        capi.check(L.s2p_session_prefill(s, ids.ctypes.data_as(C.c_void_p), None, len(ids), None, 0), "prefill")
        sess.append(s)
    arr = (C.c_void_p * n_sess)(*[s.value for s in sess])
    codes = (C.c_int32 * (10 * n_sess))()
    eos = (C.c_int * n_sess)()
    all_codes = []
    new_rows = None
    for f in range(frames):
        capi.check(L.s2p_model_batch_next_frame(m, arr, n_sess, codes, eos), "tick")
        all_codes.append(np.array(codes[:], dtype=np.int32).reshape(n_sess, 10).copy())
        if f == 1:  # the first tick with a backbone step: every session's input is still identical on both paths
            rows = []
            n_tok = prompt_len + 1
            for s in sess:
                nb = L.s2p_session_kv_bytes(m, n_tok)
                blob = torch.empty(nb, dtype=torch.uint8, device="cuda")
                capi.check(L.s2p_session_kv_save(s, n_tok, C.c_void_p(blob.data_ptr())), "kv_save")
                kv = blob.view(torch.bfloat16).view(36, 16, n_tok, 128)  # [layer][8 K planes, 8 V planes][token][128]
                rows.append(kv[:, :, n_tok - 1, :].float().cpu().numpy())
            new_rows = np.stack(rows)  # [session][layer][16][128]
    st = capi.Stats()
    capi.check(L.s2p_b200_model_stats(m, C.byref(st)), "stats")
    np.savez(out, rows=new_rows, codes=np.stack(all_codes), kernels=st.last_tick_kernels, graph=st.last_tick_graph)
    for s in sess:
        L.s2p_session_destroy(s)
    L.s2p_model_free(m)
    print("done", path)


if __name__ == "__main__":
    main()
