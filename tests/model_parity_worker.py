"""Child process of the model-level parity tests (one quantisation mode per
process: the reference caches its S2P_* switches on first use).

Loads the same synthetic checkpoint into the reference library rebuilt for
sm_100a and into this library (persistent tick kernel, per-stage fused batch-1
path and general path), runs
identical API calls on both and prints one JSON object with what matched.
Usage: model_parity_worker.py MODE N_SLOW FRAMES   (MODE: int8 | int4)
"""
import ctypes as C
import importlib
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    mode, n_slow, frames = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    prompt_len = int(sys.argv[4]) if len(sys.argv) > 4 else 64
    os.environ["S2P_INT8"] = "1"
    os.environ["S2P_QCACHE"] = "0"
    if mode == "int4":
        os.environ["S2P_INT4"] = "1"
        os.environ["S2P_INT4_ALL"] = "1"
    import torch
    capi = importlib.import_module("s2pro-native_b200.capi")
    synth = importlib.import_module("s2pro-native_b200.synth")
    ckpt = os.environ.get("S2P_TEST_CKPT_DIR", "/dev/shm") + f"/s2p_synth_l{n_slow}"
    synth.write_checkpoint(ckpt, n_slow=n_slow, seed=0 if n_slow == 2 else 1, generator="auto")
    mine = capi.load_library()
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libs2pref_l2.so" if n_slow == 2 else "libs2pref.so"))
    capi.bind(ref, capi.PROTOTYPES, strict=False)

    def load(L, fused, persistent=True):
        os.environ["S2P_NO_FUSED"] = "0" if fused else "1"
        os.environ["S2P_NO_MEGA"] = "0" if persistent else "1"
        opts = capi.ModelOpts(capi.GEMM_INT8, 4096, 4)
        m = C.c_void_p()
        rc = L.s2p_model_load(ckpt.encode(), C.byref(opts), C.byref(m))
        assert rc == 0, rc
        return m

    def session(L, m, temp, seed):
        cfg = L.s2p_sampling_defaults()
        cfg.temperature = temp
        cfg.seed = seed
        s = C.c_void_p()
        rc = L.s2p_session_create(m, C.byref(cfg), C.byref(s))
        assert rc == 0, rc
        return s

    def prefill(L, s, ids):
        rc = L.s2p_session_prefill(s, ids.ctypes.data_as(C.c_void_p), None, len(ids), None, 0)
        assert rc == 0, rc

    def run(L, s, n):
        out = []
        codes = (C.c_int32 * 10)()
        eos = C.c_int(0)
        t = time.time()
        for _ in range(n):
            rc = L.s2p_session_next_frame(s, codes, C.byref(eos))
            assert rc == 0, rc
            if eos.value:
                out.append(None)
                break
            out.append(list(codes))
        return out, (time.time() - t) / max(1, len(out)) * 1e3

    def kvblob(L, m, s, n):
        nb = L.s2p_session_kv_bytes(m, n)
        buf = torch.empty(nb, dtype=torch.uint8, device="cuda")
        rc = L.s2p_session_kv_save(s, n, C.c_void_p(buf.data_ptr()))
        assert rc == 0, rc
        return buf

    ids = synth.random_prompt(prompt_len, 7)
    models = {"ref": (ref, load(ref, True)), "persistent": (mine, load(mine, True)),
              "fused": (mine, load(mine, True, persistent=False)), "general": (mine, load(mine, False))}
    paths = ("persistent", "fused", "general")
    result = {"mode": mode, "n_slow": n_slow, "frames": frames, "runs": {}}
    for temp, seed0, tag in ((0.0, 0, "greedy"), (0.8, 42, "sampled")):
        # A random-weight model samples EOS now and then (one of 4097 candidates), which ends the session:
        # take the first prompt / seed with which the reference produces every requested frame.
        Lr, mr = models["ref"]
        for attempt in range(8):
            ids = synth.random_prompt(prompt_len, 7 + attempt)
            seed = seed0 + attempt
            s = session(Lr, mr, temp, seed)
            prefill(Lr, s, ids)
            probe, _ = run(Lr, s, frames)
            Lr.s2p_session_destroy(s)
            if probe[-1] is not None:
                break
        res = {}
        for name, (L, m) in models.items():
            s = session(L, m, temp, seed)
            prefill(L, s, ids)
            kv = kvblob(L, m, s, prompt_len)
            out, ms = run(L, s, frames)
            kv_after = kvblob(L, m, s, prompt_len + len([o for o in out if o is not None]) - 1) if len(out) > 1 else kv
            res[name] = (out, kv, kv_after, ms)
            if name != "ref":
                st = capi.Stats()
                assert L.s2p_b200_model_stats(m, C.byref(st)) == 0
                res[name] += ((st.last_tick_persistent, st.last_tick_fused, st.last_tick_kernels, st.last_tick_device_ms),)
            L.s2p_session_destroy(s)
        entry = {"frames_ref": len([o for o in res["ref"][0] if o is not None]), "eos": res["ref"][0][-1] is None,
                 "prompt_seed": 7 + attempt, "sampling_seed": seed}
        for name in paths:
            n_same = sum(1 for a, b in zip(res[name][0], res["ref"][0]) if a == b)
            entry[name] = {"kv_prefill_identical": bool(torch.equal(res[name][1], res["ref"][1])),
                           "kv_after_identical": bool(res[name][2].shape == res["ref"][2].shape and torch.equal(res[name][2], res["ref"][2])),
                           "frames_identical": n_same, "frames": len(res[name][0]), "ms_wall": res[name][3], "tick": res[name][4]}
        entry["ref_ms_wall"] = res["ref"][3]
        result["runs"][tag] = entry
    # lockstep batch of 3 sessions with different prompts: general path vs reference
    outs = {}
    for name in ("ref", "general"):
        L, m = models[name]
        ss = [session(L, m, 0.8, 100 + i) for i in range(3)]
        for i, s in enumerate(ss):
            prefill(L, s, synth.random_prompt(40 + 13 * i, 20 + i))
        arr = (C.c_void_p * 3)(*[s.value for s in ss])
        codes = (C.c_int32 * 30)()
        eos = (C.c_int * 3)()
        seq = []
        for _ in range(12):
            rc = L.s2p_model_batch_next_frame(m, arr, 3, codes, eos)
            assert rc == 0, rc
            seq.append((list(codes), list(eos)))
        outs[name] = seq
        for s in ss:
            L.s2p_session_destroy(s)
    result["batch3_identical"] = sum(1 for a, b in zip(outs["ref"], outs["general"]) if a == b)
    # chunked prefill == one-shot prefill (the reference states this invariant, slowar.c:271-276)
    L, m = models["general"]
    s1 = session(L, m, 0.0, 0); prefill(L, s1, ids)
    s2 = session(L, m, 0.0, 0); prefill(L, s2, ids[:prompt_len // 3]); prefill(L, s2, ids[prompt_len // 3:])
    o1, _ = run(L, s1, 4); o2, _ = run(L, s2, 4)
    result["chunked_prefill_same_frames"] = o1 == o2
    L.s2p_session_destroy(s1); L.s2p_session_destroy(s2)
    # KV-prefix reuse (the scheduler's prefix cache, src/sched/scheduler.c:384-391): save the cache of a prompt prefix,
    # load it into a fresh session, prefill only the rest; frames must equal a full prefill, here and in the reference
    k = (2 * prompt_len) // 3
    prefix_frames = {}
    for name in ("ref", "persistent"):
        L, m = models[name]
        sa = session(L, m, 0.8, 7); prefill(L, sa, ids[:k])
        blob = kvblob(L, m, sa, k)
        sb = session(L, m, 0.8, 7)
        rc = L.s2p_session_kv_load(sb, C.c_void_p(blob.data_ptr()), k)
        assert rc == 0, rc
        prefill(L, sb, ids[k:])
        sc = session(L, m, 0.8, 7); prefill(L, sc, ids)
        ob, _ = run(L, sb, 6); oc, _ = run(L, sc, 6)
        prefix_frames[name] = (ob, oc)
        for x in (sa, sb, sc):
            L.s2p_session_destroy(x)
    result["kv_prefix_equals_full_prefill"] = prefix_frames["persistent"][0] == prefix_frames["persistent"][1]
    result["kv_prefix_equals_reference"] = prefix_frames["persistent"][0] == prefix_frames["ref"][0]
    print("RESULT " + json.dumps(result))


if __name__ == "__main__":
    main()
