"""One rank of a tensor-parallel decode run (launch with torch.distributed.run, one process per GPU).

Every rank loads the same synthetic checkpoint on its own GPU, the ranks exchange the handles
of their exchange arenas (all_gather over the process group) and attach, then every rank issues
the same prefill and the same frames.  Rank 0 also runs the same prompt on a single-GPU model
first; the tensor-parallel frames must equal it code for code (every row of every matrix is
still computed by one thread block with the single-GPU arithmetic).
Usage: tp_parity_worker.py MODE N_SLOW FRAMES [PROMPT]      (MODE: int8 | int4)
Prints on rank 0: RESULT {json}
"""
import ctypes as C
import importlib
import json
import os
import sys
import time
import zlib

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
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    os.environ["S2P_DEVICE"] = str(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    capi = importlib.import_module("s2pro-native_b200.capi")
    synth = importlib.import_module("s2pro-native_b200.synth")
    ckpt = os.environ.get("S2P_TEST_CKPT_DIR", "/dev/shm") + f"/s2p_synth_l{n_slow}"
    if rank == 0:
        synth.write_checkpoint(ckpt, n_slow=n_slow, seed=0 if n_slow == 2 else 1, generator="auto")
    dist.barrier()
    L = capi.load_library()

    def load():
        opts = capi.ModelOpts(capi.GEMM_INT8, 4096, 2)
        m = C.c_void_p()
        assert L.s2p_model_load(ckpt.encode(), C.byref(opts), C.byref(m)) == 0
        return m

    def decode(m, temp, seed, n, sync=False):
        cfg = L.s2p_sampling_defaults()
        cfg.temperature, cfg.seed = temp, seed
        s = C.c_void_p()
        assert L.s2p_session_create(m, C.byref(cfg), C.byref(s)) == 0
        ids = synth.random_prompt(prompt_len, 7)
        assert L.s2p_session_prefill(s, ids.ctypes.data_as(C.c_void_p), None, len(ids), None, 0) == 0
        out, codes, eos = [], (C.c_int32 * 10)(), C.c_int(0)
        st = capi.Stats()
        dev_ms = []
        if sync:
            dist.barrier()
        t0 = time.time()
        for _ in range(n):
            rc = L.s2p_session_next_frame(s, codes, C.byref(eos))
            assert rc == 0, rc
            if eos.value:
                out.append(None)
                break
            out.append(list(codes))
            L.s2p_b200_model_stats(m, C.byref(st))
            dev_ms.append(st.last_tick_device_ms)
        wall = (time.time() - t0) / max(1, len(out)) * 1e3
        L.s2p_b200_model_stats(m, C.byref(st))
        L.s2p_session_destroy(s)
        dev_ms = sorted(dev_ms[1:]) or [0.0]
        return out, wall, dev_ms[len(dev_ms) // 2], int(st.last_tick_persistent)

    runs = ((0.0, 0, "greedy"), (0.8, 42, "sampled"))
    single = {}
    if rank == 0:
        m1 = load()
        for temp, seed, tag in runs:
            single[tag] = decode(m1, temp, seed, frames)
        L.s2p_model_free(m1)
    dist.barrier()

    m = load()
    handle = (C.c_ubyte * 64)()
    assert L.s2p_b200_model_tp_export(m, handle) == 0
    mine = torch.tensor(list(handle), dtype=torch.uint8, device="cuda")
    allh = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allh, mine)
    blob = (C.c_ubyte * (64 * world))(*[int(v) for t in allh for v in t.cpu().tolist()])
    assert L.s2p_b200_model_tp_attach(m, rank, world, blob) == 0
    dist.barrier()
    result = {"mode": mode, "n_slow": n_slow, "world": world, "runs": {}}
    for temp, seed, tag in runs:
        out, wall, dev, persistent = decode(m, temp, seed, frames, sync=True)
        # every rank must have produced the same frames
        mine_sig = torch.tensor([zlib.crc32(json.dumps(out).encode())], dtype=torch.int64, device="cuda")
        sigs = [torch.empty_like(mine_sig) for _ in range(world)]
        dist.all_gather(sigs, mine_sig)
        t = torch.tensor([wall, dev], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            ref = single[tag]
            result["runs"][tag] = {
                "frames_single": len(ref[0]), "frames_tp": len(out),
                "frames_identical": sum(1 for a, b in zip(out, ref[0]) if a == b),
                "ranks_agree": len({int(s.item()) for s in sigs}) == 1,
                "persistent": persistent, "single_persistent": ref[3],
                "ms_wall_tp": float(t[0]), "ms_device_tp": float(t[1]), "ms_wall_single": ref[1], "ms_device_single": ref[2]}
    dist.barrier()
    L.s2p_model_free(m)
    if rank == 0:
        print("RESULT " + json.dumps(result))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
