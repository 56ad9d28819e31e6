"""bench.py's own multi-rank bookkeeping on CPU ranks (gloo, world size 2): the timed region takes the
maximum over the ranks, and the job throughput is the sum of what every rank advances per tick."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import ctypes as C, json, os, sys, time
    sys.path.insert(0, os.environ["S2P_ROOT"])
    import torch.distributed as dist
    import bench

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")

    class Stats(C.Structure):
        _fields_ = [("last_tick_device_ms", C.c_float)]
    class Capi:
        Stats = Stats
    class Lib:  # stands in for the C library's stats call: rank r reports 2 + r ms of device time per tick
        @staticmethod
        def s2p_b200_model_stats(model, ref):
            ref._obj.last_tick_device_ms = 2.0 + rank
    class Engine:
        m = None
        ticks = 0
        def tick(self):
            self.ticks += 1
            time.sleep(0.010 * (1 + rank))  # rank 1 is the slow one
            return False

    eng = Engine()
    wall, dev, dev_ms, eos = bench.timed_ticks(eng, Lib, Capi, 5, world, device="cpu")
    mx = bench.max_over_ranks([rank + 0.5, 10 - rank], world, device="cpu")
    if rank == 0:
        print(json.dumps({"wall": wall, "dev": dev, "own": dev_ms, "ticks": eng.ticks, "eos": eos, "mx": mx,
                          "fps": bench.job_frames_per_s(world, 32, wall)}))
    dist.barrier()
    dist.destroy_process_group()
""")


def test_timed_region_takes_the_slowest_rank(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, S2P_ROOT=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29631", WORLD_SIZE="2")
    procs = []
    for rank in range(2):
        procs.append(subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(rank)), stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=120) for p in procs]
    assert all(p.returncode == 0 for p in procs), [o[1][-2000:] for o in outs]
    import json
    r = json.loads(outs[0][0].strip().splitlines()[-1])
    assert r["ticks"] == 5 and r["eos"] is False
    assert r["own"] == [2.0] * 5            # rank 0's own device times ...
    assert abs(r["dev"] - 3.0) < 1e-9       # ... but the reported one is the slowest rank's
    assert r["wall"] >= 20.0 * 0.95         # rank 1 sleeps 20 ms per tick
    assert r["mx"] == [1.5, 10.0]
    assert abs(r["fps"] - 2 * 32 * 1e3 / r["wall"]) < 1e-6


def test_job_throughput_and_single_rank_passthrough():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.job_frames_per_s(8, 32, 16.0) == 8 * 32 * 1e3 / 16.0
    assert bench.max_over_ranks([1.25, 2], 1) == [1.25, 2.0]
    a = bench.algorithmic_bytes_per_frame("int4", 36)
    assert abs(a - 4378151428) < 64  # weights + scales one all-INT4 batch-1 frame streams
