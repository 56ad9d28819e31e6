"""The N > 1 path of the benchmark is data parallel: every rank runs an independent
replica and the ranks only meet to take the max of their timings.  This runs that
reduction with world_size 2 on the gloo backend."""
import os
import socket
import subprocess
import sys
import textwrap


def test_max_over_ranks_gloo(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    script = tmp_path / "w.py"
    script.write_text(textwrap.dedent("""
        import os, torch, torch.distributed as dist
        dist.init_process_group("gloo")
        r = dist.get_rank()
        t = torch.tensor([1.5 + r, 0.9 - 0.1 * r], dtype=torch.float64)   # (wall ms, device ms) of this replica
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        if r == 0:
            frames_per_s = dist.get_world_size() * 1 * 1e3 / float(t[0])   # replicas * batch / slowest step
            print("RESULT", float(t[0]), float(t[1]), frames_per_s)
        dist.destroy_process_group()
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", str(port), str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RESULT")][0].split()
    assert float(line[1]) == 2.5 and float(line[2]) == 0.9 and abs(float(line[3]) - 800.0) < 1e-9
