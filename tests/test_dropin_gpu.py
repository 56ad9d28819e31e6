"""Drop-in proof with compiled C callers: programs written only against the reference's public
headers (tests/dropin/*.c), and the reference's own request scheduler compiled unchanged, are linked
once with this repository's library and once with the reference's sources built as a library.  On the
same seeded checkpoint both binaries of a pair must print the same frames.

The binaries are built where the reference checkout is available (`make -C oracle dropin`, run by the
build entry) and travel prebuilt; without them the tests skip."""
import importlib
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
DROP = os.path.join(ROOT, "oracle", "_ref", "dropin")
sys.path.insert(0, ROOT)


def checkpoint():
    synth = importlib.import_module("s2pro-native_b200.synth")
    ckpt = os.environ.get("S2P_TEST_CKPT_DIR", "/dev/shm") + "/s2p_synth_l2"
    synth.write_checkpoint(ckpt, n_slow=2, seed=0, generator="auto")
    return ckpt


def run(binary, args, mode):
    path = os.path.join(DROP, binary)
    if not os.path.exists(path):
        pytest.skip("drop-in callers not built on this machine")
    env = dict(os.environ, S2P_INT8="1", S2P_QCACHE="0")
    if mode == "int4":
        env.update(S2P_INT4="1", S2P_INT4_ALL="1")
    out = subprocess.run([path] + [str(a) for a in args], capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, f"{binary}: exit {out.returncode}\n{out.stdout[-2000:]}\n{out.stderr[-3000:]}"
    assert out.stdout.rstrip().endswith("done"), out.stdout[-500:]
    return out.stdout


@pytest.mark.parametrize("mode", ["int4", "int8"])
def test_c_caller_same_frames_with_either_library(mode):
    """load -> prefill (ragged prompts) -> lockstep s2p_model_batch_next_frame, one greedy and two sampled sessions;
    then the same with a single session, which this library serves with its persistent tick kernel."""
    ckpt = checkpoint()
    for prompt, frames, sessions in ((48, 6, 3), (64, 8, 1)):
        mine = run("model_caller_mine", [ckpt, prompt, frames, sessions], mode)
        ref = run("model_caller_ref", [ckpt, prompt, frames, sessions], mode)
        assert mine == ref, f"{sessions} session(s):\n--- this library\n{mine}\n--- reference\n{ref}"
        assert mine.count("tick ") >= 3


@pytest.mark.parametrize("mode", ["int4", "int8"])
def test_reference_scheduler_runs_on_this_library(mode):
    """The reference's scheduler - admission, chunked prefill with VQ rows, KV-prefix cache save and load,
    priority first frame, lockstep batches of changing size, cancellation by the client - produces the same
    audio callbacks on top of either library (the stand-in vocoder encodes each frame's codes in its chunk)."""
    ckpt = checkpoint()
    mine = run("sched_caller_mine", [ckpt, 10], mode)
    ref = run("sched_caller_ref", [ckpt, 10], mode)
    assert mine == ref, f"--- this library\n{mine}\n--- reference\n{ref}"
    for tag in ("text-greedy", "registry-voice", "own-clip", "clone-first", "clone-again", "text-sampled"):
        assert f"{tag} frame 0" in mine, f"{tag} produced no audio:\n{mine}"
    assert "0 malformed" in mine and " 1 malformed" not in mine
