"""Bounded waits that run out.  Every wait of the persistent tick kernel (mbarrier, flagged word, grid
barrier) has a deadline on the GPU-wide timer; past it the wait records a code, the kernel winds down
and ends normally, and the host turns the code into S2P_ERR_INTERNAL.  Here the deadline is lowered so
that this happens within microseconds: nothing hangs, traps or faults.

Uses the test twin of the library throughout (the deadline is a constant of the library image that
launches the kernels)."""
import ctypes as C
import importlib
import os

import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

PIPE_ERR_TMA_WAIT, PIPE_ERR_FLAG_WAIT = 1, 3
S2P_ERR_INTERNAL = -8


def _hooks(tl):
    tl.pipe_wait_probe.restype = C.c_int
    tl.pipe_wait_probe.argtypes = [C.c_int, C.c_ulonglong, C.POINTER(C.c_int), C.POINTER(C.c_ulonglong), C.POINTER(C.c_int)]
    tl.mega_set_wait_ns.restype = C.c_int
    tl.mega_set_wait_ns.argtypes = [C.c_ulonglong]
    return tl


@pytest.mark.parametrize("which,code", [(0, PIPE_ERR_TMA_WAIT), (1, PIPE_ERR_FLAG_WAIT)])
def test_a_wait_nobody_satisfies_gives_up_at_its_deadline(testlib, which, code):
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    tl = _hooks(testlib)
    limit_ns = 200_000
    status, elapsed, got = C.c_int(0), C.c_ulonglong(0), C.c_int(1)
    assert tl.pipe_wait_probe(which, limit_ns, C.byref(status), C.byref(elapsed), C.byref(got)) == 0
    assert got.value == 0, "the wait must report failure"
    assert status.value == code
    assert limit_ns <= elapsed.value < 50 * limit_ns, elapsed.value  # gave up at the deadline, not at a poll-count backstop


def test_persistent_tick_gives_up_cleanly_and_the_model_falls_back(testlib, capi):
    """A model on the persistent tick; then the deadline drops to 100 ns, so the kernel's first wait runs
    out: that tick answers S2P_ERR_INTERNAL, the persistent path is switched off, and with the deadline
    restored the session goes on through per-stage launches."""
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    tl = _hooks(testlib)
    capi.bind(tl, capi.EXT_PROTOTYPES)
    synth = importlib.import_module("s2pro-native_b200.synth")
    os.environ.update({"S2P_INT8": "1", "S2P_INT4": "1", "S2P_INT4_ALL": "1", "S2P_QCACHE": "0", "S2P_NO_FUSED": "0", "S2P_NO_MEGA": "0"})
    ckpt = os.environ.get("S2P_TEST_CKPT_DIR", "/dev/shm") + "/s2p_synth_l2"
    synth.write_checkpoint(ckpt, n_slow=2, seed=0, generator="auto")
    opts = capi.ModelOpts(capi.GEMM_INT8, 1024, 1)
    m = C.c_void_p()
    capi.check(tl.s2p_model_load(ckpt.encode(), C.byref(opts), C.byref(m)), "load")
    cfg = tl.s2p_sampling_defaults(); cfg.temperature = 0.0
    s = C.c_void_p()
    capi.check(tl.s2p_session_create(m, C.byref(cfg), C.byref(s)), "session")
    ids = synth.random_prompt(24, 5)
    capi.check(tl.s2p_session_prefill(s, ids.ctypes.data_as(C.c_void_p), None, len(ids), None, 0), "prefill")
    codes = (C.c_int32 * 10)(); eos = C.c_int(0)
    st = capi.Stats()
    for _ in range(3):
        capi.check(tl.s2p_session_next_frame(s, codes, C.byref(eos)), "frame")
    capi.check(tl.s2p_b200_model_stats(m, C.byref(st)), "stats")
    assert st.last_tick_persistent == 1
    try:
        assert tl.mega_set_wait_ns(100) == 0
        rc = tl.s2p_session_next_frame(s, codes, C.byref(eos))
    finally:
        assert tl.mega_set_wait_ns(2_000_000_000) == 0
    assert rc == S2P_ERR_INTERNAL, rc
    torch.cuda.synchronize()  # the context is intact
    for _ in range(3):
        capi.check(tl.s2p_session_next_frame(s, codes, C.byref(eos)), "frame after the give-up")
        assert all(0 <= c < 4096 for c in codes)
    capi.check(tl.s2p_b200_model_stats(m, C.byref(st)), "stats")
    assert st.last_tick_persistent == 0, "the persistent path must stay off after a give-up"
    tl.s2p_session_destroy(s)
    tl.s2p_model_free(m)


def test_batched_tensor_core_linear_gives_up_cleanly_and_the_exact_kernel_takes_over(testlib, capi):
    """A lockstep batch of 17 sessions runs its linears on the tensor-core kernel; with that kernel's wait
    deadline at 100 ns its first wait runs out: the tick answers S2P_ERR_INTERNAL, TMEM is released, the
    status code and the arrival counters are cleared, and later ticks take the exact-order kernel."""
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    tl = _hooks(testlib)
    tl.skinny_set_wait_ns.restype = C.c_int
    tl.skinny_set_wait_ns.argtypes = [C.c_ulonglong]
    capi.bind(tl, capi.EXT_PROTOTYPES)
    synth = importlib.import_module("s2pro-native_b200.synth")
    os.environ.update({"S2P_INT8": "1", "S2P_INT4": "1", "S2P_INT4_ALL": "1", "S2P_QCACHE": "0", "S2P_NO_TC": "0"})
    ckpt = os.environ.get("S2P_TEST_CKPT_DIR", "/dev/shm") + "/s2p_synth_l2"
    synth.write_checkpoint(ckpt, n_slow=2, seed=0, generator="auto")
    n = 17
    opts = capi.ModelOpts(capi.GEMM_INT8, 256, n)
    m = C.c_void_p()
    capi.check(tl.s2p_model_load(ckpt.encode(), C.byref(opts), C.byref(m)), "load")
    sess = []
    for i in range(n):
        cfg = tl.s2p_sampling_defaults(); cfg.temperature = 0.0
        s = C.c_void_p()
        capi.check(tl.s2p_session_create(m, C.byref(cfg), C.byref(s)), "session")
        ids = synth.random_prompt(12, 40 + i)
        capi.check(tl.s2p_session_prefill(s, ids.ctypes.data_as(C.c_void_p), None, len(ids), None, 0), "prefill")
        sess.append(s)
    arr = (C.c_void_p * n)(*[s.value for s in sess])
    codes = (C.c_int32 * (10 * n))(); eos = (C.c_int * n)()
    st = capi.Stats()
    for _ in range(3):
        capi.check(tl.s2p_model_batch_next_frame(m, arr, n, codes, eos), "tick")
    capi.check(tl.s2p_b200_model_stats(m, C.byref(st)), "stats")
    kernels_tc = st.last_tick_kernels
    try:
        assert tl.skinny_set_wait_ns(100) == 0
        rc = tl.s2p_model_batch_next_frame(m, arr, n, codes, eos)
    finally:
        assert tl.skinny_set_wait_ns(2_000_000_000) == 0
    assert rc == S2P_ERR_INTERNAL, rc
    torch.cuda.synchronize()
    for _ in range(3):
        capi.check(tl.s2p_model_batch_next_frame(m, arr, n, codes, eos), "tick after the give-up")
        assert all(0 <= c < 4096 for c in codes)
    capi.check(tl.s2p_b200_model_stats(m, C.byref(st)), "stats")
    assert st.last_tick_kernels > kernels_tc, "later ticks must run the exact-order linears (more launches: 16 rows at a time)"
    for s in sess:
        tl.s2p_session_destroy(s)
    tl.s2p_model_free(m)
