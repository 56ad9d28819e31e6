"""What a tensor-parallel model refuses (host logic, no GPU): each kv head's cache is current on one
rank only, so ticks that cannot run as the persistent kernel and cache saves answer S2P_ERR_UNSUPPORTED
instead of producing wrong frames."""
import ctypes as C

OK, UNSUPPORTED = 0, -7


def test_tick_guard(testlib):
    g = testlib.s2p_tp_guard_tick
    g.restype, g.argtypes = C.c_int, [C.c_int, C.c_int, C.c_int]
    for world in (2, 4, 8):
        assert g(world, 1, 1) == OK                 # one decoding row on the persistent kernel
        assert g(world, 1, 0) == UNSUPPORTED        # persistent path disabled (a wait gave up earlier)
        assert g(world, 2, 0) == UNSUPPORTED        # more than one session: no sharded batch path
        assert g(world, 0, 0) == OK                 # first frame after prefill: no backbone step, no cache read
    for rows in (0, 1, 5):
        assert g(1, rows, 0) == OK and g(1, rows, 1) == OK  # an unsharded model has its fallbacks


def test_kv_save_guard(testlib):
    g = testlib.s2p_tp_guard_kv_save
    g.restype, g.argtypes = C.c_int, [C.c_int]
    assert g(1) == OK
    assert all(g(w) == UNSUPPORTED for w in (2, 4, 8))
