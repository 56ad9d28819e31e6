"""Host-side launch plan of the batched tensor-core linear (s2pro-native_b200/csrc/cuda/skinny.cu), no GPU:
for every decode shape of the model and every batch size the plan must fit the SM's shared memory, keep the
ring depths the kernel's copy-group counting assumes, cover every row tile exactly once and stay inside the
split-K scratch."""
import ctypes as C
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "s2pro-native_b200", "libs2pro_b200_test.so")

KINDS = {0: "int8 per channel", 1: "int8 grouped", 2: "int4 packed"}
SHAPES = [(6144, 2560), (2560, 4096), (19456, 2560), (2560, 9728), (4096, 2560), (4097, 2560), (384, 512)]
SMEM_MAX = 226 * 1024          # dynamic shared memory the kernels ask the driver for
SCRATCH_FLOATS_PER_ROW = 8 * 6144


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        pytest.fail("test twin of the library is not built (run __graft_entry__.build())")
    L = C.CDLL(LIB)
    L.skinny_plan_probe.argtypes = [C.c_int] * 5 + [C.POINTER(C.c_int)]
    L.skinny_plan_probe.restype = C.c_int
    L.skinny_tune.argtypes = [C.c_int, C.c_int]
    return L


def plan(L, kind, N, K, M, scratch_rows):
    out = (C.c_int * 10)()
    ok = L.skinny_plan_probe(kind, N, K, M, scratch_rows, out)
    keys = ("lgNB", "tiles", "S", "KS", "nt", "kc", "D", "DW", "grid", "smem")
    return ok, dict(zip(keys, out))


def stage_and_ring_bytes(kind, p):
    """Shared memory the kernel carves up, from the same formulas as its geometry struct."""
    NB, kc, nt = 1 << p["lgNB"], p["kc"], p["nt"]
    upr = kc // 32 if kind == 2 else kc // 16
    nld = upr * 128 // nt
    ncp = nld * (256 // kc)
    sup = ncp * nt * 16 + (0 if kind == 0 else ncp * nt * 4)
    return 3 * (128 * kc * 2 + NB * kc * 2) + 128 + p["D"] * NB * kc * 2 + p["DW"] * sup


@pytest.mark.parametrize("shape", [1, 0, 2])
@pytest.mark.parametrize("kind", [0, 1, 2])
def test_plan_fits_and_covers(lib, kind, shape):
    lib.skinny_tune(148, shape)
    try:
        for N, K in SHAPES:
            for M in (1, 16, 17, 32, 33, 64, 100, 128):
                for scratch_rows in (0, M, 256):
                    ok, p = plan(lib, kind, N, K, M, scratch_rows)
                    what = f"{KINDS[kind]} N={N} K={K} M={M} scratch={scratch_rows} shape={shape}: {p}"
                    assert ok == 1, what
                    assert (1 << p["lgNB"]) >= M and p["lgNB"] >= 4 and ((1 << p["lgNB"]) < 2 * M or p["lgNB"] == 4), what
                    assert p["tiles"] == (N + 127) // 128, what
                    assert (p["nt"], p["kc"]) in ((512, 128), (256, 128), (256, 64)), what
                    assert p["smem"] <= SMEM_MAX and p["smem"] == stage_and_ring_bytes(kind, p), what
                    sps = 256 // p["kc"]
                    assert p["DW"] in (2, 3) and 2 <= p["D"] <= min(8, sps * (p["DW"] - 1) + 1), what
                    # the split: pieces first, whole tiles behind them; every tile exactly once
                    assert 0 <= p["S"] <= p["tiles"] and p["S"] <= 256, what
                    assert p["grid"] == p["tiles"] - p["S"] + p["S"] * p["KS"], what
                    if p["S"]:
                        assert 2 <= p["KS"] <= min(10, K // 256), what
                        assert scratch_rows >= M, what
                        assert p["S"] * p["KS"] * M * 128 <= SCRATCH_FLOATS_PER_ROW * scratch_rows, what
                    else:
                        assert p["KS"] == 1, what
    finally:
        lib.skinny_tune(148, 1)


def test_model_shapes_fill_the_gpu(lib):
    """With scratch, the model's four decode matrices launch about one CTA per SM, or a little more in pieces."""
    lib.skinny_tune(148, 1)
    for (N, K), want in (((6144, 2560), (48, 48, 3)), ((2560, 4096), (20, 20, 7)), ((2560, 9728), (20, 20, 7)),
                         ((19456, 2560), (152, 4, 10))):
        ok, p = plan(lib, 2, N, K, 32, 32)
        assert ok == 1 and (p["tiles"], p["S"], p["KS"]) == want, p
        assert p["grid"] <= 148 or p["S"] * p["KS"] <= 148, p
