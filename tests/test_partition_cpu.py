"""Host-side logic of the persistent tick that needs no GPU: the row partition that the CTAs of
one GPU - or of all ranks of a tensor-parallel group - share, the chunking of a CTA's rows into
ring slots, the shared-memory layout, and the kv-head-to-rank placement."""
import ctypes as C
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "s2pro-native_b200", "libs2pro_b200_test.so")


class Layout(C.Structure):
    _fields_ = [("x_bytes", C.c_int), ("slot_bytes", C.c_int), ("part_bytes", C.c_int), ("total_bytes", C.c_int)]


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        pytest.fail("test twin of the library is not built (run __graft_entry__.build())")
    L = C.CDLL(LIB)
    L.mega_geom_probe.argtypes = [C.c_int] * 5 + [C.POINTER(C.c_int)]
    L.mega_layout.argtypes = [C.c_int, C.POINTER(Layout)]
    L.mega_max_local_rows.argtypes = [C.POINTER(Layout), C.c_int]
    return L


def geom(L, N, swiglu, rpc, cta, n_cta):
    out = (C.c_int * 4)()
    L.mega_geom_probe(N, swiglu, rpc, cta, n_cta, out)
    return tuple(out)


SHAPES = [(6144, 0), (2560, 0), (19456, 1), (4096, 0), (1, 0)]  # (rows, SwiGLU pairs?) of the model's linears + the EOS row


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_rows_are_partitioned_once_over_all_ranks(lib, world):
    n_cta = 148 * world
    for N, sw in SHAPES:
        units = N // 2 if sw else N
        nxt = 0
        sizes = []
        for cta in range(n_cta):
            row0, cnt, rc, n_chunks = geom(lib, N, sw, 13, cta, n_cta)
            assert row0 == nxt and cnt >= 0
            nxt += cnt
            sizes.append(cnt)
            if cnt:
                assert 1 <= rc <= 13 and (n_chunks - 1) * rc < cnt <= n_chunks * rc
            else:
                assert n_chunks == 0
        assert nxt == units
        assert max(sizes) - min(sizes) <= 1  # balanced to one row


@pytest.mark.parametrize("x_bytes", [2 * 9728, 4 * 9728])
def test_layout_fits_and_chunks_have_equal_counts(lib, x_bytes):
    lay = Layout()
    lib.mega_layout(x_bytes, C.byref(lay))
    assert lay.total_bytes <= 225 * 1024 and lay.slot_bytes % 16 == 0 and lay.part_bytes % 16 == 0
    assert lay.total_bytes >= 4 * lay.slot_bytes + lay.x_bytes + 2 * lay.part_bytes
    int4 = x_bytes == 2 * 9728
    for N, K, sw in [(6144, 2560, 0), (2560, 4096, 0), (19456, 2560, 1), (2560, 9728, 0)]:
        row_bytes = (K // 2 + K // 16) if int4 else K  # packed nibbles + f16 group scales, or int8 codes
        regions = 2 if sw else 1
        rpc = min(lay.slot_bytes // (regions * row_bytes), lib.mega_max_local_rows(C.byref(lay), K) // regions)
        assert rpc >= 1
        assert rpc * regions * (K // 512) * 128 <= lay.part_bytes  # the partial buffer holds a chunk
        counts = {geom(lib, N, sw, rpc, cta, 148)[3] for cta in range(148)}
        assert len(counts) == 1, (N, K, counts)  # no CTA needs an extra chunk


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_kv_head_workers_share_a_rank(lib, world):
    n_local, n_cta = 148, 148 * world
    workers = n_cta // 8
    for g in range(workers * 8):
        kvh = g // workers
        assert g // n_local == (kvh * world) // 8 or world == 1  # rank of the CTA == rank that owns the head
    # fast-AR heads: head h runs in CTA h % (8 / world) of rank h // (8 / world)
    per = 8 // world
    assert sorted((h // per, h % per) for h in range(8)) == [(r, c) for r in range(world) for c in range(per)]


@pytest.mark.parametrize("N,n_cta", [(19456, 148), (155776, 1184), (1813000, 1184), (1814000, 1184), (4000000, 1184), (2**31 - 1, 148)])
def test_partition_matches_the_exact_quotients_on_both_arithmetic_paths(lib, N, n_cta):
    """The row partition uses 32-bit divisions where the products fit and 64-bit ones beyond (around 1.81 M rows
    at 1184 CTAs): both must give floor(N * cta / n_cta)."""
    for cta in (0, 1, n_cta // 3, n_cta - 2, n_cta - 1):
        row0, cnt, rc, n_chunks = geom(lib, N, 0, 1 << 20, cta, n_cta)
        assert row0 == N * cta // n_cta
        assert cnt == N * (cta + 1) // n_cta - row0
