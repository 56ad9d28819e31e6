"""Kernel-level parity on the GPU: every primitive of the decode tick against
the reference's own CUDA kernels rebuilt for sm_100a (bitwise), on seeded
inputs.  The reference library and this library receive the same device
buffers through the same C signatures."""
import ctypes as C

import numpy as np
import pytest

from _internal_abi import (AttnArgs, KvRef, LinRef, QkvPostArgs, SamplerState, TickBeginArgs, VecRef, bind_internal,
                           bind_ref_private)

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

QH, KVH, HD, D, F = 32, 8, 128, 2560, 9728
EPS, BASE = 1e-6, 1000000.0


def dev():
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    return torch.device("cuda:0")


def p(t):
    return C.c_void_p(t.data_ptr())


def bits(t):
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16)
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    return t


def assert_same(a, b, what):
    torch.cuda.synchronize()
    a, b = bits(a), bits(b)
    n = int((a != b).sum())
    assert n == 0, f"{what}: {n} of {a.numel()} elements differ"


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


@pytest.fixture(scope="module")
def libs(mine, testlib, ref):
    dev()
    return mine, bind_internal(testlib), bind_ref_private(ref)


def test_rms_norm_and_head_norm(libs):
    mine, _, ref = libs
    x = rnd(7, D, seed=1); w = rnd(D, seed=2) + 1.0
    y1 = torch.empty_like(x); y2 = torch.empty_like(x)
    assert mine.s2pk_rms_norm(p(x), p(w), p(y1), 7, D, EPS, None) == 0
    assert ref.s2pk_rms_norm(p(x), p(w), p(y2), 7, D, EPS, None) == 0
    assert_same(y1, y2, "rms_norm")
    q1 = rnd(3, QH, HD, seed=3); q2 = q1.clone(); hw = rnd(HD, seed=4) + 1.0
    assert mine.s2pk_qk_norm(p(q1), p(hw), 3, QH, HD, EPS, None) == 0
    assert ref.s2pk_qk_norm(p(q2), p(hw), 3, QH, HD, EPS, None) == 0
    assert_same(q1, q2, "qk_norm")


def test_rope_silu_add_embed_argmax(libs):
    mine, _, ref = libs
    q1 = rnd(5, QH, HD, seed=5); k1 = rnd(5, KVH, HD, seed=6); q2, k2 = q1.clone(), k1.clone()
    assert mine.s2pk_rope(p(q1), p(k1), 5, QH, KVH, HD, 700, BASE, None) == 0
    assert ref.s2pk_rope(p(q2), p(k2), 5, QH, KVH, HD, 700, BASE, None) == 0
    assert_same(q1, q2, "rope q"); assert_same(k1, k2, "rope k")
    gu = rnd(4, 2 * F, scale=3.0, seed=7); h1 = torch.empty(4, F, dtype=torch.bfloat16, device="cuda"); h2 = torch.empty_like(h1)
    assert mine.s2pk_silu_mul(p(gu), p(h1), 4, F, None) == 0
    assert ref.s2pk_silu_mul(p(gu), p(h2), 4, F, None) == 0
    assert_same(h1, h2, "silu_mul")
    a1 = rnd(4, D, seed=8); a2 = a1.clone(); b = rnd(4, D, seed=9)
    assert mine.s2pk_add(p(a1), p(b), 4 * D, None) == 0
    assert ref.s2pk_add(p(a2), p(b), 4 * D, None) == 0
    assert_same(a1, a2, "add")
    table = rnd(1000, D, seed=10); ids = torch.tensor([5, 999, 0, 17], dtype=torch.int64, device="cuda")
    o1 = torch.empty(4, D, dtype=torch.bfloat16, device="cuda"); o2 = torch.empty_like(o1)
    assert mine.s2pk_embed(p(table), p(ids), p(o1), 4, D, None) == 0
    assert ref.s2pk_embed(p(table), p(ids), p(o2), 4, D, None) == 0
    assert_same(o1, o2, "embed")
    lg = rnd(6, 4096, seed=11); lg[2, 77] = lg[2].max() + 1; lg[2, 3000] = lg[2, 77]  # exact tie: lowest index wins
    i1 = torch.empty(6, dtype=torch.int32, device="cuda"); i2 = torch.empty_like(i1)
    assert mine.s2pk_argmax(p(lg), p(i1), 6, 4096, None) == 0
    assert ref.s2pk_argmax(p(lg), p(i2), 6, 4096, None) == 0
    assert_same(i1, i2, "argmax")
    assert int(i1[2]) == 77


def _ref_qkv_post(ref, qkv, rows, pos0, max_seq, qn, kn, kv8):
    """The reference's op sequence: split, qk-norm x2, rope, append (src/slowar/slowar.c:166-243)."""
    q = torch.empty(rows, QH * HD, dtype=torch.bfloat16, device="cuda")
    k = torch.empty(rows, KVH * HD, dtype=torch.bfloat16, device="cuda"); v = torch.empty_like(k)
    assert ref.s2pk_qkv_split(p(qkv), p(q), p(k), p(v), rows, QH * HD, KVH * HD, None) == 0
    if qn is not None:
        assert ref.s2pk_qk_norm(p(q), p(qn), rows, QH, HD, EPS, None) == 0
        assert ref.s2pk_qk_norm(p(k), p(kn), rows, KVH, HD, EPS, None) == 0
    assert ref.s2pk_rope(p(q), p(k), rows, QH, KVH, HD, pos0, BASE, None) == 0
    if kv8:
        kc = torch.zeros(KVH, max_seq, HD, dtype=torch.int8, device="cuda"); vc = torch.zeros_like(kc)
        ks = torch.zeros(KVH, max_seq, 4, dtype=torch.float16, device="cuda"); vs = torch.zeros_like(ks)
        assert ref.s2pk_kv_append8(p(k), p(v), p(kc), p(vc), p(ks), p(vs), rows, KVH, HD, pos0, max_seq, 8, None) == 0
        return q, kc, vc, ks, vs
    kc = torch.zeros(KVH, max_seq, HD, dtype=torch.bfloat16, device="cuda"); vc = torch.zeros_like(kc)
    assert ref.s2pk_kv_append(p(k), p(v), p(kc), p(vc), rows, KVH, HD, pos0, max_seq, None) == 0
    return q, kc, vc, None, None


def _my_caches(max_seq, kv8):
    """[2][KVH][max_seq][128] payload (+ [2][KVH][max_seq][4] f16 scales)."""
    kv = torch.zeros(2, KVH, max_seq, HD, dtype=torch.int8 if kv8 else torch.bfloat16, device="cuda")
    kvs = torch.zeros(2, KVH, max_seq, 4, dtype=torch.float16, device="cuda")
    ref_ = KvRef()
    ref_.base0 = kv.data_ptr(); ref_.k_off = 0; ref_.v_off = kv[0].numel() * kv.element_size()
    ref_.sbase0 = kvs.data_ptr(); ref_.ks_off = 0; ref_.vs_off = kvs[0].numel() * 2
    return kv, kvs, ref_


@pytest.mark.parametrize("kv8", [0, 1])
@pytest.mark.parametrize("with_norm", [True, False])
def test_qkv_post_matches_reference_sequence(libs, kv8, with_norm):
    _, tl, ref = libs
    rows, pos0, max_seq = 9, 37, 128
    qkv = rnd(rows, (QH + 2 * KVH) * HD, seed=20 + kv8)
    qn = (rnd(HD, seed=21) + 1.0) if with_norm else None
    kn = (rnd(HD, seed=22) + 1.0) if with_norm else None
    q_ref, kc, vc, ks, vs = _ref_qkv_post(ref, qkv, rows, pos0, max_seq, qn, kn, kv8)
    kv, kvs, kvref = _my_caches(max_seq, kv8)
    q = torch.empty(rows, QH * HD, dtype=torch.bfloat16, device="cuda")
    a = QkvPostArgs()
    a.qkv = qkv.data_ptr(); a.q = q.data_ptr()
    a.q_norm = qn.data_ptr() if with_norm else None; a.k_norm = kn.data_ptr() if with_norm else None
    a.eps = EPS; a.rope_base = BASE; a.q_heads = QH; a.kv_heads = KVH; a.max_seq = max_seq; a.kv8 = kv8; a.head_dim = HD
    a.pos0 = pos0; a.pos_row_step = 1; a.kv = kvref
    assert tl.qkv_post(C.byref(a), rows, None) == 0
    assert_same(q, q_ref, "q"); assert_same(kv[0], kc, "k cache"); assert_same(kv[1], vc, "v cache")
    if kv8:
        assert_same(kvs[0], ks, "k scales"); assert_same(kvs[1], vs, "v scales")


def _filled_cache(max_seq, kv8, seed):
    """A cache produced by the reference's own append path, so both sides read real quantised data."""
    kvbuf, kvs, kvref = _my_caches(max_seq, kv8)
    k = rnd(max_seq, KVH * HD, seed=seed); v = rnd(max_seq, KVH * HD, seed=seed + 1)
    return kvbuf, kvs, kvref, k, v


@pytest.mark.parametrize("kv8", [0, 1])
@pytest.mark.parametrize("pos0,rows", [(0, 1), (0, 40), (100, 30), (250, 6), (0, 300), (120, 9), (127, 2), (190, 130), (0, 1100), (1000, 50)])
def test_single_pass_attention(libs, kv8, pos0, rows):
    """One row goes to the single-row kernel, several consecutive rows of one cache (a prompt slice) to the
    row-block kernel: blocks of 4 rows, ragged last block, blocks that straddle a 128-position tile boundary."""
    mine, tl, ref = libs
    max_seq = max(320, ((pos0 + rows + 63) // 64) * 64)
    kvbuf, kvs, kvref, k, v = _filled_cache(max_seq, kv8, 30)
    if kv8:
        assert ref.s2pk_kv_append8(p(k), p(v), p(kvbuf[0]), p(kvbuf[1]), p(kvs[0]), p(kvs[1]), max_seq, KVH, HD, 0, max_seq, 8, None) == 0
    else:
        assert ref.s2pk_kv_append(p(k), p(v), p(kvbuf[0]), p(kvbuf[1]), max_seq, KVH, HD, 0, max_seq, None) == 0
    q = rnd(rows, QH * HD, seed=33)
    o1 = torch.empty_like(q); o2 = torch.empty_like(q)
    a = AttnArgs()
    a.q = q.data_ptr(); a.out = o1.data_ptr(); a.q_heads = QH; a.kv_heads = KVH; a.max_seq = max_seq; a.kv8 = kv8; a.head_dim = HD
    a.pos0 = pos0; a.pos_row_step = 1; a.kv = kvref
    assert tl.attn_single(C.byref(a), rows, None) == 0
    if kv8:
        assert ref.s2pk_attention8(p(q), p(kvbuf[0]), p(kvbuf[1]), p(kvs[0]), p(kvs[1]), p(o2), rows, QH, KVH, HD, pos0, max_seq, 8, None) == 0
    else:
        assert ref.s2pk_attention(p(q), p(kvbuf[0]), p(kvbuf[1]), p(o2), rows, QH, KVH, HD, pos0, max_seq, None) == 0
    assert_same(o1, o2, f"single-pass attention kv8={kv8}")
    if not kv8:  # the contract launcher goes the same way
        o3 = torch.empty_like(q)
        assert mine.s2pk_attention(p(q), p(kvbuf[0]), p(kvbuf[1]), p(o3), rows, QH, KVH, HD, pos0, max_seq, None) == 0
        assert_same(o3, o2, "s2pk_attention")


@pytest.mark.parametrize("kv8", [0, 1])
@pytest.mark.parametrize("lens", [[1], [63], [64], [65], [200, 7, 713], [1024]])
def test_split_k_decode_attention(libs, kv8, lens):
    _split_k_decode_attention(libs, kv8, lens, 1088, (1, 3, 16))


@pytest.mark.parametrize("kv8", [1, 0])
def test_split_k_decode_attention_batch_of_32(libs, kv8):
    """A lockstep batch: 32 rows with contexts of 1300-3100 positions (the shared 1024-token prefix plus
    256-2048 own tokens), 8 workers per (row, kv head) as the batched tick launches it (the grid is large
    enough for the variant in which one thread scores all four heads of a position)."""
    lens = [int(v) for v in np.random.default_rng(7).integers(1300, 3101, size=32)]
    _split_k_decode_attention(libs, kv8, lens, 3136, (8,))


def test_split_k_decode_attention_8192_positions(libs):
    """The long-context end of the data-parallel configuration: two rows with 8192 and 8000 cached
    positions in an INT8 cache of 8256 slots (129 splits), with the worker counts the tick uses."""
    _split_k_decode_attention(libs, 1, [8192, 8000], 8256, (8, 18))


@pytest.mark.parametrize("kv8", [1, 0])
def test_split_k_decode_attention_cache_not_16_byte_aligned(libs, kv8):
    """Caches whose base addresses are only 8-byte aligned: the lockstep kernel must take its 4-byte copy path
    (a 16-byte asynchronous copy from such an address would be illegal) and give the same bits."""
    _split_k_decode_attention(libs, kv8, [130, 64, 700], 768, (4,), shift_bytes=8)


def _split_k_decode_attention(libs, kv8, lens, max_seq, workers_list, shift_bytes=0):
    _, tl, ref = libs
    rows = len(lens)
    caches = []
    for r in range(rows):
        kvbuf, kvs, kvref, k, v = _filled_cache(max_seq, kv8, 40 + 2 * r)
        if kv8:
            assert ref.s2pk_kv_append8(p(k), p(v), p(kvbuf[0]), p(kvbuf[1]), p(kvs[0]), p(kvs[1]), max_seq, KVH, HD, 0, max_seq, 8, None) == 0
        else:
            assert ref.s2pk_kv_append(p(k), p(v), p(kvbuf[0]), p(kvbuf[1]), max_seq, KVH, HD, 0, max_seq, None) == 0
        caches.append((kvbuf, kvs))
    q = rnd(rows, QH * HD, seed=50)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device="cuda")
    ptr_t = lambda xs: torch.tensor(xs, dtype=torch.int64, device="cuda")
    kptr = ptr_t([c[0][0].data_ptr() for c in caches]); vptr = ptr_t([c[0][1].data_ptr() for c in caches])
    ksptr = ptr_t([c[1][0].data_ptr() for c in caches]); vsptr = ptr_t([c[1][1].data_ptr() for c in caches])
    n_slots = (max_seq + 63) // 64
    part = torch.empty(rows * QH * n_slots * 130, dtype=torch.float32, device="cuda")
    o_ref = torch.empty_like(q)
    max_len = max(lens)
    if kv8:
        assert ref.s2pk_attention8_decode(p(q), p(kptr), p(vptr), p(ksptr), p(vsptr), p(o_ref), rows, QH, KVH, HD, p(pos), max_seq, max_len, p(part), 8, None) == 0
    else:
        assert ref.s2pk_attention_decode(p(q), p(kptr), p(vptr), p(o_ref), rows, QH, KVH, HD, p(pos), max_seq, max_len, p(part), None) == 0
    torch.cuda.synchronize()
    v_off = caches[0][0][0].numel() * caches[0][0].element_size()
    vs_off = caches[0][1][0].numel() * 2
    keep = []
    if shift_bytes:  # byte copies of every cache at an address shift_bytes past a 256-byte boundary
        def shifted(t):
            raw = torch.empty(t.numel() * t.element_size() + 256, dtype=torch.uint8, device="cuda")
            view = raw[shift_bytes:shift_bytes + t.numel() * t.element_size()]
            view.copy_(t.contiguous().view(torch.uint8).flatten())
            keep.append(raw)
            assert view.data_ptr() % 16 == shift_bytes % 16
            return view
        caches = [(shifted(c[0]), shifted(c[1])) for c in caches]
    for workers in workers_list:
        o = torch.zeros_like(q)
        ctr = torch.zeros(rows * KVH, dtype=torch.int32, device="cuda")
        base = ptr_t([c[0].data_ptr() for c in caches]); sbase = ptr_t([c[1].data_ptr() for c in caches])
        a = AttnArgs()
        a.q = q.data_ptr(); a.out = o.data_ptr(); a.q_heads = QH; a.kv_heads = KVH; a.max_seq = max_seq; a.kv8 = kv8; a.head_dim = HD
        a.pos_arr = pos.data_ptr()
        a.kv.bases = base.data_ptr(); a.kv.k_off = 0; a.kv.v_off = v_off
        a.kv.sbases = sbase.data_ptr(); a.kv.ks_off = 0; a.kv.vs_off = vs_off
        a.part = part.data_ptr(); a.counters = ctr.data_ptr(); a.n_split_slots = n_slots; a.workers = workers
        assert tl.attn_decode(C.byref(a), rows, None) == 0
        assert_same(o, o_ref, f"split-K decode attention kv8={kv8} workers={workers}")
        assert int(ctr.abs().sum()) == 0, "arrival counters must be left at zero"


@pytest.mark.parametrize("kv8", [0, 1])
def test_fused_attention_prologue(libs, kv8):
    """Attention that does qk-norm, RoPE and the KV append itself == qkv_post then attention."""
    _, tl, ref = libs
    max_seq, pos_v = 512, 300
    kvbuf, kvs, kvref, k, v = _filled_cache(max_seq, kv8, 60)
    if kv8:
        assert ref.s2pk_kv_append8(p(k), p(v), p(kvbuf[0]), p(kvbuf[1]), p(kvs[0]), p(kvs[1]), pos_v, KVH, HD, 0, max_seq, 8, None) == 0
    else:
        assert ref.s2pk_kv_append(p(k), p(v), p(kvbuf[0]), p(kvbuf[1]), pos_v, KVH, HD, 0, max_seq, None) == 0
    kv_b, kvs_b = kvbuf.clone(), kvs.clone()
    qkv = rnd(1, (QH + 2 * KVH) * HD, seed=61); qn = rnd(HD, seed=62) + 1.0; kn = rnd(HD, seed=63) + 1.0
    pos = torch.tensor([pos_v], dtype=torch.int32, device="cuda")
    n_slots = (max_seq + 63) // 64
    part = torch.empty(QH * n_slots * 130, dtype=torch.float32, device="cuda")
    ctr = torch.zeros(KVH, dtype=torch.int32, device="cuda")

    def args(kvt, kvst, out, q=None):
        a = AttnArgs()
        a.q = q.data_ptr() if q is not None else None
        a.out = out.data_ptr(); a.q_heads = QH; a.kv_heads = KVH; a.max_seq = max_seq; a.kv8 = kv8; a.head_dim = HD
        a.pos_arr = pos.data_ptr()
        a.kv.base0 = kvt.data_ptr(); a.kv.k_off = 0; a.kv.v_off = kvt[0].numel() * kvt.element_size()
        a.kv.sbase0 = kvst.data_ptr(); a.kv.ks_off = 0; a.kv.vs_off = kvst[0].numel() * 2
        a.part = part.data_ptr(); a.counters = ctr.data_ptr(); a.n_split_slots = n_slots; a.workers = 16
        return a
    # unfused
    q = torch.empty(1, QH * HD, dtype=torch.bfloat16, device="cuda")
    qa = QkvPostArgs()
    qa.qkv = qkv.data_ptr(); qa.q = q.data_ptr(); qa.q_norm = qn.data_ptr(); qa.k_norm = kn.data_ptr()
    qa.eps = EPS; qa.rope_base = BASE; qa.q_heads = QH; qa.kv_heads = KVH; qa.max_seq = max_seq; qa.kv8 = kv8
    qa.pos_arr = pos.data_ptr(); qa.kv = args(kvbuf, kvs, q).kv
    assert tl.qkv_post(C.byref(qa), 1, None) == 0
    o_a = torch.empty_like(q)
    a = args(kvbuf, kvs, o_a, q)
    assert tl.attn_decode(C.byref(a), 1, None) == 0
    # fused
    o_b = torch.empty_like(q)
    b = args(kv_b, kvs_b, o_b)
    assert tl.stage_attn_decode_prep(C.byref(b), p(qkv), p(qn), p(kn), EPS, BASE, 1, None) == 0
    assert_same(o_a, o_b, "fused attention output")
    assert_same(kvbuf, kv_b, "cache after append"); assert_same(kvs, kvs_b, "scales after append")


def _quantised(mine, N, K, kind, seed):
    w = rnd(N, K, scale=0.02, seed=seed)
    if kind == 0:
        q = torch.empty(N, K, dtype=torch.int8, device="cuda"); s = torch.empty(N, dtype=torch.float32, device="cuda")
        assert mine.s2p_int8_quant(p(q), p(s), p(w), N, K, None) == 0
        return q, s
    q = torch.empty(N, K, dtype=torch.int8, device="cuda"); s = torch.empty(N, K // 32, dtype=torch.float16, device="cuda")
    assert mine.s2p_intq_quant(p(q), p(s), p(w), N, K, 32, 7, 1, None) == 0
    if kind == 1:
        return q, s
    pk = torch.empty(N, K // 2, dtype=torch.uint8, device="cuda")
    assert mine.s2p_int4_pack(p(pk), p(q), N, K, None) == 0
    return pk, s


def _ref_gemv(ref, kind, y, x, w, s, N, K):
    if kind == 0:
        return ref.s2p_int8_gemv(p(y), p(x), p(w), p(s), 1, N, K, None)
    if kind == 1:
        return ref.s2p_intq_gemv(p(y), p(x), p(w), p(s), 1, N, K, 32, None)
    return ref.s2p_int4p_gemv(p(y), p(x), p(w), p(s), 1, N, K, 32, None)


@pytest.mark.parametrize("kind", [0, 1, 2])
@pytest.mark.parametrize("M", [2, 3, 5, 8, 11, 16])
def test_batched_gemv_rows_match_reference(libs, kind, M):
    """The lockstep GEMV for 2..16 rows (every row its own chain, tiles folded in order) against the
    reference's batched kernels, bitwise, on a ragged N and the model's longest K."""
    mine, _, ref = libs
    N, K = 1031, 9728
    w, s = _quantised(mine, N, K, kind, seed=21 + kind)
    x = rnd(M, K, seed=9)
    y1 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda"); y2 = torch.empty_like(y1)
    for lib, y in ((mine, y1), (ref, y2)):
        if kind == 0:
            assert lib.s2p_int8_gemv(p(y), p(x), p(w), p(s), M, N, K, None) == 0
        elif kind == 1:
            assert lib.s2p_intq_gemv(p(y), p(x), p(w), p(s), M, N, K, 32, None) == 0
        else:
            assert lib.s2p_int4p_gemv(p(y), p(x), p(w), p(s), M, N, K, 32, None) == 0
    assert_same(y1, y2, f"batched gemv kind={kind} M={M}")


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_fused_gemv_stages_equal_unfused_reference_ops(libs, kind):
    """norm->GEMV, GEMV->residual, norm->GEMV->SwiGLU and head->arg-max stages against the
    reference's separate kernels chained the way its run_layer chains them."""
    mine, tl, ref = libs
    assert tl.gemv_setup_all() == 0
    gs = 5 if kind else 0
    x = rnd(1, D, seed=70); nw = rnd(D, seed=71) + 1.0
    xn = torch.empty_like(x)
    assert ref.s2pk_rms_norm(p(x), p(nw), p(xn), 1, D, EPS, None) == 0
    # norm -> GEMV (wqkv shape)
    w, s = _quantised(mine, 6144, D, kind, 72)
    y_ref = torch.empty(1, 6144, dtype=torch.bfloat16, device="cuda"); y = torch.empty_like(y_ref)
    assert _ref_gemv(ref, kind, y_ref, xn, w, s, 6144, D) == 0
    lin = LinRef(kind, w.data_ptr(), s.data_ptr(), 6144, D, gs); vx = VecRef(x.data_ptr(), None, None)
    assert tl.stage_norm_gemv(C.byref(lin), C.byref(vx), p(nw), EPS, p(y), None) == 0
    assert_same(y, y_ref, "norm->gemv")
    # GEMV -> residual (w2 shape, K = 9728)
    h = rnd(1, F, seed=73); w2, s2 = _quantised(mine, D, F, kind, 74)
    proj = torch.empty(1, D, dtype=torch.bfloat16, device="cuda")
    assert _ref_gemv(ref, kind, proj, h, w2, s2, D, F) == 0
    r_ref = x.clone()
    assert ref.s2pk_add(p(r_ref), p(proj), D, None) == 0
    r = x.clone()
    lin2 = LinRef(kind, w2.data_ptr(), s2.data_ptr(), D, F, gs); vr = VecRef(r.data_ptr(), None, None)
    assert tl.stage_gemv_resid(C.byref(lin2), p(h), C.byref(vr), p(r), None) == 0
    assert_same(r, r_ref, "gemv->residual")
    # norm -> gate_up -> SwiGLU
    wg, sg = _quantised(mine, 2 * F, D, kind, 75)
    gu = torch.empty(1, 2 * F, dtype=torch.bfloat16, device="cuda")
    assert _ref_gemv(ref, kind, gu, xn, wg, sg, 2 * F, D) == 0
    hh_ref = torch.empty(1, F, dtype=torch.bfloat16, device="cuda"); hh = torch.empty_like(hh_ref)
    assert ref.s2pk_silu_mul(p(gu), p(hh_ref), 1, F, None) == 0
    lin3 = LinRef(kind, wg.data_ptr(), sg.data_ptr(), 2 * F, D, gs)
    assert tl.stage_norm_swiglu(C.byref(lin3), C.byref(vx), p(nw), EPS, p(hh), None) == 0
    assert_same(hh, hh_ref, "norm->gemv->swiglu")
    # norm -> head -> arg-max, with the input row picked by a device index
    table = rnd(16, D, seed=76); idx = torch.tensor([11], dtype=torch.int32, device="cuda")
    wh, sh = _quantised(mine, 4096, D, kind, 77)
    tn = torch.empty(1, D, dtype=torch.bfloat16, device="cuda")
    assert ref.s2pk_rms_norm(p(table[11:12].contiguous()), p(nw), p(tn), 1, D, EPS, None) == 0
    lg_ref = torch.empty(1, 4096, dtype=torch.bfloat16, device="cuda"); lg = torch.empty_like(lg_ref)
    assert _ref_gemv(ref, kind, lg_ref, tn, wh, sh, 4096, D) == 0
    am_ref = torch.empty(1, dtype=torch.int32, device="cuda")
    assert ref.s2pk_argmax(p(lg_ref), p(am_ref), 1, 4096, None) == 0
    key = torch.zeros(1, dtype=torch.int64, device="cuda")
    lin4 = LinRef(kind, wh.data_ptr(), sh.data_ptr(), 4096, D, gs)
    assert tl.stage_norm_argmax(C.byref(lin4), p(table[11:12].contiguous()), p(nw), EPS, p(lg), p(key), None) == 0
    assert_same(lg, lg_ref, "head logits")
    torch.cuda.synchronize()
    assert 0xFFFFFFFF - (int(key[0]) & 0xFFFFFFFF) == int(am_ref[0])
    # the same stage reading its input through the index
    y2 = torch.empty(1, 6144, dtype=torch.bfloat16, device="cuda"); y2_ref = torch.empty_like(y2)
    vx_i = VecRef(table.data_ptr(), idx.data_ptr(), None)
    assert tl.stage_norm_gemv(C.byref(lin), C.byref(vx_i), p(nw), EPS, p(y2), None) == 0
    assert _ref_gemv(ref, kind, y2_ref, tn, w, s, 6144, D) == 0
    assert_same(y2, y2_ref, "norm->gemv via device index")


@pytest.mark.parametrize("temp,seed", [(0.0, 0), (0.8, 42), (0.8, 0), (1e-7, 5)])
def test_sampler_matches_reference_device_sampler(libs, temp, seed):
    _, tl, ref = libs
    rows = 3
    for step in range(6):
        lg = rnd(rows, 4096, scale=2.0, seed=80 + step); eos = rnd(rows, 1, scale=2.0, seed=90 + step)
        if step == 0:
            states = []
            for r in range(rows):
                st = SamplerState(); st.temperature = temp; st.top_p = 0.8; st.rep_penalty = 1.1; st.window = 16
                st.seeded = 1 if seed else 0; st.seed31 = seed & 0x7FFFFFFF
                for i in range(4): st.rng[i] = 0x9E3779B97F4A7C15 * (i + 1 + r) & 0xFFFFFFFFFFFFFFFF
                states.append(st)
            buf = b"".join(bytes(s) for s in states)
            d1 = torch.frombuffer(bytearray(buf), dtype=torch.uint8).cuda(); d2 = d1.clone()
            sz = C.sizeof(SamplerState)
            p1 = torch.tensor([d1.data_ptr() + sz * r for r in range(rows)], dtype=torch.int64, device="cuda")
            p2 = torch.tensor([d2.data_ptr() + sz * r for r in range(rows)], dtype=torch.int64, device="cuda")
        outs = []
        for which, ptrs in (("mine", p1), ("ref", p2)):
            tok = torch.zeros(rows, dtype=torch.int64, device="cuda"); sem = torch.zeros(rows, dtype=torch.int32, device="cuda")
            codes = torch.zeros(rows * 10, dtype=torch.int32, device="cuda"); e = torch.zeros(rows, dtype=torch.uint8, device="cuda")
            if which == "mine":
                assert tl.sample_rows(p(lg), 4096, p(eos), 1, p(ptrs), rows, p(tok), p(sem), p(codes), p(e), None) == 0
            else:
                assert ref.s2pk_sample(p(lg), 4096, p(eos), p(ptrs), rows, p(tok), p(sem), p(codes), p(e), None) == 0
            outs.append((tok, sem, codes, e))
        for a_, b_, nm in zip(outs[0], outs[1], ("tok", "sem", "codes", "eos")):
            assert_same(a_, b_, f"sampler {nm} step {step}")
        assert_same(d1, d2, f"sampler state step {step}")


def test_linear_forward_prefill_path_matches_reference(libs, capi):
    """M > 16: dequantise + library GEMM with the reference's GemmEx arguments."""
    mine, _, ref = libs
    assert mine.s2p_gemm_init(256) == 0 and ref.s2p_gemm_init(256) == 0
    N, K, M = 6144, D, 64
    for kind in (0, 2):
        w, s = _quantised(mine, N, K, kind, 100 + kind)
        lin = capi.Linear(); lin.in_features = K; lin.out_features = N; lin.int8_ready = 1
        if kind == 0:
            lin.w_int8.data = w.data_ptr(); lin.w_iscale.data = s.data_ptr()
        else:
            lin.w_pack.data = w.data_ptr(); lin.w_iscale.data = s.data_ptr(); lin.q_group = 32; lin.q_packed = 1
        x = rnd(M, K, seed=110)
        y1 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda"); y2 = torch.empty_like(y1)
        assert mine.s2p_linear_forward(C.byref(lin), p(x), p(y1), M, capi.GEMM_INT8, None) == 0
        assert ref.s2p_linear_forward(C.byref(lin), p(x), p(y2), M, capi.GEMM_INT8, None) == 0
        assert_same(y1, y2, f"linear_forward M={M} kind={kind}")


def test_tick_begin_matches_reference_glue(libs):
    """embed (INT8 sidecar) + VQ sum + masked 1/sqrt(11) scale, against the oracle-free
    composition of the library's own unfused kernels (each pinned against the reference)."""
    mine, tl, ref = libs
    V = 300
    tab = rnd(V, D, scale=0.02, seed=120)
    q = torch.empty(V, D, dtype=torch.int8, device="cuda"); sc = torch.empty(V, dtype=torch.float32, device="cuda")
    assert mine.s2p_int8_quant(p(q), p(sc), p(tab), V, D, None) == 0
    cb = rnd(10 * 4096, D, scale=0.02, seed=121)
    rows = 3
    ids = torch.tensor([5, 299, 17], dtype=torch.int64, device="cuda")
    codes = torch.randint(0, 4096, (rows, 10), dtype=torch.int32, device="cuda")
    mask = torch.tensor([1, 0, 1], dtype=torch.uint8, device="cuda")
    # reference-order composition
    x_ref = torch.empty(rows, D, dtype=torch.bfloat16, device="cuda")
    assert ref.s2pk_embed_i8(p(q), p(sc), p(ids), p(x_ref), rows, D, None) == 0
    for r in range(rows):
        if int(mask[r]):
            cm = codes[r].contiguous()  # [10] cb-major with T = 1
            assert tl.vq_embed_add(p(cb), p(cm), 1, C.c_void_p(x_ref[r].data_ptr()), None) == 0
    inv = float(np.float32(1.0 / 3.3166247903554))
    assert ref.s2pk_scale_rows_masked(p(x_ref), p(mask), rows, D, inv, None) == 0
    x = torch.empty_like(x_ref); keys = torch.ones(rows * 9, dtype=torch.int64, device="cuda")
    a = TickBeginArgs(None, q.data_ptr(), sc.data_ptr(), cb.data_ptr(), ids.data_ptr(), codes.data_ptr(), mask.data_ptr(),
                      x.data_ptr(), keys.data_ptr())
    assert tl.tick_begin(C.byref(a), rows, None) == 0
    assert_same(x, x_ref, "tick_begin rows")
    assert int(keys.abs().sum()) == 0


# the shapes of the decode tick's linears (N x K): wqkv, wo, gate_up, w2, the fast head, the tied-head slice, the EOS row
MODEL_SHAPES = [(6144, 2560), (2560, 4096), (19456, 2560), (2560, 9728), (4096, 2560), (4097, 2560), (1, 2560)]


@pytest.mark.parametrize("N,K", MODEL_SHAPES)
def test_quantisers_pack_and_dequant_equal_reference(libs, N, K):
    """Load-time conversion, bit for bit: per-channel INT8, g32 INT4 with and without the MSE clip search,
    nibble packing, and the three dequantisers, against the reference's own kernels."""
    mine, _, ref = libs
    w = rnd(N, K, scale=0.02, seed=900 + N % 97)
    w[0, : min(K, 64)] = 0  # an all-zero group (and, for N == 1, a partly zero row)
    # per-channel INT8
    q1 = torch.empty(N, K, dtype=torch.int8, device="cuda"); q2 = torch.empty_like(q1)
    s1 = torch.empty(N, dtype=torch.float32, device="cuda"); s2 = torch.empty_like(s1)
    assert mine.s2p_int8_quant(p(q1), p(s1), p(w), N, K, None) == 0
    assert ref.s2p_int8_quant(p(q2), p(s2), p(w), N, K, None) == 0
    assert_same(q1, q2, "int8 codes"); assert_same(s1, s2, "int8 row scales")
    d1 = torch.empty(N, K, dtype=torch.bfloat16, device="cuda"); d2 = torch.empty_like(d1)
    assert mine.s2p_int8_dequant(p(d1), p(q1), p(s1), N, K, None) == 0
    assert ref.s2p_int8_dequant(p(d2), p(q2), p(s2), N, K, None) == 0
    assert_same(d1, d2, "int8 dequant")
    # g32 INT4, plain absmax and MSE clip search
    for mse in (0, 1):
        g1 = torch.empty(N, K, dtype=torch.int8, device="cuda"); g2 = torch.empty_like(g1)
        h1 = torch.empty(N, K // 32, dtype=torch.float16, device="cuda"); h2 = torch.empty_like(h1)
        assert mine.s2p_intq_quant(p(g1), p(h1), p(w), N, K, 32, 7, mse, None) == 0
        assert ref.s2p_intq_quant(p(g2), p(h2), p(w), N, K, 32, 7, mse, None) == 0
        assert_same(g1, g2, f"int4 codes mse={mse}"); assert_same(h1, h2, f"int4 group scales mse={mse}")
    assert mine.s2p_intq_dequant(p(d1), p(g1), p(h1), N, K, 32, None) == 0
    assert ref.s2p_intq_dequant(p(d2), p(g2), p(h2), N, K, 32, None) == 0
    assert_same(d1, d2, "int4 container dequant")
    k1 = torch.empty(N, K // 2, dtype=torch.uint8, device="cuda"); k2 = torch.empty_like(k1)
    assert mine.s2p_int4_pack(p(k1), p(g1), N, K, None) == 0
    assert ref.s2p_int4_pack(p(k2), p(g2), N, K, None) == 0
    assert_same(k1, k2, "packed nibbles")
    assert mine.s2p_int4p_dequant(p(d1), p(k1), p(h1), N, K, 32, None) == 0
    assert ref.s2p_int4p_dequant(p(d2), p(k2), p(h2), N, K, 32, None) == 0
    assert_same(d1, d2, "packed int4 dequant")
