"""The allocation-free decode attention (s2p_b200_attention_decode_noalloc).

Hosts that must not allocate device memory while running — a real-time worker that
cannot afford the device-wide serialisation of cudaMalloc/cudaFree, or a plug-in that
is given no memory pool — call this entry point instead of the regular split-K
attention, whose scratch is allocated at model load.  The test calls it through the
C ABI twice in a row (the built-in scratch keeps the first call's contents) and checks
each result against the existing attention entry points on the same inputs.

Collected last on purpose: a failure here cannot hide the rest of a `-x` run."""
import ctypes as C

import pytest

from _internal_abi import AttnArgs, bind_internal

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

QH, KVH, HD = 32, 8, 128


def p(t):
    return C.c_void_p(t.data_ptr())


def rnd(*shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, device="cuda", generator=g).to(torch.bfloat16)


def test_noalloc_attention_twice_in_a_row(mine, testlib):
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    tl = bind_internal(testlib)
    max_seq = 1024
    for call, (pos, seed) in enumerate(((700, 11), (129, 12))):  # second call: shorter context, stale partials behind it
        k = rnd(KVH, max_seq, HD, seed=seed); v = rnd(KVH, max_seq, HD, seed=seed + 100)
        kv = torch.stack([k, v]).contiguous()  # planes of one allocation, as the regular path lays them out
        q = rnd(1, QH * HD, seed=seed + 200)
        out = torch.zeros_like(q)
        rc = mine.s2p_b200_attention_decode_noalloc(p(q), p(kv[0]), p(kv[1]), p(out), QH, KVH, HD, pos, max_seq, None)
        assert rc == 0, rc
        torch.cuda.synchronize()
        # (1) the library's regular split-K decode attention, scratch allocated by the caller: bit-identical
        n_slots = (max_seq + 63) // 64
        part = torch.empty(QH * n_slots * 130, dtype=torch.float32, device="cuda")
        ctr = torch.zeros(KVH, dtype=torch.int32, device="cuda")
        ref_out = torch.zeros_like(q)
        a = AttnArgs()
        a.q = q.data_ptr(); a.out = ref_out.data_ptr(); a.q_heads = QH; a.kv_heads = KVH; a.max_seq = max_seq; a.kv8 = 0
        a.head_dim = HD; a.pos0 = pos; a.pos_row_step = 0
        a.kv.base0 = kv.data_ptr(); a.kv.k_off = 0; a.kv.v_off = kv[0].numel() * 2
        a.part = part.data_ptr(); a.counters = ctr.data_ptr(); a.n_split_slots = n_slots; a.workers = 16
        assert tl.attn_decode(C.byref(a), 1, None) == 0
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), ref_out.view(torch.int16)), f"call {call}: differs from the regular split-K path"
        # (2) the exported single-pass attention (different summation order): bf16 tolerance of the parity tests
        sp_out = torch.zeros_like(q)
        assert mine.s2pk_attention(p(q), p(kv[0]), p(kv[1]), p(sp_out), 1, QH, KVH, HD, pos, max_seq, None) == 0
        torch.cuda.synchronize()
        diff = (out.float() - sp_out.float()).abs().max().item()
        cos = torch.nn.functional.cosine_similarity(out.float().flatten(), sp_out.float().flatten(), dim=0).item()
        assert diff <= 2e-2 and cos >= 0.9999, (call, diff, cos)


def _regular(tl, q, k, v, pos, max_seq):
    """The library's regular split-K decode attention with caller-allocated scratch, K and V as two bases."""
    n_slots = (max_seq + 63) // 64
    part = torch.empty(QH * n_slots * 130, dtype=torch.float32, device="cuda")
    ctr = torch.zeros(KVH, dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    lo = min(k.data_ptr(), v.data_ptr())
    a = AttnArgs()
    a.q = q.data_ptr(); a.out = out.data_ptr(); a.q_heads = QH; a.kv_heads = KVH; a.max_seq = max_seq; a.kv8 = 0
    a.head_dim = HD; a.pos0 = pos; a.pos_row_step = 0
    a.kv.base0 = lo; a.kv.k_off = k.data_ptr() - lo; a.kv.v_off = v.data_ptr() - lo
    a.part = part.data_ptr(); a.counters = ctr.data_ptr(); a.n_split_slots = n_slots; a.workers = 16
    assert tl.attn_decode(C.byref(a), 1, None) == 0
    torch.cuda.synchronize()
    return out


def test_noalloc_attention_separate_allocations_either_order(mine, testlib):
    """K and V are two independent pointers of the entry point: separate allocations, V above K and V below K."""
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    tl = bind_internal(testlib)
    max_seq, pos = 512, 300
    a = rnd(KVH, max_seq, HD, seed=31); b = rnd(KVH, max_seq, HD, seed=32)
    q = rnd(1, QH * HD, seed=33)
    for k, v in ((a, b), (b, a)):  # one of the two orders has the value plane at the lower address
        out = torch.zeros_like(q)
        assert mine.s2p_b200_attention_decode_noalloc(p(q), p(k), p(v), p(out), QH, KVH, HD, pos, max_seq, None) == 0
        torch.cuda.synchronize()
        want = _regular(tl, q, k, v, pos, max_seq)
        assert torch.equal(out.view(torch.int16), want.view(torch.int16)), ("V below K" if v.data_ptr() < k.data_ptr() else "V above K")


def test_noalloc_attention_at_the_size_limit(mine, testlib):
    """The largest accepted call (8192 cached positions: the top split slot sits directly below the arrival
    counters in the built-in array), then a short call that would see counters left non-zero."""
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    tl = bind_internal(testlib)
    max_seq = 8192
    k = rnd(KVH, max_seq, HD, seed=41); v = rnd(KVH, max_seq, HD, seed=42)
    q = rnd(1, QH * HD, seed=43)
    for pos in (8191, 70):
        out = torch.zeros_like(q)
        assert mine.s2p_b200_attention_decode_noalloc(p(q), p(k), p(v), p(out), QH, KVH, HD, pos, max_seq, None) == 0
        torch.cuda.synchronize()
        want = _regular(tl, q, k, v, pos, max_seq)
        assert torch.equal(out.view(torch.int16), want.view(torch.int16)), f"pos {pos}"


def test_noalloc_attention_rejects_oversize(mine):
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    q = rnd(1, QH * HD, seed=1); out = torch.zeros_like(q); kv = rnd(2, KVH, 16, HD, seed=2)
    assert mine.s2p_b200_attention_decode_noalloc(p(q), p(kv[0]), p(kv[1]), p(out), QH, KVH, HD, 8192, 16384, None) == -1
    assert mine.s2p_b200_attention_decode_noalloc(p(q), p(kv[0]), p(kv[1]), p(out), QH, KVH, HD, 16, 16, None) == -1
    assert mine.s2p_b200_attention_decode_noalloc(p(q), p(kv[0]), p(kv[1]), p(out), 16, KVH, HD, 3, 16, None) == -1
    assert mine.s2p_b200_attention_decode_noalloc(None, p(kv[0]), p(kv[1]), p(out), QH, KVH, HD, 3, 16, None) == -1
