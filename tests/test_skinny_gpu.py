"""The tensor-core batched decode linear (tcgen05, more than 16 rows) against the exact-order
GEMV of this library, which is bit-identical to the reference's.  The two accumulate in
different orders (and INT4 rounds code x scale to f16 once), so this is a tolerance check:
bf16 outputs may differ by a rounding step, not more."""
import ctypes as C

import pytest

from _internal_abi import LinRef
from test_kernels_gpu import _quantised, dev, p, rnd

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def exact(mine, kind, y, x, w, s, M, N, K):
    for m0 in range(0, M, 16):
        mm = min(16, M - m0)
        ys, xs = y[m0:m0 + mm], x[m0:m0 + mm]
        if kind == 0:
            rc = mine.s2p_int8_gemv(p(ys), p(xs), p(w), p(s), mm, N, K, None)
        elif kind == 1:
            rc = mine.s2p_intq_gemv(p(ys), p(xs), p(w), p(s), mm, N, K, 32, None)
        else:
            rc = mine.s2p_int4p_gemv(p(ys), p(xs), p(w), p(s), mm, N, K, 32, None)
        assert rc == 0


@pytest.mark.parametrize("kind", [2, 0, 1])
@pytest.mark.parametrize("M,N,K", [(32, 6144, 2560), (32, 19456, 2560), (17, 2560, 4096), (128, 2560, 9728), (48, 4097, 2560), (256, 384, 512)])
def test_tensor_core_linear_matches_exact_gemv(mine, testlib, kind, M, N, K):
    dev()
    testlib.skinny_gemm_tc.argtypes = [C.POINTER(LinRef), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    testlib.skinny_status.argtypes = [C.POINTER(C.c_int)]
    w, s = _quantised(mine, N, K, kind, seed=11 + kind)
    x = rnd(M, K, seed=5)
    y_exact = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    y_tc = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    exact(mine, kind, y_exact, x, w, s, M, N, K)
    lin = LinRef(kind, w.data_ptr(), s.data_ptr(), N, K, 0 if kind == 0 else 5)
    testlib.skinny_setup.argtypes = [C.c_int]
    a0 = None
    for with_split_scratch in (False, True):  # single pass over K, then K split over several CTAs where rows are few
        if with_split_scratch:
            assert testlib.skinny_setup(256) == 0
        y_tc.fill_(float("nan"))
        assert testlib.skinny_gemm_tc(C.byref(lin), p(x), M, p(y_tc), None, None) == 0
        torch.cuda.synchronize()
        st = C.c_int(-1)
        assert testlib.skinny_status(C.byref(st)) == 0 and st.value == 0, "a bounded wait inside the kernel gave up"
        a, b = y_tc.float(), y_exact.float()
        assert torch.isfinite(a).all()
        scale = float(b.abs().max())
        diff = (a - b).abs()
        mag = torch.maximum(a.abs(), b.abs()).clamp_min(2.0 ** -20)
        step = torch.exp2(torch.floor(torch.log2(mag)) - 7)  # one bf16 step at that magnitude
        # one rounding step of the output, plus the accumulated f16 rounding of code x scale (INT4 / grouped INT8)
        assert bool((diff <= step + 2e-3 * scale).all()), f"max diff {float(diff.max())} at scale {scale}"
        assert float((diff == 0).float().mean()) >= 0.8, "most outputs should round to the same bf16"
        cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0)
        assert float(cos) >= 0.99999
        # the same launch again gives the same bits (the split partials are added in a fixed order)
        y2 = torch.empty_like(y_tc)
        assert testlib.skinny_gemm_tc(C.byref(lin), p(x), M, p(y2), None, None) == 0
        torch.cuda.synchronize()
        assert torch.equal(y2.view(torch.int16), y_tc.view(torch.int16))
        # fused residual add, in place: y = bf16(f32(r) + f32(bf16(product)))
        r = rnd(M, N, seed=77)
        y3 = r.clone()
        assert testlib.skinny_gemm_tc(C.byref(lin), p(x), M, p(y3), p(y3), None) == 0
        torch.cuda.synchronize()
        want = (r.float() + y_tc.float()).to(torch.bfloat16)
        assert torch.equal(y3.view(torch.int16), want.view(torch.int16))
        a0 = a


@pytest.mark.parametrize("kind", [2, 0, 1])
@pytest.mark.parametrize("M,ffn,K", [(32, 6400, 512), (17, 4810, 512), (200, 6400, 512), (32, 9728, 2560), (17, 200, 512)])
def test_fused_swiglu_equals_linear_then_swiglu(mine, testlib, kind, M, ffn, K):
    """The gate/up linear with SwiGLU in its epilogue against the same linear followed by the SwiGLU kernel.
    76..148 row tiles (no tile is split over K in either launch, both accumulate every row in one pass): the same
    bits, also with a ragged last tile and more than 128 rows.  Shapes whose tiles are split (the two launches
    split different rows, so f32 partial sums are added in different orders): a rounding step of difference."""
    dev()
    N = 2 * ffn
    testlib.skinny_gemm_tc.argtypes = [C.POINTER(LinRef), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    testlib.skinny_gemm_tc_swiglu.argtypes = [C.POINTER(LinRef), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    testlib.silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    testlib.skinny_status.argtypes = [C.POINTER(C.c_int)]
    testlib.skinny_setup.argtypes = [C.c_int]
    assert testlib.skinny_setup(256) == 0
    w, s = _quantised(mine, N, K, kind, seed=31 + kind)
    x = rnd(M, K, seed=6)
    lin = LinRef(kind, w.data_ptr(), s.data_ptr(), N, K, 0 if kind == 0 else 5)
    gu = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    want = torch.empty(M, ffn, dtype=torch.bfloat16, device="cuda")
    got = torch.full((M, ffn), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert testlib.skinny_gemm_tc(C.byref(lin), p(x), M, p(gu), None, None) == 0
    assert testlib.silu_mul(p(gu), p(want), M, ffn, None) == 0
    assert testlib.skinny_gemm_tc_swiglu(C.byref(lin), p(x), M, p(got), None) == 0
    torch.cuda.synchronize()
    st = C.c_int(-1)
    assert testlib.skinny_status(C.byref(st)) == 0 and st.value == 0, "a bounded wait inside the kernel gave up"
    assert torch.isfinite(got.float()).all()
    tiles = (ffn + 63) // 64
    if 75 <= tiles <= 148:
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    else:
        a, b = got.float(), want.float()
        diff = (a - b).abs()
        scale = float(b.abs().max())
        mag = torch.maximum(a.abs(), b.abs()).clamp_min(2.0 ** -20)
        step = torch.exp2(torch.floor(torch.log2(mag)) - 7)  # one bf16 step at that magnitude
        assert bool((diff <= 2 * step + 2e-3 * scale).all()), f"max diff {float(diff.max())} at scale {scale}"
        assert float((diff == 0).float().mean()) >= 0.9
        # the fused launch is reproducible run to run
        got2 = torch.empty_like(got)
        assert testlib.skinny_gemm_tc_swiglu(C.byref(lin), p(x), M, p(got2), None) == 0
        torch.cuda.synchronize()
        assert torch.equal(got2.view(torch.int16), got.view(torch.int16))


@pytest.mark.parametrize("kind", [2, 0, 1])
@pytest.mark.parametrize("M,N,K", [(300, 6144, 2560), (512, 2560, 4096), (1000, 19456, 2560), (40, 4097, 2560), (257, 2560, 9728), (2048, 384, 512),
                                   (1024, 2560, 4096), (1300, 6144, 2560)])
def test_prompt_sized_linear_matches_exact_gemv(mine, testlib, kind, M, N, K):
    """The prefill form of the tensor-core linear: any number of rows in blocks of 256, activations
    pre-tiled in f16 and brought in by bulk copies, a weight slab converted once per block; from 1024 rows on a CTA
    of the packed-INT4 kind takes two blocks (two accumulators side by side in TMEM), ragged last pair included."""
    dev()
    testlib.skinny_prefill_tc.argtypes = [C.POINTER(LinRef), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    testlib.skinny_status.argtypes = [C.POINTER(C.c_int)]
    testlib.skinny_setup.argtypes = [C.c_int]
    w, s = _quantised(mine, N, K, kind, seed=21 + kind)
    x = rnd(M, K, seed=6)
    y_exact = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    exact(mine, kind, y_exact, x, w, s, M, N, K)
    lin = LinRef(kind, w.data_ptr(), s.data_ptr(), N, K, 0 if kind == 0 else 5)
    assert testlib.skinny_setup(256) == 0  # split-K scratch: short prompts on matrices of few rows use it
    y = torch.full((M + 1, N), float("nan"), dtype=torch.bfloat16, device="cuda")  # one guard row behind the output
    assert testlib.skinny_prefill_tc(C.byref(lin), p(x), M, p(y), None) == 0
    torch.cuda.synchronize()
    st = C.c_int(-1)
    assert testlib.skinny_status(C.byref(st)) == 0 and st.value == 0, "a bounded wait inside the kernel gave up"
    assert bool(torch.isnan(y[M].float()).all()), "wrote behind the last row"
    a, b = y[:M].float(), y_exact.float()
    assert torch.isfinite(a).all()
    scale = float(b.abs().max())
    diff = (a - b).abs()
    mag = torch.maximum(a.abs(), b.abs()).clamp_min(2.0 ** -20)
    step = torch.exp2(torch.floor(torch.log2(mag)) - 7)
    assert bool((diff <= step + 2e-3 * scale).all()), f"max diff {float(diff.max())} at scale {scale}"
    assert float((diff == 0).float().mean()) >= 0.8
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0)
    assert float(cos) >= 0.99999
    y2 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    assert testlib.skinny_prefill_tc(C.byref(lin), p(x), M, p(y2), None) == 0
    torch.cuda.synchronize()
    assert torch.equal(y2.view(torch.int16), y[:M].view(torch.int16)), "not reproducible run to run"
