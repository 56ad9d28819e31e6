"""ctypes access to oracle/libs2p_oracle.so (TEST INFRASTRUCTURE — the checker,
never the product path) with numpy-friendly helpers."""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libs2p_oracle.so")

_P = C.c_void_p
_I = C.c_int


def build():
    subprocess.check_call(["make", "-C", HERE, "oracle"], stdout=subprocess.DEVNULL)


def load():
    if not os.path.exists(LIB):
        build()
    lib = C.CDLL(LIB)
    lib.s2po_bf2f.restype = C.c_float; lib.s2po_bf2f.argtypes = [C.c_uint16]
    lib.s2po_f2bf.restype = C.c_uint16; lib.s2po_f2bf.argtypes = [C.c_float]
    lib.s2po_h2f.restype = C.c_float; lib.s2po_h2f.argtypes = [C.c_uint16]
    lib.s2po_f2h.restype = C.c_uint16; lib.s2po_f2h.argtypes = [C.c_float]
    lib.s2po_quant_int8.argtypes = [_P, _P, _P, _I, _I]
    lib.s2po_quant_g.argtypes = [_P, _P, _P, _I, _I, _I, _I, _I]
    lib.s2po_pack.argtypes = [_P, _P, C.c_size_t]
    lib.s2po_unpack.argtypes = [_P, _P, C.c_size_t]
    lib.s2po_dequant_int8.argtypes = [_P, _P, _P, _I, _I]
    lib.s2po_dequant_g.argtypes = [_P, _P, _P, _I, _I, _I]
    lib.s2po_dequant_p.argtypes = [_P, _P, _P, _I, _I, _I]
    lib.s2po_gemv_int8.argtypes = [_P, _P, _P, _P, _I, _I, _I]
    lib.s2po_gemv_g.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I]
    lib.s2po_gemv_p.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I]
    lib.s2po_rms_norm.argtypes = [_P, _P, _P, _I, _I, C.c_float, _I]
    lib.s2po_rope.argtypes = [_P, _I, _I, _I, _P, C.c_float]
    lib.s2po_kv8_quant.argtypes = [_P, _P, _P, _I]
    lib.s2po_silu_mul.argtypes = [_P, _P, _I, _I]
    lib.s2po_add.argtypes = [_P, _P, C.c_int64]
    lib.s2po_embed_i8.argtypes = [_P, _P, _P, _P, _I, _I]
    lib.s2po_vq_embed_add.argtypes = [_P, _P, _I, _P, _I, _I, _I]
    lib.s2po_argmax.argtypes = [_P, _P, _I, _I]
    lib.s2po_attn_decode_bf16.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I]
    lib.s2po_attn_decode_kv8.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I]
    lib.s2po_attn_single.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I]
    lib.s2po_sampler_size.restype = C.c_size_t
    lib.s2po_sampler_init.argtypes = [_P, C.c_float, C.c_float, C.c_float, _I, C.c_uint64, C.c_uint64]
    lib.s2po_sample.restype = C.c_int64
    lib.s2po_sample.argtypes = [_P, _P, C.c_uint16, _I, C.c_int64, C.c_int64, _P, _P]
    lib.s2po_model_new.restype = _P
    lib.s2po_model_new.argtypes = [_I] * 9 + [C.c_int64, C.c_int64] + [_I] * 6
    lib.s2po_model_set_layer.argtypes = [_P, _I, _I, _I, _P]
    lib.s2po_model_set_global.argtypes = [_P, _I, _P]
    lib.s2po_model_free.argtypes = [_P]
    lib.s2po_session_new.restype = _P
    lib.s2po_session_new.argtypes = [_P, C.c_float, C.c_float, C.c_float, _I, C.c_uint64]
    lib.s2po_session_free.argtypes = [_P]
    lib.s2po_prefill.argtypes = [_P, _P, _I, _P]
    lib.s2po_next_frame.argtypes = [_P, _P, _P, _P]
    lib.s2po_fast_frame.argtypes = [_P, _P, _I, _P, _P]
    lib.s2po_layer_gemv_sample.argtypes = [_P, _P, _P, _P, _P, _I, _I]
    lib.s2po_set_threads.restype = _I; lib.s2po_set_threads.argtypes = [_I]
    lib.s2po_model_fill_synthetic.argtypes = [_P, C.c_uint64]
    return lib


def ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def f32_to_bf16(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)
