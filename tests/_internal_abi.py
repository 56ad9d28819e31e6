"""ctypes mirrors of the internal launch structs (s2pro-native_b200/csrc/cuda/ops.h)
and of the reference's private launchers, for kernel-level parity tests."""
import ctypes as C

_P, _I, _F = C.c_void_p, C.c_int, C.c_float


class KvRef(C.Structure):
    _fields_ = [("base0", _P), ("bases", _P), ("row_stride", C.c_size_t), ("k_off", C.c_size_t), ("v_off", C.c_size_t),
                ("sbase0", _P), ("sbases", _P), ("srow_stride", C.c_size_t), ("ks_off", C.c_size_t), ("vs_off", C.c_size_t)]


class QkvPostArgs(C.Structure):
    _fields_ = [("qkv", _P), ("q", _P), ("q_norm", _P), ("k_norm", _P), ("eps", _F), ("rope_base", _F),
                ("q_heads", _I), ("kv_heads", _I), ("max_seq", _I), ("kv8", _I), ("pos0", _I), ("pos_row_step", _I),
                ("pos_arr", _P), ("kv", KvRef)]


class AttnArgs(C.Structure):
    _fields_ = [("q", _P), ("out", _P), ("q_heads", _I), ("kv_heads", _I), ("max_seq", _I), ("kv8", _I),
                ("pos0", _I), ("pos_row_step", _I), ("pos_arr", _P), ("kv", KvRef), ("part", _P), ("counters", _P),
                ("n_split_slots", _I), ("workers", _I), ("n_out_peers", _I), ("out_peer_delta", _P), ("out_ll", _I), ("out_ll_tag", C.c_uint), ("head_dim", _I)]


class SamplerState(C.Structure):
    _fields_ = [("prev", C.c_int64 * 64), ("count", C.c_uint64), ("rng", C.c_uint64 * 4), ("temperature", _F),
                ("top_p", _F), ("rep_penalty", _F), ("window", C.c_int32), ("seeded", C.c_int32),
                ("seed31", C.c_uint32), ("pad_", C.c_uint32)]


class LinRef(C.Structure):
    _fields_ = [("kind", _I), ("w", _P), ("scales", _P), ("N", _I), ("K", _I), ("gshift", _I)]


class VecRef(C.Structure):
    _fields_ = [("base", _P), ("index", _P), ("key", _P)]


class TickBeginArgs(C.Structure):
    _fields_ = [("embed", _P), ("embed_i8", _P), ("embed_scale", _P), ("cb_emb", _P), ("ids", _P), ("codes", _P),
                ("mask", _P), ("x", _P), ("keys", _P)]


def bind_internal(lib):
    lib.qkv_post.argtypes = [C.POINTER(QkvPostArgs), _I, _P]
    lib.attn_single.argtypes = [C.POINTER(AttnArgs), _I, _P]
    lib.attn_decode.argtypes = [C.POINTER(AttnArgs), _I, _P]
    lib.stage_attn_decode_prep.argtypes = [C.POINTER(AttnArgs), _P, _P, _P, _F, _F, _I, _P]
    lib.sample_rows.argtypes = [_P, C.c_int64, _P, C.c_int64, _P, _I, _P, _P, _P, _P, _P]
    lib.stage_norm_gemv.argtypes = [C.POINTER(LinRef), C.POINTER(VecRef), _P, _F, _P, _P]
    lib.stage_gemv_resid.argtypes = [C.POINTER(LinRef), _P, C.POINTER(VecRef), _P, _P]
    lib.stage_norm_swiglu.argtypes = [C.POINTER(LinRef), C.POINTER(VecRef), _P, _F, _P, _P]
    lib.stage_norm_argmax.argtypes = [C.POINTER(LinRef), _P, _P, _F, _P, _P, _P]
    lib.tick_begin.argtypes = [C.POINTER(TickBeginArgs), _I, _P]
    lib.tick_finish_keys.argtypes = [_P, _I, _P, _P]
    lib.gemv_setup_all.argtypes = []
    lib.vq_embed_add.argtypes = [_P, _P, _I, _P, _P]
    lib.scale_div.argtypes = [_P, C.c_int64, _F, _P]
    lib.scale_rows_masked.argtypes = [_P, _P, _I, _I, _F, _P]
    lib.embed_rows_i8.argtypes = [_P, _P, _P, _P, _I, _I, _P]
    return lib


def bind_ref_private(ref):
    """Private launchers the rebuilt reference library happens to export
    (src/slowar/slowar_kernels.h of the reference)."""
    ref.s2pk_qkv_split.argtypes = [_P, _P, _P, _P, _I, _I, _I, _P]
    ref.s2pk_rope_pos.argtypes = [_P, _P, _I, _I, _I, _I, _P, _F, _P]
    ref.s2pk_kv_append_ptrs.argtypes = [_P, _P, _P, _P, _I, _I, _I, _P, _I, _P]
    ref.s2pk_kv_append8.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]
    ref.s2pk_kv_append8_ptrs.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _I, _I, _P]
    ref.s2pk_attention_ptrs.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _P]
    ref.s2pk_attention8.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P]
    ref.s2pk_attention_decode.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _P, _P]
    ref.s2pk_attention8_decode.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _P, _I, _P]
    ref.s2pk_embed_i8.argtypes = [_P, _P, _P, _P, _I, _I, _P]
    ref.s2pk_sample.argtypes = [_P, C.c_int64, _P, _P, _I, _P, _P, _P, _P, _P]
    ref.s2pk_scale_div.argtypes = [_P, C.c_int64, _F, _P]
    ref.s2pk_scale_rows_masked.argtypes = [_P, _P, _I, _I, _F, _P]
    return ref
