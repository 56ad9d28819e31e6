"""ctypes declarations for libs2pro_b200.so (see include/s2p_b200_abi.h)."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libs2pro_b200.so")

GEMM_BF16, GEMM_FP8, GEMM_INT8 = 0, 1, 2
STATUS_NAMES = {0: "OK", -1: "INVALID", -2: "CUDA", -3: "IO", -4: "OOM", -5: "FORMAT", -6: "STATE",
                -7: "UNSUPPORTED", -8: "INTERNAL", -9: "FULL"}


class S2PError(RuntimeError):
    def __init__(self, status, what=""):
        self.status = status
        super().__init__(f"{what}: s2p_status {status} ({STATUS_NAMES.get(status, '?')})")


def check(status, what=""):
    if status != 0:
        raise S2PError(status, what)


class Tensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int), ("ndim", C.c_int), ("shape", C.c_int64 * 4),
                ("bytes", C.c_size_t), ("on_device", C.c_int)]


class Linear(C.Structure):
    _fields_ = [("in_features", C.c_int), ("out_features", C.c_int), ("w_bf16", Tensor), ("w_fp8", Tensor),
                ("w_scales", Tensor), ("fp8_ready", C.c_int), ("w_int8", Tensor), ("w_iscale", Tensor),
                ("w_pack", Tensor), ("int8_ready", C.c_int), ("q_group", C.c_int), ("q_packed", C.c_int)]


class ModelOpts(C.Structure):
    _fields_ = [("gemm_mode", C.c_int), ("ctx_len", C.c_int), ("max_sessions", C.c_int)]


class SamplingCfg(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("repetition_penalty", C.c_float),
                ("repetition_window", C.c_int), ("seed", C.c_uint64)]


class VqPart(C.Structure):
    _fields_ = [("codes", C.POINTER(C.c_int32)), ("T", C.c_int)]


_P, _I, _S = C.c_void_p, C.c_int, C.c_void_p  # pointer, int, cudaStream_t

# name -> (restype, argtypes); the same table types both this library and the
# rebuilt reference library, which exports the same entry points.
PROTOTYPES = {
    "s2p_status_str": (C.c_char_p, [_I]),
    "s2p_dtype_size": (C.c_size_t, [_I]),
    "s2p_tensor_numel": (C.c_int64, [C.POINTER(Tensor)]),
    "s2p_tensor_device_alloc": (_I, [C.POINTER(Tensor), _I, _I, C.POINTER(C.c_int64)]),
    "s2p_tensor_host_alloc": (_I, [C.POINTER(Tensor), _I, _I, C.POINTER(C.c_int64)]),
    "s2p_tensor_upload": (_I, [C.POINTER(Tensor), _P, C.c_size_t, _S]),
    "s2p_tensor_download": (_I, [_P, C.POINTER(Tensor), C.c_size_t, _S]),
    "s2p_tensor_free": (None, [C.POINTER(Tensor)]),
    "s2p_st_open_dir": (_I, [C.c_char_p, C.POINTER(_P)]),
    "s2p_st_find": (_I, [_P, C.c_char_p, _P]),
    "s2p_st_count": (_I, [_P]),
    "s2p_st_at": (_I, [_P, _I, _P]),
    "s2p_st_close": (None, [_P]),
    "s2p_st_load_device": (_I, [_P, C.c_char_p, _I, _I, C.POINTER(C.c_int64), C.POINTER(Tensor), _S]),
    "s2p_gemm_init": (_I, [_I]),
    "s2p_gemm_shutdown": (None, []),
    "s2p_gemm_mode_from_env": (_I, []),
    "s2p_fso_available": (_I, []),
    "s2p_linear_from_st": (_I, [C.POINTER(Linear), _P, C.c_char_p, _I, _I, _S]),
    "s2p_linear_prepare_fp8": (_I, [C.POINTER(Linear), _S]),
    "s2p_linear_prepare_int8": (_I, [C.POINTER(Linear), _S]),
    "s2p_linear_prepare_int8_site": (_I, [C.POINTER(Linear), _I, _S]),
    "s2p_linear_forward": (_I, [C.POINTER(Linear), _P, _P, _I, _I, _S]),
    "s2p_linear_free": (None, [C.POINTER(Linear)]),
    "s2p_gemm_bf16": (_I, [_P, _P, _P, _I, _I, _I, _S]),
    "s2p_int8_quant": (_I, [_P, _P, _P, _I, _I, _S]),
    "s2p_int8_gemv": (_I, [_P, _P, _P, _P, _I, _I, _I, _S]),
    "s2p_int8_dequant": (_I, [_P, _P, _P, _I, _I, _S]),
    "s2p_intq_quant": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _S]),
    "s2p_intq_gemv": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _S]),
    "s2p_intq_dequant": (_I, [_P, _P, _P, _I, _I, _I, _S]),
    "s2p_int4_pack": (_I, [_P, _P, _I, _I, _S]),
    "s2p_int4p_gemv": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _S]),
    "s2p_int4p_dequant": (_I, [_P, _P, _P, _I, _I, _I, _S]),
    "s2p_qcache_open": (_I, [C.c_char_p, _I, C.POINTER(_P)]),
    "s2p_qcache_reading": (_I, [_P]),
    "s2p_qcache_try_load": (_I, [_P, C.c_char_p, _I, _I, C.POINTER(Linear), _S]),
    "s2p_qcache_put_linear": (_I, [_P, C.c_char_p, C.POINTER(Linear), _S]),
    "s2p_qcache_finish": (_I, [_P, _S]),
    "s2p_qcache_free": (None, [_P]),
    "s2pk_rms_norm": (_I, [_P, _P, _P, _I, _I, C.c_float, _S]),
    "s2pk_qk_norm": (_I, [_P, _P, _I, _I, _I, C.c_float, _S]),
    "s2pk_rope": (_I, [_P, _P, _I, _I, _I, _I, _I, C.c_float, _S]),
    "s2pk_kv_append": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _S]),
    "s2pk_attention": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _S]),
    "s2pk_silu_mul": (_I, [_P, _P, _I, _I, _S]),
    "s2pk_add": (_I, [_P, _P, C.c_int64, _S]),
    "s2pk_embed": (_I, [_P, _P, _P, _I, _I, _S]),
    "s2pk_sample_prepare": (_I, [_P, _P, _I, _S]),
    "s2pk_argmax": (_I, [_P, _P, _I, _I, _S]),
    "s2p_sampling_defaults": (SamplingCfg, []),
    "s2p_model_load": (_I, [C.c_char_p, C.POINTER(ModelOpts), C.POINTER(_P)]),
    "s2p_model_free": (None, [_P]),
    "s2p_session_create": (_I, [_P, C.POINTER(SamplingCfg), C.POINTER(_P)]),
    "s2p_session_prefill": (_I, [_P, _P, _P, _I, _P, _I]),
    "s2p_session_kv_bytes": (C.c_size_t, [_P, _I]),
    "s2p_session_kv_save": (_I, [_P, _I, _P]),
    "s2p_session_kv_load": (_I, [_P, _P, _I]),
    "s2p_session_next_frame": (_I, [_P, C.POINTER(C.c_int32), C.POINTER(_I)]),
    "s2p_session_destroy": (None, [_P]),
    "s2p_model_batch_next_frame": (_I, [_P, C.POINTER(_P), _I, C.POINTER(C.c_int32), C.POINTER(_I)]),
}

# additive entry points of this library only (include/s2p_b200_ext.h)
class Stats(C.Structure):
    _fields_ = [("frames_decoded", C.c_uint64), ("n_slow_layers", C.c_int), ("last_tick_rows", C.c_int),
                ("last_tick_fused", C.c_int), ("last_tick_graph", C.c_int), ("last_tick_kernels", C.c_int),
                ("last_tick_device_ms", C.c_float), ("upload_bytes", C.c_size_t), ("download_bytes", C.c_size_t),
                ("weight_bytes_per_frame", C.c_double), ("kv_bytes_per_token", C.c_double),
                ("last_tick_persistent", C.c_int)]


EXT_PROTOTYPES = {
    "s2p_b200_version": (C.c_char_p, []),
    "s2p_b200_model_stats": (_I, [_P, C.POINTER(Stats)]),
    "s2p_b200_model_stream": (C.c_void_p, [_P]),
    "s2p_b200_model_tick_trace": (_I, [_P, _P, _P, _I, C.POINTER(C.c_int)]),
    "s2p_b200_model_tick_trace_ctas": (_I, [_P, _P, _P, _I, _I, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "s2p_b200_model_tp_export": (_I, [_P, _P]),
    "s2p_b200_model_tp_attach": (_I, [_P, _I, _I, _P]),
    "s2p_b200_attention_decode_noalloc": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _S]),
}


def bind(cdll, table, strict=True):
    """Attach restype/argtypes for every name in `table` that the library exports."""
    missing = []
    for name, (res, args) in table.items():
        try:
            fn = getattr(cdll, name)
        except AttributeError:
            missing.append(name)
            continue
        fn.restype = res
        fn.argtypes = args
    if strict and missing:
        raise ImportError(f"{cdll._name} lacks entry points: {missing}")
    return missing


_lib = None


def load_library(path=None):
    """Load libs2pro_b200.so.  Raises ImportError if it is not built: there is no fallback."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise ImportError(f"{p} not found: build it with `make -C {os.path.join(HERE, 'csrc')}` "
                          "(or __graft_entry__.build()); there is no CPU fallback")
    cdll = C.CDLL(p)
    bind(cdll, PROTOTYPES)
    bind(cdll, EXT_PROTOTYPES)
    if path is None:
        _lib = cdll
    return cdll


def lib():
    return load_library()
