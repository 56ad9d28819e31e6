"""CPU tests of the C-ABI library and its host logic: the library loads without a
GPU, exports every entry point the header declares, and the checkpoint reader,
status strings and argument validation behave as the reference's contracts say."""
import ctypes as C
import json
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions(header):
    src = open(os.path.join(ROOT, "include", header)).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    src = re.sub(r"#define[^\n]*(\\\n[^\n]*)*", "", src)
    return sorted(set(re.findall(r"\b(s2pk?_[a-z0-9_]+)\s*\(", src)) - {"s2p_try_rc_", "s2p_try_ce_"})


def test_library_exports_every_declared_symbol(mine, capi):
    names = declared_functions("s2p_b200_abi.h") + declared_functions("s2p_b200_ext.h")
    assert len(names) > 60
    missing = [n for n in names if not hasattr(mine, n)]
    assert not missing, missing
    # and nothing but the declared interface is exported
    out = subprocess.run(["nm", "-D", "--defined-only", capi.LIB_PATH], capture_output=True, text=True).stdout
    exported = {l.split()[-1] for l in out.splitlines() if " T " in l}
    extra = sorted(e for e in exported if e not in names and not e.startswith("_"))
    assert not extra, extra


def test_python_prototypes_cover_the_header(capi):
    names = set(declared_functions("s2p_b200_abi.h") + declared_functions("s2p_b200_ext.h"))
    table = set(capi.PROTOTYPES) | set(capi.EXT_PROTOTYPES)
    assert names == table, (names ^ table)


def test_status_strings_and_dtype_sizes(mine):
    assert mine.s2p_status_str(0) == b"ok"
    assert mine.s2p_status_str(-9) == b"capacity exhausted"
    assert mine.s2p_status_str(-6) == b"invalid state"
    assert mine.s2p_status_str(-77) == b"unknown status"
    assert [mine.s2p_dtype_size(i) for i in range(7)] == [2, 4, 2, 1, 4, 8, 1]
    assert mine.s2p_dtype_size(99) == 0
    assert mine.s2p_fso_available() == 0


def test_struct_layouts_match_the_reference_abi(capi):
    """sizes / offsets of the structs that cross the ABI (include/s2pro/tensor.h:23-30,
    gemm.h:42-62, model.h:28-38 of the reference) on LP64."""
    assert C.sizeof(capi.Tensor) == 64
    assert capi.Tensor.shape.offset == 16 and capi.Tensor.bytes.offset == 48 and capi.Tensor.on_device.offset == 56
    assert C.sizeof(capi.Linear) == 8 + 3 * 64 + 8 + 3 * 64 + 16
    assert capi.Linear.w_int8.offset == 8 + 3 * 64 + 8
    assert capi.Linear.q_packed.offset == C.sizeof(capi.Linear) - 8
    assert C.sizeof(capi.ModelOpts) == 12 and C.sizeof(capi.SamplingCfg) == 24 and capi.SamplingCfg.seed.offset == 16


def test_sampling_defaults(mine):
    d = mine.s2p_sampling_defaults()
    assert (round(d.temperature, 3), round(d.top_p, 3), round(d.repetition_penalty, 3), d.repetition_window, d.seed) == (0.8, 0.8, 1.1, 16, 0)


def write_safetensors(path, tensors, pad=0):
    header, off, blobs = {}, 0, []
    for name, (dtype, arr) in tensors.items():
        b = arr.tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        off += len(b); blobs.append(b)
    header["__metadata__"] = {"format": "pt", "note": 'with "escapes" and {braces}'}
    hj = json.dumps(header).encode() + b" " * pad
    with open(path, "wb") as f:
        f.write(len(hj).to_bytes(8, "little")); f.write(hj)
        for b in blobs:
            f.write(b)


def test_safetensors_reader_single_and_sharded(mine, capi, tmp_path):
    a = np.arange(24, dtype=np.uint16).reshape(4, 6); b = np.arange(5, dtype=np.float32); c = np.arange(7, dtype=np.int64)
    d1 = tmp_path / "single"; d1.mkdir()
    write_safetensors(d1 / "model.safetensors", {"a.weight": ("BF16", a), "b": ("F32", b)}, pad=3)
    st = C.c_void_p()
    assert mine.s2p_st_open_dir(str(d1).encode(), C.byref(st)) == 0
    assert mine.s2p_st_count(st) == 2

    class View(C.Structure):
        _fields_ = [("name", C.c_char_p), ("dtype", C.c_int), ("ndim", C.c_int), ("shape", C.c_int64 * 4),
                    ("data", C.c_void_p), ("nbytes", C.c_size_t)]
    v = View()
    assert mine.s2p_st_find(st, b"a.weight", C.byref(v)) == 0
    assert (v.dtype, v.ndim, list(v.shape)[:2], v.nbytes) == (0, 2, [4, 6], 48)
    assert np.array_equal(np.frombuffer(C.string_at(v.data, v.nbytes), np.uint16).reshape(4, 6), a)
    assert mine.s2p_st_find(st, b"missing", C.byref(v)) == -1  # S2P_ERR_INVALID, as the reference
    assert mine.s2p_st_at(st, 1, C.byref(v)) == 0 and mine.s2p_st_at(st, 2, C.byref(v)) == -1
    mine.s2p_st_close(st)
    # sharded, with the index naming two shards
    d2 = tmp_path / "sharded"; d2.mkdir()
    write_safetensors(d2 / "model-00001-of-00002.safetensors", {"a.weight": ("BF16", a)})
    write_safetensors(d2 / "model-00002-of-00002.safetensors", {"b": ("F32", b), "c": ("I64", c)})
    (d2 / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": 1}, "weight_map": {
        "a.weight": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors", "c": "model-00002-of-00002.safetensors"}}))
    assert mine.s2p_st_open_dir(str(d2).encode(), C.byref(st)) == 0
    assert mine.s2p_st_count(st) == 3
    assert mine.s2p_st_find(st, b"c", C.byref(v)) == 0 and v.dtype == 5 and v.nbytes == 56
    mine.s2p_st_close(st)


def test_safetensors_reader_rejects_bad_files(mine, tmp_path):
    st = C.c_void_p()
    assert mine.s2p_st_open_dir(str(tmp_path / "nope").encode(), C.byref(st)) == -3      # IO
    d = tmp_path / "bad"; d.mkdir()
    (d / "model.safetensors").write_bytes(b"\x05")
    assert mine.s2p_st_open_dir(str(d).encode(), C.byref(st)) == -5                      # FORMAT: truncated
    (d / "model.safetensors").write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    assert mine.s2p_st_open_dir(str(d).encode(), C.byref(st)) == -5                      # header longer than the file
    hj = json.dumps({"x": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 6]}}).encode()
    (d / "model.safetensors").write_bytes(len(hj).to_bytes(8, "little") + hj + b"\0" * 6)
    assert mine.s2p_st_open_dir(str(d).encode(), C.byref(st)) == -5                      # size != shape * dtype
    hj = json.dumps({"x": {"dtype": "F64", "shape": [1], "data_offsets": [0, 8]}}).encode()
    (d / "model.safetensors").write_bytes(len(hj).to_bytes(8, "little") + hj + b"\0" * 8)
    assert mine.s2p_st_open_dir(str(d).encode(), C.byref(st)) == -7                      # UNSUPPORTED dtype
    dup = b'{"x":{"dtype":"U8","shape":[1],"data_offsets":[0,1]},"x":{"dtype":"U8","shape":[1],"data_offsets":[0,1]}}'
    (d / "model.safetensors").write_bytes(len(dup).to_bytes(8, "little") + dup + b"\0")
    assert mine.s2p_st_open_dir(str(d).encode(), C.byref(st)) == -5                      # duplicate tensor name


def test_argument_validation_without_a_gpu(mine, capi):
    """Entry points reject bad arguments before touching the device (gemm.h / model.h contracts)."""
    p = C.c_void_p(256)
    assert mine.s2p_int8_gemv(p, p, p, p, 1, 8, 500, None) == -1       # K % 512
    assert mine.s2p_int8_gemv(p, p, p, p, 17, 8, 512, None) == -1      # M > 16
    assert mine.s2p_int8_gemv(None, p, p, p, 1, 8, 512, None) == -1
    assert mine.s2p_int4p_gemv(p, p, p, p, 1, 8, 512, 24, None) == -1  # group not a power of two
    assert mine.s2p_int4p_gemv(p, p, p, p, 1, 8, 512, 8, None) == -1   # group < 16
    assert mine.s2p_intq_quant(p, p, p, 4, 100, 32, 7, 1, None) == -1  # K % G
    assert mine.s2p_int4_pack(p, p, 4, 7, None) == -1                  # odd K
    assert mine.s2p_int8_gemv(p, C.c_void_p(258), p, p, 1, 8, 512, None) == -1  # misaligned activations
    assert mine.s2p_model_load(None, None, None) == -1
    assert mine.s2p_session_create(None, None, None) == -1
    assert mine.s2p_session_kv_bytes(None, 5) == 0
    assert mine.s2p_model_batch_next_frame(None, None, 0, None, None) == -1
    lin = capi.Linear()
    assert mine.s2p_linear_forward(C.byref(lin), p, p, 1, capi.GEMM_INT8, None) == -6  # gemm context not initialised: STATE
    assert mine.s2p_qcache_try_load(None, b"x", 1, 1, C.byref(lin), None) == 0
    qc = C.c_void_p(123)
    assert mine.s2p_qcache_open(b"/nonexistent", capi.GEMM_BF16, C.byref(qc)) == 0 and qc.value is None  # no cache for BF16


def test_synthetic_checkpoint_names_and_determinism(synth, mine, tmp_path):
    specs = synth.tensor_specs(2)
    names = [s[0] for s in specs]
    assert "text_model.model.layers.1.feed_forward.w3.weight" in names and "text_model.model.layers.2.attention.wo.weight" not in names
    assert ("audio_decoder.codebook_embeddings.weight", (40960, 2560), "w") in specs
    a = synth.tensor_values("x", (8, 16), "w", 3); b = synth.tensor_values("x", (8, 16), "w", 3); c = synth.tensor_values("y", (8, 16), "w", 3)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert np.array_equal(synth.f32_to_bf16_bits(np.array([1.0, 1.00390625, 1.01171875], np.float32)), np.array([0x3F80, 0x3F80, 0x3F82], np.uint16))
    ids = synth.random_prompt(64, 7)
    assert ids.dtype == np.int64 and ids.min() >= 0 and ids.max() < 155776 and np.array_equal(ids, synth.random_prompt(64, 7))


def test_bench_byte_model():
    import bench
    per_layer = 6144 * 2560 + 2560 * 4096 + 19456 * 2560 + 2560 * 9728
    assert per_layer == 100925440
    int4 = bench.algorithmic_bytes_per_frame("int4")
    int8 = bench.algorithmic_bytes_per_frame("int8")
    assert abs(int4 - 4.378e9) < 2e6 and abs(int8 - 7.785e9) < 5e6
