"""Seeded synthetic checkpoints with the tensor names and shapes of the S2-Pro
dual-AR model (reference: src/slowar/model.c:3-14, src/fastar/fastar.cu:219-274).

The real checkpoint is gated and cannot be fetched, so parity tests and the
benchmark run on random-initialised weights: every matrix and embedding table is
N(0, 0.02^2) drawn in f32 from a per-tensor seeded generator and rounded to bf16
(round to nearest even); RMSNorm / qk-norm gains are 1.0.  The file is a plain
single-shard ``model.safetensors`` (u64 header length, JSON header, raw data).
"""
import json
import os
import zlib
from concurrent.futures import ThreadPoolExecutor

import numpy as np

DIM, QKV, QW, FFN, VOCAB = 2560, 6144, 4096, 9728, 155776
HEAD_DIM, FAST_LAYERS, CB_SIZE, NUM_CB = 128, 4, 4096, 10


def tensor_specs(n_slow=36):
    """[(name, shape, kind)] in file order; kind 'w' = N(0, 0.02), 'g' = ones."""
    specs = [("text_model.model.embeddings.weight", (VOCAB, DIM), "w")]
    for i in range(n_slow):
        p = f"text_model.model.layers.{i}."
        specs += [(p + "attention.wqkv.weight", (QKV, DIM), "w"), (p + "attention.wo.weight", (DIM, QW), "w"),
                  (p + "attention.q_norm.weight", (HEAD_DIM,), "g"), (p + "attention.k_norm.weight", (HEAD_DIM,), "g"),
                  (p + "attention_norm.weight", (DIM,), "g"), (p + "ffn_norm.weight", (DIM,), "g"),
                  (p + "feed_forward.w1.weight", (FFN, DIM), "w"), (p + "feed_forward.w3.weight", (FFN, DIM), "w"),
                  (p + "feed_forward.w2.weight", (DIM, FFN), "w")]
    specs.append(("text_model.model.norm.weight", (DIM,), "g"))
    for i in range(FAST_LAYERS):
        p = f"audio_decoder.layers.{i}."
        specs += [(p + "attention.wqkv.weight", (QKV, DIM), "w"), (p + "attention.wo.weight", (DIM, QW), "w"),
                  (p + "attention_norm.weight", (DIM,), "g"), (p + "ffn_norm.weight", (DIM,), "g"),
                  (p + "feed_forward.w1.weight", (FFN, DIM), "w"), (p + "feed_forward.w3.weight", (FFN, DIM), "w"),
                  (p + "feed_forward.w2.weight", (DIM, FFN), "w")]
    specs += [("audio_decoder.norm.weight", (DIM,), "g"), ("audio_decoder.output.weight", (CB_SIZE, DIM), "w"),
              ("audio_decoder.codebook_embeddings.weight", (NUM_CB * CB_SIZE, DIM), "w"),
              ("audio_decoder.embeddings.weight", (CB_SIZE, DIM), "w")]
    return specs


def f32_to_bf16_bits(x):
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)).astype(np.uint16)


def tensor_values(name, shape, kind, seed, std=0.02):
    """bf16 bit patterns of one tensor; deterministic in (seed, name)."""
    n = int(np.prod(shape))
    if kind == "g":
        return np.full(n, 0x3F80, dtype=np.uint16).reshape(shape)
    rng = np.random.Generator(np.random.Philox(key=[seed, zlib.crc32(name.encode())]))
    out = np.empty(n, dtype=np.uint16)
    step = 1 << 24
    for lo in range(0, n, step):
        hi = min(n, lo + step)
        out[lo:hi] = f32_to_bf16_bits(rng.standard_normal(hi - lo, dtype=np.float32) * np.float32(std))
    return out.reshape(shape)


def _cuda_tensor_values(name, shape, kind, seed, std=0.02):
    """Same distribution drawn on the GPU (much faster for the 9 GB full model).
    The values differ from the numpy generator's; both are deterministic."""
    import torch
    n = int(np.prod(shape))
    if kind == "g":
        return np.full(n, 0x3F80, dtype=np.uint16)
    g = torch.Generator(device="cuda")
    g.manual_seed((seed << 32) ^ zlib.crc32(name.encode()))
    t = (torch.randn(n, device="cuda", dtype=torch.float32, generator=g) * std).to(torch.bfloat16)
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def write_checkpoint(model_dir, n_slow=36, seed=1, threads=None, generator="numpy"):
    """Write <model_dir>/model.safetensors; returns its path.  Existing files with
    the same stamp are reused.  generator: "numpy" (portable, deterministic
    everywhere), "cuda" (torch on the GPU) or "auto" (cuda when available)."""
    os.makedirs(model_dir, exist_ok=True)
    path = os.path.join(model_dir, "model.safetensors")
    stamp = os.path.join(model_dir, "synth.json")
    if generator == "auto":
        try:
            import torch
            generator = "cuda" if torch.cuda.is_available() else "numpy"
        except ImportError:
            generator = "numpy"
    want = {"n_slow": n_slow, "seed": seed, "std": 0.02, "generator": generator}
    if os.path.exists(path) and os.path.exists(stamp):
        with open(stamp) as f:
            if json.load(f) == want:
                return path
    specs = tensor_specs(n_slow)
    header, off = {}, 0
    for name, shape, _ in specs:
        nbytes = int(np.prod(shape)) * 2
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    total = 8 + len(hjson) + off
    with open(path, "wb") as f:
        f.write(len(hjson).to_bytes(8, "little"))
        f.write(hjson)
        f.truncate(total)
    mm = np.memmap(path, dtype=np.uint16, mode="r+", offset=8 + len(hjson), shape=(off // 2,))

    def fill(spec):
        name, shape, kind = spec
        lo, hi = header[name]["data_offsets"]
        vals = (_cuda_tensor_values if generator == "cuda" else tensor_values)(name, shape, kind, seed)
        mm[lo // 2:hi // 2] = vals.reshape(-1)

    if generator == "cuda":
        for spec in specs:
            fill(spec)
    else:
        with ThreadPoolExecutor(max_workers=threads or min(16, os.cpu_count() or 4)) as ex:
            list(ex.map(fill, specs))
    mm.flush()
    del mm
    with open(stamp, "w") as f:
        json.dump(want, f)
    return path


def random_prompt(n_ids, seed):
    """Uniform token ids over the text vocabulary, seeded."""
    rng = np.random.Generator(np.random.Philox(key=[seed, 0xC0FFEE]))
    return rng.integers(0, VOCAB, size=n_ids, dtype=np.int64)
