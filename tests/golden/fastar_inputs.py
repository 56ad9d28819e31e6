"""Seeded inputs of the fast-AR golden case, shared by the fixture generator
(which feeds them to the reference's torch model) and the test (which feeds them
to the CPU oracle).  torch's CPU generator is deterministic across machines."""
import torch

DIMS = {"dim": 512, "q_heads": 4, "kv_heads": 1, "ffn": 1024, "layers": 4, "rows": 6}


def bf16_round(t):
    return t.to(torch.bfloat16).float()


def make_inputs():
    g = torch.Generator().manual_seed(77)
    D, FFN = DIMS["dim"], DIMS["ffn"]
    QKV, QW = (DIMS["q_heads"] + 2 * DIMS["kv_heads"]) * 128, DIMS["q_heads"] * 128

    def mat(n, k, std=0.05):
        return bf16_round(torch.randn(n, k, generator=g) * std)
    tensors = {}
    for i in range(DIMS["layers"]):
        p = f"audio_decoder.layers.{i}"
        tensors[f"{p}.attention.wqkv.weight"] = mat(QKV, D)
        tensors[f"{p}.attention.wo.weight"] = mat(D, QW)
        tensors[f"{p}.feed_forward.w1.weight"] = mat(FFN, D)
        tensors[f"{p}.feed_forward.w3.weight"] = mat(FFN, D)
        tensors[f"{p}.feed_forward.w2.weight"] = mat(D, FFN)
        tensors[f"{p}.attention_norm.weight"] = bf16_round(1.0 + 0.1 * torch.randn(D, generator=g))
        tensors[f"{p}.ffn_norm.weight"] = bf16_round(1.0 + 0.1 * torch.randn(D, generator=g))
    tensors["audio_decoder.norm.weight"] = bf16_round(1.0 + 0.1 * torch.randn(D, generator=g))
    tensors["audio_decoder.output.weight"] = mat(4096, D)
    tensors["audio_decoder.embeddings.weight"] = mat(4096, D, std=1.0)
    hidden = bf16_round(torch.randn(DIMS["rows"], D, generator=g))
    sem = torch.randint(0, 4096, (DIMS["rows"],), generator=g)
    return tensors, hidden, sem
