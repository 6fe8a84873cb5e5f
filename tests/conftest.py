import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    with np.load(ROOT / "tests" / "golden" / "bctx_golden.npz") as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def orc():
    from oracle import bcx_oracle

    bcx_oracle.build()
    return bcx_oracle


@pytest.fixture(scope="session")
def oracle_coder(orc):
    return orc.Coder("oracle")


def _write_decoder_checkpoint(model_dir, *, hidden, layers, heads, kv_heads, ffn, vocab, head_dim=128, seed=0, mtp=True, tied=False,
                              extra=None):
    """A random-init safetensors checkpoint of a plain grouped-query decoder under the usual tensor names, with its
    config.json.  Returns {tensor name: BF16 bit patterns}."""
    import json
    import struct

    import torch

    g = torch.Generator().manual_seed(seed)

    def matrix(rows, cols):
        w = torch.randn(rows, cols, generator=g) * 0.05 * torch.exp(0.25 * torch.randn(rows, 1, generator=g))
        return w.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)

    def scale():
        return (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)

    def layer(prefix):
        return {prefix + "input_layernorm.weight": scale(), prefix + "post_attention_layernorm.weight": scale(),
                prefix + "self_attn.q_proj.weight": matrix(heads * head_dim, hidden), prefix + "self_attn.k_proj.weight": matrix(kv_heads * head_dim, hidden),
                prefix + "self_attn.v_proj.weight": matrix(kv_heads * head_dim, hidden), prefix + "self_attn.o_proj.weight": matrix(hidden, heads * head_dim),
                prefix + "mlp.gate_proj.weight": matrix(ffn, hidden), prefix + "mlp.up_proj.weight": matrix(ffn, hidden),
                prefix + "mlp.down_proj.weight": matrix(hidden, ffn)}

    tensors = {"model.embed_tokens.weight": matrix(vocab, hidden), "model.norm.weight": scale()}
    if not tied:
        tensors["lm_head.weight"] = matrix(vocab, hidden)
    for i in range(layers):
        tensors.update(layer(f"model.layers.{i}."))
    if mtp:
        tensors.update({"mtp.fc.weight": matrix(hidden, 2 * hidden), "mtp.pre_fc_norm_embedding.weight": scale(),
                        "mtp.pre_fc_norm_hidden.weight": scale(), "mtp.norm.weight": scale()})
        tensors.update(layer("mtp.layers.0."))
    tensors.update(extra or {})
    model_dir.mkdir(parents=True, exist_ok=True)
    header, blob = {}, b""
    for name, words in tensors.items():
        raw = np.ascontiguousarray(words).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(words.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    (model_dir / "model.safetensors").write_bytes(struct.pack("<Q", len(text)) + text + blob)
    (model_dir / "config.json").write_text(json.dumps({
        "hidden_size": hidden, "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
        "head_dim": head_dim, "intermediate_size": ffn, "vocab_size": vocab, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
        "tie_word_embeddings": tied}))
    return tensors


@pytest.fixture(scope="session")
def write_decoder_checkpoint():
    return _write_decoder_checkpoint
