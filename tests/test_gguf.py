"""GGUF: block decoders against llama.cpp-derived golden vectors (``GRIMOIRE_GGUF_GOLDEN_DIR`` names a directory of
``<TYPE>.bin`` files: b"GGLD", type, n_expected, raw_size, raw blocks, expected fp32; the reference project ships them
under tests/gguf/data), the container parser on a file written by the test, and the name adapter."""
import os
import struct
from pathlib import Path

import pytest
import torch

from grimoire_b200.formats import gguf

def _golden_dir() -> Path:
    env = os.environ.get("GRIMOIRE_GGUF_GOLDEN_DIR")
    if env:
        return Path(env)
    # a reference checkout beside this repository, when there is one
    return Path(__file__).resolve().parents[2] / "reference" / "tests" / "gguf" / "data"


GOLD = _golden_dir()
DECODED = ["F32", "F16", "BF16", "F64", "I8", "I16", "I32", "I64", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q8_1", "Q2_K", "Q3_K",
           "Q4_K", "Q5_K", "Q6_K", "Q8_K", "IQ4_NL", "IQ4_XS", "TQ2_0", "MXFP4"]


@pytest.mark.skipif(not GOLD.exists(), reason="golden vectors not available on this machine")
@pytest.mark.parametrize("name", DECODED)
def test_block_decoders_match_goldens(name):
    blob = (GOLD / f"{name}.bin").read_bytes()
    assert blob[:4] == b"GGLD"
    qtype, n_exp, raw_size = struct.unpack_from("<III", blob, 4)
    raw = blob[16: 16 + raw_size]
    want = torch.frombuffer(bytearray(blob[16 + raw_size: 16 + raw_size + 4 * n_exp]), dtype=torch.float32)
    got = gguf.dequantize(qtype, raw, n_exp)
    assert torch.equal(got, want), (name, float((got - want).abs().max()))


def test_undecoded_types_are_reported():
    with pytest.raises(NotImplementedError):
        gguf.dequantize(16, b"\0" * 66, 256)          # IQ2_XXS needs a codebook this build does not carry
    with pytest.raises(ValueError):
        gguf.dequantize(2, b"\0" * 17, 32)            # wrong byte count


def _write_gguf(path, kv, tensors, version=3, alignment=32):
    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    out = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kv))
    for k, (t, v) in kv.items():
        out += s(k) + struct.pack("<I", t)
        if t == 4:
            out += struct.pack("<I", v)
        elif t == 6:
            out += struct.pack("<f", v)
        elif t == 8:
            out += s(v)
        elif t == 9:
            et, items = v
            out += struct.pack("<IQ", et, len(items))
            for it in items:
                out += s(it) if et == 8 else struct.pack("<i", it)
    data, off = b"", 0
    for name, (typ, dims, raw) in tensors.items():
        out += s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, off)
        pad = (alignment - len(raw) % alignment) % alignment
        data += raw + b"\0" * pad
        off += len(raw) + pad
    out += b"\0" * ((alignment - len(out) % alignment) % alignment)
    Path(path).write_bytes(out + data)


def test_container_parser_and_adapter(tmp_path):
    torch.manual_seed(0)
    w = torch.randn(8, 64)
    q8 = b""
    for row in w:
        for blk in row.reshape(-1, 32):
            d = float(blk.abs().max()) / 127
            q8 += struct.pack("<e", d) + bytes((torch.round(blk / d).to(torch.int8).view(torch.uint8)).tolist())
    kv = {"general.architecture": (8, "qwen3"), "qwen3.block_count": (4, 1), "qwen3.embedding_length": (4, 64),
          "qwen3.attention.head_count": (4, 2), "qwen3.attention.head_count_kv": (4, 1), "qwen3.feed_forward_length": (4, 128),
          "qwen3.rope.freq_base": (6, 1e6), "tokenizer.ggml.model": (8, "gpt2"), "tokenizer.ggml.tokens": (9, (8, ["a", "b", "ab"])),
          "tokenizer.ggml.merges": (9, (8, ["a b"])), "tokenizer.ggml.token_type": (9, (5, [1, 1, 1]))}
    tensors = {"blk.0.attn_q.weight": (8, (64, 8), q8), "output_norm.weight": (0, (64,), torch.ones(64).numpy().tobytes())}
    _write_gguf(tmp_path / "m.gguf", kv, tensors)
    g = gguf.GGUFFile(tmp_path / "m.gguf")
    assert g.version == 3 and g.arch == "qwen3" and g.metadata["qwen3.block_count"] == 1
    t = g.tensor("blk.0.attn_q.weight")
    assert t.shape == (8, 64) and float((t - w).abs().max()) < 0.02
    assert gguf.hf_name("blk.0.attn_q.weight") == "model.layers.0.self_attn.q_proj.weight"
    assert gguf.hf_name("blk.12.ffn_down.weight") == "model.layers.12.mlp.down_proj.weight"
    cfg = gguf.config_from_gguf(g)
    assert cfg.num_hidden_layers == 1 and cfg.hidden_size == 64 and cfg.num_key_value_heads == 1 and cfg.tie_word_embeddings
    tj = gguf.tokenizer_json_from_gguf(g)
    assert tj["model"]["vocab"] == {"a": 0, "b": 1, "ab": 2} and tj["model"]["merges"] == ["a b"]
    with pytest.raises(ValueError):
        (tmp_path / "bad.gguf").write_bytes(b"GGUX" + b"\0" * 64)
        gguf.GGUFFile(tmp_path / "bad.gguf")


def test_gguf_file_loads_into_the_engine(tmp_path):
    """A whole (tiny, F32) GGUF model through the public API: config + tensors + tokenizer from the file, and the
    tokens must equal those of the same weights loaded as a state dict."""
    from grimoire_b200.api import Grimoire
    from grimoire_b200.config import EngineConfig
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.config import ModelConfig
    from grimoire_b200.models.dense import DenseModel

    H, I, L, V, Hq, Hkv, D = 128, 256, 2, 64, 2, 1, 64
    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.05
    sd, tensors = {}, {}

    def put(gname, hname, t):
        sd[hname] = t
        tensors[gname] = (0, tuple(reversed(t.shape)), t.contiguous().numpy().tobytes())      # type 0 = F32, ggml dims are reversed
    put("token_embd.weight", "model.embed_tokens.weight", rnd(V, H))
    put("output_norm.weight", "model.norm.weight", torch.ones(H))
    for i in range(L):
        for gn, hn, shape in (("attn_q", "self_attn.q_proj", (Hq * D, H)), ("attn_k", "self_attn.k_proj", (Hkv * D, H)),
                              ("attn_v", "self_attn.v_proj", (Hkv * D, H)), ("attn_output", "self_attn.o_proj", (H, Hq * D)),
                              ("ffn_gate", "mlp.gate_proj", (I, H)), ("ffn_up", "mlp.up_proj", (I, H)), ("ffn_down", "mlp.down_proj", (H, I))):
            put(f"blk.{i}.{gn}.weight", f"model.layers.{i}.{hn}.weight", rnd(*shape))
        put(f"blk.{i}.attn_norm.weight", f"model.layers.{i}.input_layernorm.weight", torch.ones(H))
        put(f"blk.{i}.ffn_norm.weight", f"model.layers.{i}.post_attention_layernorm.weight", torch.ones(H))
    toks = [chr(0x100 + i) for i in range(V)]
    kv = {"general.architecture": (8, "qwen3"), "qwen3.block_count": (4, L), "qwen3.embedding_length": (4, H),
          "qwen3.attention.head_count": (4, Hq), "qwen3.attention.head_count_kv": (4, Hkv), "qwen3.attention.key_length": (4, D),
          "qwen3.feed_forward_length": (4, I), "qwen3.rope.freq_base": (6, 1e6), "tokenizer.ggml.model": (8, "gpt2"),
          "tokenizer.ggml.tokens": (9, (8, toks)), "tokenizer.ggml.merges": (9, (8, [])), "tokenizer.ggml.token_type": (9, (5, [1] * V))}
    _write_gguf(tmp_path / "tiny.gguf", kv, tensors)
    llm = Grimoire.load(EngineConfig(model=str(tmp_path / "tiny.gguf"), ctx=64, seq_slots=2, prefill_chunk=32), device="cpu")
    assert llm.model.cfg.num_hidden_layers == L and llm.model.cfg.head_dim == D and llm.tokenizer is not None
    prompt = [3, 9, 27, 11, 5]
    got, _ = llm.generate(prompt, 6)
    cfg = ModelConfig(model_type="qwen3", hidden_size=H, num_hidden_layers=L, num_attention_heads=Hq, num_key_value_heads=Hkv, head_dim=D,
                      vocab_size=V, intermediate_size=I, tie_word_embeddings=True, rope_theta=1e6)
    want = Engine(DenseModel.from_state_dict(cfg, sd, "cpu"), EngineLimits(max_slots=2, max_ctx=64, prefill_chunk=32, max_decode_rows=4)).generate(prompt, 6)
    assert list(got) == list(want)
    llm.close()


def _q8_0_rows(w: torch.Tensor) -> bytes:
    out = b""
    for row in w:
        for blk in row.reshape(-1, 32):
            d = float(blk.abs().max()) / 127 or 1.0
            out += struct.pack("<e", d) + bytes((torch.round(blk / d).clamp(-127, 127).to(torch.int8).view(torch.uint8)).tolist())
    return out


def test_gguf_native_projections_keep_the_files_blocks(tmp_path):
    """``--proj native`` on a GGUF file: the projections stay the stored Q8_0 blocks (GgufLinear over the raw rows) and the
    logits agree with the same file loaded through the dequantise-and-requantise path at bf16."""
    from grimoire_b200.api import Grimoire
    from grimoire_b200.config import EngineConfig
    from grimoire_b200.ops.linear import GgufLinear

    H, I, L, V, Hq, Hkv, D = 128, 256, 2, 64, 2, 1, 64
    g = torch.Generator().manual_seed(1)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.05
    tensors = {}
    f32 = lambda name, t: tensors.__setitem__(name, (0, tuple(reversed(t.shape)), t.contiguous().numpy().tobytes()))
    q8 = lambda name, t: tensors.__setitem__(name, (8, tuple(reversed(t.shape)), _q8_0_rows(t)))
    f32("token_embd.weight", rnd(V, H))
    f32("output_norm.weight", torch.ones(H))
    q8("output.weight", rnd(V, H))
    for i in range(L):
        for gn, shape in (("attn_q", (Hq * D, H)), ("attn_k", (Hkv * D, H)), ("attn_v", (Hkv * D, H)), ("attn_output", (H, Hq * D)),
                          ("ffn_gate", (I, H)), ("ffn_up", (I, H)), ("ffn_down", (H, I))):
            q8(f"blk.{i}.{gn}.weight", rnd(*shape))
        f32(f"blk.{i}.attn_norm.weight", torch.ones(H))
        f32(f"blk.{i}.ffn_norm.weight", torch.ones(H))
    toks = [chr(0x100 + i) for i in range(V)]
    kv = {"general.architecture": (8, "qwen3"), "qwen3.block_count": (4, L), "qwen3.embedding_length": (4, H),
          "qwen3.attention.head_count": (4, Hq), "qwen3.attention.head_count_kv": (4, Hkv), "qwen3.attention.key_length": (4, D),
          "qwen3.feed_forward_length": (4, I), "qwen3.rope.freq_base": (6, 1e6), "tokenizer.ggml.model": (8, "gpt2"),
          "tokenizer.ggml.tokens": (9, (8, toks)), "tokenizer.ggml.merges": (9, (8, [])), "tokenizer.ggml.token_type": (9, (5, [1] * V))}
    path = tmp_path / "q8.gguf"
    _write_gguf(path, kv, tensors)
    gf = gguf.GGUFFile(path)
    raw, typ = gf.raw_rows("blk.0.ffn_down.weight")
    assert typ == 8 and raw.shape == (H, I // 32 * 34) and gguf.native_ok(gf, gguf.config_from_gguf(gf))
    gf.close()
    ids = torch.randint(0, V, (19,), generator=g).tolist()
    nat = Grimoire.load(EngineConfig(model=str(path), proj="native", ctx=64, seq_slots=2, prefill_chunk=32), device="cpu")
    assert all(isinstance(l.qkv, GgufLinear) and isinstance(l.down, GgufLinear) for l in nat.model.layers)
    assert isinstance(nat.model.lm_head, GgufLinear) and len(nat.model.layers[0].qkv.parts) == 3
    a = nat.score_ids(ids)
    ref = Grimoire.load(EngineConfig(model=str(path), proj="bf16", ctx=64, seq_slots=2, prefill_chunk=32), device="cpu")
    b = ref.score_ids(ids)
    assert float((a - b).abs().max()) < 0.03 * max(1.0, float(b.abs().max()))
    assert float((a.argmax(-1) == b.argmax(-1)).float().mean()) >= 0.9
    nat.close(), ref.close()
