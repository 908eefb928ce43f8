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
        elif t == 7:
            out += struct.pack("<B", 1 if v else 0)
        elif t == 8:
            out += s(v)
        elif t == 9:
            et, items = v
            out += struct.pack("<IQ", et, len(items))
            for it in items:
                out += s(it) if et == 8 else struct.pack("<f", it) if et == 6 else struct.pack("<i", it)
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


def _hybrid_gguf(path, cfg, sd, arch):
    """Write ``sd`` (HF names, key-grouped value heads) the way llama.cpp's converter stores the hybrid family: value heads
    tiled, ``ssm_a`` = -exp(A_log), zero-centred norms as 1 + w, experts stacked per layer, conv filter as [C][K]."""
    q35 = arch != "qwen3moe"
    L, H = cfg.num_hidden_layers, cfg.hidden_size
    nk, nv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    tensors = {}

    def put(name, t):
        t = t.float().contiguous()
        tensors[name] = (0, tuple(reversed(t.shape)), t.numpy().tobytes())

    def tile(t, width, dim=0):                 # forward transform: stored[order[g]] = hf[g]
        order = gguf.v_head_order(nk, nv, width)
        out = torch.empty_like(t)
        out.index_copy_(dim, order, t)
        return out

    bf = lambda t: t.bfloat16().float()
    norm = (lambda t: 1.0 + bf(t)) if q35 else bf
    put("token_embd.weight", bf(sd["model.embed_tokens.weight"]))
    put("output_norm.weight", norm(sd["model.norm.weight"]))
    if "lm_head.weight" in sd:
        put("output.weight", bf(sd["lm_head.weight"]))
    for i in range(L):
        p, b = f"model.layers.{i}.", f"blk.{i}."
        w = lambda k: bf(sd[p + k])
        put(b + "attn_norm.weight", norm(sd[p + "input_layernorm.weight"]))
        put(b + ("post_attention_norm.weight" if q35 else "ffn_norm.weight"), norm(sd[p + "post_attention_layernorm.weight"]))
        if cfg.is_attention_layer(i):
            for hf, gg in (("q_proj", "attn_q"), ("k_proj", "attn_k"), ("v_proj", "attn_v"), ("o_proj", "attn_output")):
                put(b + gg + ".weight", w(f"self_attn.{hf}.weight"))
            put(b + "attn_q_norm.weight", norm(sd[p + "self_attn.q_norm.weight"]))
            put(b + "attn_k_norm.weight", norm(sd[p + "self_attn.k_norm.weight"]))
        else:
            a, qk = "linear_attn.", 2 * nk * dk
            qkv, conv = w(a + "in_proj_qkv.weight"), w(a + "conv1d.weight").reshape(-1, cfg.linear_conv_kernel_dim)
            put(b + "attn_qkv.weight", torch.cat([qkv[:qk], tile(qkv[qk:], dv)]))
            put(b + "ssm_conv1d.weight", torch.cat([conv[:qk], tile(conv[qk:], dv)]))
            put(b + "attn_gate.weight", tile(w(a + "in_proj_z.weight"), dv))
            put(b + "ssm_alpha.weight", tile(w(a + "in_proj_a.weight"), 1))
            put(b + "ssm_beta.weight", tile(w(a + "in_proj_b.weight"), 1))
            put(b + "ssm_a", tile(-torch.exp(w(a + "A_log")), 1))
            put(b + "ssm_dt.bias", tile(w(a + "dt_bias"), 1))
            put(b + "ssm_norm.weight", w(a + "norm.weight"))
            put(b + "ssm_out.weight", tile(w(a + "out_proj.weight"), dv, dim=1))
        if not cfg.layer_is_sparse(i):
            for hf, gg in (("gate_proj", "ffn_gate"), ("up_proj", "ffn_up"), ("down_proj", "ffn_down")):
                put(b + gg + ".weight", w(f"mlp.{hf}.weight"))
            continue
        put(b + "ffn_gate_inp.weight", w("mlp.gate.weight"))
        if cfg.shared_expert_intermediate_size:
            put(b + "ffn_gate_inp_shexp.weight", w("mlp.shared_expert_gate.weight").reshape(-1))       # stored as a vector
            for hf, gg in (("gate_proj", "ffn_gate_shexp"), ("up_proj", "ffn_up_shexp"), ("down_proj", "ffn_down_shexp")):
                put(b + gg + ".weight", w(f"mlp.shared_expert.{hf}.weight"))
        E = cfg.num_experts
        for hf, gg in (("gate_proj", "ffn_gate_exps"), ("up_proj", "ffn_up_exps"), ("down_proj", "ffn_down_exps")):
            put(b + gg + ".weight", torch.stack([w(f"mlp.experts.{e}.{hf}.weight") for e in range(E)]))
    mtp = 1 if "mtp.fc.weight" in sd else 0
    if mtp:
        # the draft head travels as one more block: its layer under the decoder layers' roles, the rest under nextn.*
        p, b = "mtp.layers.0.", f"blk.{L}."
        for hf, gg in (("self_attn.q_proj", "attn_q"), ("self_attn.k_proj", "attn_k"), ("self_attn.v_proj", "attn_v"),
                       ("self_attn.o_proj", "attn_output"), ("mlp.gate_proj", "ffn_gate"), ("mlp.up_proj", "ffn_up"), ("mlp.down_proj", "ffn_down")):
            put(b + gg + ".weight", bf(sd[p + hf + ".weight"]))
        for hf, gg in (("input_layernorm", "attn_norm"), ("post_attention_layernorm", "post_attention_norm"),
                       ("self_attn.q_norm", "attn_q_norm"), ("self_attn.k_norm", "attn_k_norm")):
            put(b + gg + ".weight", norm(sd[p + hf + ".weight"]))
        put(b + "nextn.eh_proj.weight", bf(sd["mtp.fc.weight"]))
        put(b + "nextn.enorm.weight", norm(sd["mtp.pre_fc_norm_embedding.weight"]))
        put(b + "nextn.hnorm.weight", norm(sd["mtp.pre_fc_norm_hidden.weight"]))
        put(b + "nextn.shared_head_norm.weight", norm(sd["mtp.norm.weight"]))
    toks = [chr(0x100 + i) for i in range(cfg.vocab_size)]
    a = arch + "."
    kv = {"general.architecture": (8, arch), a + "block_count": (4, L + mtp), a + "embedding_length": (4, H),
          a + "attention.head_count": (4, cfg.num_attention_heads), a + "attention.head_count_kv": (4, cfg.num_key_value_heads),
          a + "attention.key_length": (4, cfg.head_dim), a + "attention.value_length": (4, cfg.head_dim),
          a + "rope.dimension_count": (4, int(cfg.head_dim * cfg.partial_rotary_factor)), a + "rope.freq_base": (6, cfg.rope_theta),
          a + "attention.layer_norm_rms_epsilon": (6, cfg.rms_norm_eps), a + "context_length": (4, 4096),
          "tokenizer.ggml.model": (8, "gpt2"), "tokenizer.ggml.tokens": (9, (8, toks)), "tokenizer.ggml.merges": (9, (8, [])),
          "tokenizer.ggml.token_type": (9, (5, [1] * cfg.vocab_size))}
    if q35:
        kv.update({a + "ssm.group_count": (4, nk), a + "ssm.time_step_rank": (4, nv), a + "ssm.state_size": (4, dk),
                   a + "ssm.inner_size": (4, nv * dv), a + "ssm.conv_kernel": (4, cfg.linear_conv_kernel_dim),
                   a + "full_attention_interval": (4, 4), a + "rope.dimension_sections": (9, (5, [11, 11, 10, 0]))})
    if mtp:
        kv[a + "nextn_predict_layers"] = (4, mtp)
    if cfg.is_moe:
        kv.update({a + "expert_count": (4, cfg.num_experts), a + "expert_used_count": (4, cfg.num_experts_per_tok),
                   a + "expert_feed_forward_length": (4, cfg.moe_intermediate_size)})
        if q35:
            kv[a + "expert_shared_feed_forward_length"] = (4, cfg.shared_expert_intermediate_size)
    if not cfg.is_moe or not q35:
        kv[a + "feed_forward_length"] = (4, cfg.intermediate_size or 512)
    _write_gguf(path, kv, tensors)


def test_value_head_order_undoes_the_converters_tiling():
    # 2 key heads x 3 value heads each: HF head key*3+j sits at stored position j*2+key
    assert gguf.v_head_order(2, 6).tolist() == [0, 2, 4, 1, 3, 5]
    assert gguf.v_head_order(2, 4, 2).tolist() == [0, 1, 4, 5, 2, 3, 6, 7]


@pytest.mark.parametrize("preset,arch", [("tiny_hybrid_dense", "qwen35"), ("tiny_hybrid_moe", "qwen35moe"), ("tiny_moe", "qwen3moe")])
def test_hybrid_family_gguf_files_load_like_their_hf_checkpoints(preset, arch, tmp_path):
    """The hybrid / MoE architecture adapters: metadata -> config, converter names -> HF names, and the converter's tensor
    transforms undone, so that a file serves the same logits as the HF directory it was converted from."""
    import dataclasses

    from grimoire_b200.api import Grimoire
    from grimoire_b200.config import EngineConfig
    from grimoire_b200.models import config as C
    from grimoire_b200.models.hybrid import HybridModel

    from .fixtures.mini_model import write_hybrid_checkpoint

    cfg = getattr(C, preset)()
    if arch == "qwen35":
        cfg = dataclasses.replace(cfg, linear_num_value_heads=6, partial_rotary_factor=0.5)      # 3 value heads per key head: the tiling is no involution
    sd = write_hybrid_checkpoint(tmp_path / "hf", cfg, seed=4, mtp=arch == "qwen35")
    path = tmp_path / "m.gguf"
    _hybrid_gguf(path, cfg, sd, arch)
    gf = gguf.GGUFFile(path)
    got = gguf.config_from_gguf(gf)
    for f in ("num_hidden_layers", "layer_types", "linear_num_key_heads", "linear_num_value_heads", "linear_key_head_dim",
              "linear_value_head_dim", "linear_conv_kernel_dim", "num_experts", "num_experts_per_tok", "moe_intermediate_size",
              "shared_expert_intermediate_size", "attn_output_gate", "norm_zero_centered", "partial_rotary_factor", "head_dim",
              "tie_word_embeddings", "vocab_size"):
        assert getattr(got, f) == getattr(cfg, f), f
    back = gguf.state_dict_from_gguf(gf, got)
    gf.close()
    pre = "model.language_model." if arch != "qwen3moe" else "model."
    for k, v in sd.items():
        if ".mlp.experts." in k:
            continue
        t = back[pre + k[len("model."):] if k.startswith("model.") else k]
        assert torch.equal(t, v.bfloat16().float().reshape(t.shape)), k       # bit-exact round trip, A_log and the norms included
    ec = lambda m: EngineConfig(model=str(m), ctx=128, seq_slots=2, prefill_chunk=32)
    ids = torch.randint(0, cfg.vocab_size, (37,), generator=torch.Generator().manual_seed(2)).tolist()
    a, b = Grimoire.load(ec(path), device="cpu"), Grimoire.load(ec(tmp_path / "hf"), device="cpu")
    assert isinstance(a.model, HybridModel) and a.tokenizer is not None
    la, lb = a.score_ids(ids), b.score_ids(ids)
    assert torch.allclose(la, lb, atol=1e-4), float((la - lb).abs().max())
    a.close()
    if arch == "qwen35":
        # the file's nextn block is the draft head: speculation keeps the plain greedy tokens
        want, _ = b.generate(ids, 12)
        c = Grimoire.load(EngineConfig(model=str(path), ctx=128, seq_slots=2, prefill_chunk=32, mtp=1), device="cpu")
        assert c.drafter is not None and got.mtp_num_hidden_layers == 1
        out, _ = c.generate(ids, 12, draft_depth=3)
        assert out == want
        c.close()
    b.close()
