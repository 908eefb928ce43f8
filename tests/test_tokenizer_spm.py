"""SentencePiece-style BPE ``tokenizer.json`` (Llama / Gemma flavour): space marker, merges over the whole segment, byte
fallback, special tokens, round trip (src/tokenizer.cpp:427, :1627 in the reference)."""
import json

import pytest

from grimoire_b200.tokenizer import Tokenizer
from grimoire_b200.tokenizer_spm import SPACE, SpmBpe, is_spm_bpe


def _meta(prepend: bool):
    pieces = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)]
    chars = [SPACE, "h", "e", "l", "o", "w", "r", "d", ",", "a", "b"]
    merged = ["he", "ll", "hell", "hello", SPACE + "w", "or", SPACE + "wor", "ld", SPACE + "world", SPACE + "hello", "ab", "abab"]
    vocab = {t: i for i, t in enumerate(pieces + chars + merged)}
    merges = [["h", "e"], ["l", "l"], ["he", "ll"], ["hell", "o"], [SPACE, "w"], ["o", "r"], [SPACE + "w", "or"], ["l", "d"],
              [SPACE + "wor", "ld"], [SPACE, "hello"], ["a", "b"], ["ab", "ab"]]
    norm = [{"type": "Prepend", "prepend": SPACE}] if prepend else []
    norm.append({"type": "Replace", "pattern": {"String": " "}, "content": SPACE})
    return {"model": {"type": "BPE", "vocab": vocab, "merges": merges, "byte_fallback": True, "unk_token": "<unk>"},
            "normalizer": {"type": "Sequence", "normalizers": norm}, "pre_tokenizer": None,
            "added_tokens": [{"id": 1, "content": "<s>", "special": True}, {"id": 2, "content": "</s>", "special": True}]}


def test_spm_bpe_merges_space_marker_and_byte_fallback():
    meta = _meta(prepend=True)
    assert is_spm_bpe(meta)
    t = SpmBpe(meta)
    ids = t.encode("hello world")
    assert [t.inv[i] for i in ids] == [SPACE + "hello", SPACE + "world"]            # dummy prefix + whole-segment merges
    assert t.decode_bytes(ids).decode() == "hello world"
    # a character outside the vocabulary becomes its UTF-8 bytes; decode puts it back
    ids = t.encode("héllo")
    names = [t.inv[i] for i in ids]
    assert "<0xC3>" in names and "<0xA9>" in names and t.decode_bytes(ids).decode() == "héllo"
    # special tokens split the text and are not merged into; skip_special drops them on decode
    ids = t.encode("<s>abab</s>")
    assert ids[0] == 1 and ids[-1] == 2 and [t.inv[i] for i in ids[1:-1]] == [SPACE, "abab"]
    assert t.decode_bytes(ids).decode() == "abab" and "<s>" in t.decode_bytes(ids, skip_special=False).decode()
    # merges are rank ordered, not left to right: "ababab" -> abab + ab
    assert [t.inv[i] for i in t.encode("ababab")][1:] == ["abab", "ab"]
    # long inputs stay cheap (heap ordered merges)
    long = "hello world " * 2000
    assert t.decode_bytes(t.encode(long)).decode() == long


def test_spm_tokenizer_json_loads_through_the_front_end(tmp_path):
    (tmp_path / "tokenizer.json").write_text(json.dumps(_meta(prepend=False)))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"eos_token": "</s>"}))
    tok = Tokenizer(tmp_path)
    ids = tok.encode("hello world")
    assert tok.decode(ids) == "hello world" and tok.eos() == 2 and tok.is_special(2) and not tok.is_special(ids[0])
    assert tok.special_id("<s>") == 1 and tok.vocab_size > 256


def test_byte_level_tokenizer_json_is_not_taken_for_spm():
    meta = {"model": {"type": "BPE", "vocab": {}, "merges": []}, "pre_tokenizer": {"type": "ByteLevel"}, "normalizer": None}
    assert not is_spm_bpe(meta)


def test_gguf_sentencepiece_tokenizers(tmp_path):
    """GGUF ``llama`` (scores, no merges, space prefix) and ``gemma4`` (merges, no prefix) tokenizers through the GGUF
    adapter: pieces merge best score first, unknown characters fall back to bytes, BOS is added when the file says so."""
    import json

    from grimoire_b200.formats import gguf as G
    from grimoire_b200.tokenizer import Tokenizer

    from .test_gguf import _write_gguf

    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "h", "e", "l", "o", "he", "ll", "hell", "hello", "▁hello", "▁h", "w"]
    scores = [0.0] * 259 + [-1.0, -2.0, -2.0, -2.0, -2.0, -5.0, -4.0, -3.5, -3.0, -2.5, -6.0, -2.0]
    types = [2, 3, 3] + [6] * 256 + [1] * 12
    kv = {"general.architecture": (8, "llama"), "tokenizer.ggml.model": (8, "llama"), "tokenizer.ggml.tokens": (9, (8, toks)),
          "tokenizer.ggml.token_type": (9, (5, types)), "tokenizer.ggml.bos_token_id": (4, 1), "tokenizer.ggml.eos_token_id": (4, 2),
          "tokenizer.ggml.unknown_token_id": (4, 0), "tokenizer.ggml.scores": (9, (6, scores)), "tokenizer.ggml.add_bos_token": (7, True)}
    path = tmp_path / "t.gguf"
    _write_gguf(path, kv, {})
    g = G.GGUFFile(path)
    tj, tc = G.tokenizer_json_from_gguf(g), G.tokenizer_config_from_gguf(g)
    g.close()
    assert tj["model"]["scores"][267] == -3.0 and tc == {"bos_token": "<s>", "eos_token": "</s>", "add_bos_token": True}
    d = tmp_path / "tok"
    d.mkdir()
    (d / "tokenizer.json").write_text(json.dumps(tj))
    (d / "tokenizer_config.json").write_text(json.dumps(tc))
    tok = Tokenizer(d)
    v = {t: i for i, t in enumerate(toks)}
    assert tok.encode("hello") == [v["▁hello"]]                                  # a space is prepended, the best piece wins
    assert tok.encode("hello hewo") == [v["▁hello"], v["▁"], v["he"], v["w"], v["o"]]      # "he" (-5) merges before "▁h" (-6)
    assert tok.encode("hé") == [v["▁h"], v["<0xC3>"], v["<0xA9>"]]            # byte fallback
    assert tok.decode(tok.encode("hello hé")) == "hello hé"
    assert tok.bos() == 1 and tok.add_bos and tok.encode_chat([{"role": "user", "content": "hello"}])[0] == 1
    # gemma4 flavour: merges instead of scores, no space prefix
    g2 = G.GGUFFile(path)
    g2.metadata.update({"tokenizer.ggml.model": "gemma4", "tokenizer.ggml.merges": ["h e", "l l", "he ll", "hell o", "▁ hello"]})
    tj2 = G.tokenizer_json_from_gguf(g2)
    g2.metadata["tokenizer.ggml.add_space_prefix"] = True
    with pytest.raises(ValueError, match="add_space_prefix"):
        G.tokenizer_json_from_gguf(g2)
    g2.close()
    (d / "tokenizer.json").write_text(json.dumps(tj2))
    tok2 = Tokenizer(d)
    assert tok2.encode("hello hello") == [v["hello"], v["▁hello"]]
