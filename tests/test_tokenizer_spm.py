"""SentencePiece-style BPE ``tokenizer.json`` (Llama / Gemma flavour): space marker, merges over the whole segment, byte
fallback, special tokens, round trip (src/tokenizer.cpp:427, :1627 in the reference)."""
import json

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
