"""C++ byte-level BPE against the HF `tokenizers` library on a BPE trained offline with the Qwen2
pre-tokenizer pattern (the reference checks its tokenizer against HF goldens,
tests/tokenizer_golden/; no pretrained tokenizer files exist on this machine, so the oracle is the
library itself on a freshly trained vocabulary)."""
import json

import pytest

tokenizers = pytest.importorskip("tokenizers")
from tokenizers import Regex, Tokenizer as HFTok, decoders, models, normalizers, pre_tokenizers, trainers  # noqa: E402

from grimoire_b200.tokenizer import Tokenizer, render_chatml  # noqa: E402

PAT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")
CORPUS = [
    "Hello, world! 123 The quick brown fox jumps over the lazy dog. It's we're they'll I'd DON'T",
    "def main():\n    print('hi')\n\n\treturn 0  # comment\r\n", "café cafè naïve Ünïcödé straße ΑΒΓ абв",
    "你好，世界！ こんにちは 세계 مرحبا بالعالم שלום", "12345 3.14159 1,000,000 ١٢٣ ②③", "a  b   c    d\n\n\ne \t f", "emoji 🙂🙃 → ∑ ≠ ≤ «quoted» …",
] * 4


@pytest.fixture(scope="module")
def toks(tmp_path_factory):
    hf = HFTok(models.BPE())
    hf.normalizer = normalizers.NFC()
    hf.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(PAT), behavior="isolated", invert=False),
                                                pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    hf.decoder = decoders.ByteLevel()
    tr = trainers.BpeTrainer(vocab_size=700, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                             initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    hf.train_from_iterator(CORPUS, tr)
    d = tmp_path_factory.mktemp("tok")
    hf.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|im_end|>"}))
    return hf, Tokenizer(d)


CASES = CORPUS[:7] + [
    "", " ", "  ", "\n", " \n ", "x", "Hello   world  ", "tabs\t\tand  spaces \n\n  mixed\r\n\r\nend ",
    "It's 'S 'RE we'Ve you'LL", "price: $1,234.56!!! (approx.)", "   leading and trailing   ", "á è combining",
    "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n", "mixed汉字and English混排123", " line sep nbsp　ideographic",
]


@pytest.mark.parametrize("text", CASES)
def test_encode_matches_hf(toks, text):
    hf, ours = toks
    want = hf.encode(text).ids
    got = ours.encode(text)
    assert got == want, (text, got, want)
    assert ours.decode(got, skip_special=False) == hf.decode(want, skip_special_tokens=False)


def test_specials_and_eos(toks):
    hf, ours = toks
    assert ours.special_id("<|im_end|>") == hf.token_to_id("<|im_end|>")
    assert ours.eos() == hf.token_to_id("<|im_end|>") and ours.eos2() == hf.token_to_id("<|endoftext|>")
    ids = ours.encode("a<|im_end|>b")
    assert hf.token_to_id("<|im_end|>") in ids
    assert hf.token_to_id("<|im_end|>") not in ours.encode("a<|im_end|>b", allow_special=False)
    assert ours.decode(ids, skip_special=True) == "ab"
    assert ours.template_kind() == "chatml"


def test_chatml_template_with_tools_and_thinking_switch():
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "weather?"},
            {"role": "assistant", "content": "", "tool_calls": [{"type": "function", "function": {"name": "get", "arguments": "{\"c\": \"x\"}"}}]},
            {"role": "tool", "content": "sunny"}]
    tools = [{"type": "function", "function": {"name": "get", "parameters": {}}}]
    s = render_chatml(msgs, tools, True, enable_thinking=False)
    assert s.startswith("<|im_start|>system\nbe brief\n\n# Tools")
    assert "<tool_call>\n{\"name\": \"get\", \"arguments\": {\"c\": \"x\"}}\n</tool_call><|im_end|>" in s
    assert "<|im_start|>user\n<tool_response>\nsunny\n</tool_response><|im_end|>\n" in s
    assert s.endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    plain = render_chatml([{"role": "user", "content": "hi"}])
    assert plain == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
