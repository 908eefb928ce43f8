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


def test_family_turn_formats():
    """Gemma-4, Muse-Glimmer and K2-Horizon turn formats, string for string."""
    from grimoire_b200.tokenizer import render_gemma4, render_k2, render_muse

    msgs = [{"role": "system", "content": " be brief \n"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": " yo "},
            {"role": "user", "content": "again"}]
    assert render_gemma4(msgs) == ("<|turn>system\nbe brief<turn|>\n<|turn>user\nhi<turn|>\n<|turn>model\nyo<turn|>\n<|turn>user\nagain<turn|>\n"
                                   "<|turn>model\n<|channel>thought\n<channel|>")
    assert render_gemma4(msgs[1:2], thinking=True) == "<|turn>system\n<|think|>\n<turn|>\n<|turn>user\nhi<turn|>\n<|turn>model\n"
    assert render_gemma4(msgs[1:2]) == "<|turn>user\nhi<turn|>\n<|turn>model\n<|channel>thought\n<channel|>"
    with pytest.raises(ValueError):
        render_gemma4([{"role": "tool", "content": "x"}])
    meta = "\n\nReasoning strength: high.\n\n# Valid recipients: \"self\", \"user\"."
    assert render_muse(msgs[1:3], today="2026-03-01") == (
        "<|begin_of_text|><|start|>system<|message|>You are a helpful AI assistant.\nKnowledge cutoff: 2026-01-04.\nCurrent date: 2026-03-01."
        + meta + "<|eot|><|start|>user<|message|>hi<|eot|><|start|>assistant to=user<|message|> yo <|eot|><|start|>assistant")
    assert render_muse(msgs[:2]) == ("<|begin_of_text|><|start|>system<|message|> be brief \n" + meta + "<|eot|><|start|>user<|message|>hi<|eot|>"
                                     "<|start|>assistant")
    assert render_k2(msgs[1:]) == ("<|ifm|begin_of_text|><|ifm|im_start|>user\nhi<|ifm|im_end|><|ifm|im_start|>assistant<ifm|think>\n</ifm|think> yo "
                                   "<|ifm|im_end|><|ifm|im_start|>user\nagain<|ifm|im_end|><|ifm|im_start|>assistant\n<ifm|think>\n")


def test_xml_tool_template_family(toks, tmp_path):
    """The Qwen XML-tool template: recognised from the checkpoint's own Jinja text, rendered line for line -- effort line,
    tools block, past turns with their think block, function / parameter tool calls, grouped tool results."""
    import shutil

    from grimoire_b200.tokenizer import EFFORT_LOW, EFFORT_XHIGH, XML_TOOL_INSTRUCTIONS, render_chatml_xml

    _, plain = toks
    assert plain.chat_family() == {"xml_tools": False, "effort": False, "think_split": False, "default_effort": "xhigh"}
    shutil.copy(plain.dir / "tokenizer.json", tmp_path / "tokenizer.json")
    jinja = ("{%- set effort = reasoning_effort | default('low') %} multi_step_tool=true <function=example_function_name> "
             "do not tell the user about function calls Reasoning effort is set to xhigh. content.split('</think>')")
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|im_end|>", "chat_template": jinja}))
    tok = Tokenizer(tmp_path)
    fam = tok.chat_family()
    assert fam == {"xml_tools": True, "effort": True, "think_split": True, "default_effort": "low"} and tok.template_kind() == "chatml_xml"
    msgs = [{"role": "system", "content": "S"}, {"role": "user", "content": "weather?"},
            {"role": "assistant", "content": "<think>\nhm\n</think>\n\nlet me look",
             "tool_calls": [{"function": {"name": "w", "arguments": "{\"city\": \"Paris\", \"days\": [1, 2]}"}}, {"function": {"name": "t", "arguments": {}}}]},
            {"role": "tool", "content": "sunny"}, {"role": "tool", "content": "18C"}]
    tools = [{"type": "function", "function": {"name": "w"}}]
    s = tok.apply_chat_template(msgs, tools=tools)
    assert s.startswith("<|im_start|>system\n" + EFFORT_LOW + "\n\n# Tools\n\nYou have access to the following functions:\n\n<tools>\n"
                        + json.dumps(tools[0]) + "\n</tools>" + XML_TOOL_INSTRUCTIONS + "\n\nS<|im_end|>\n<|im_start|>user\nweather?<|im_end|>\n")
    assert ("<|im_start|>assistant\n<think>\nhm\n</think>\n\nlet me look\n\n<tool_call>\n<function=w>\n<parameter=city>\nParis\n</parameter>\n"
            "<parameter=days>\n[1, 2]\n</parameter>\n</function>\n</tool_call>\n<tool_call>\n<function=t>\n</function>\n</tool_call><|im_end|>\n") in s
    assert s.endswith("<|im_start|>user\n<tool_response>\nsunny\n</tool_response>\n<tool_response>\n18C\n</tool_response><|im_end|>\n"
                      "<|im_start|>assistant\n<think>\n")
    # effort choices: "high" is the template's xhigh, medium writes nothing, thinking off drops the line and closes the block
    hi = tok.apply_chat_template(msgs[1:2], reasoning_effort="high")
    assert hi == "<|im_start|>system\n" + EFFORT_XHIGH + "<|im_end|>\n<|im_start|>user\nweather?<|im_end|>\n<|im_start|>assistant\n<think>\n"
    assert tok.apply_chat_template(msgs[1:2], reasoning_effort="medium") == "<|im_start|>user\nweather?<|im_end|>\n<|im_start|>assistant\n<think>\n"
    assert tok.apply_chat_template(msgs[1:2], enable_thinking=False).endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    with pytest.raises(ValueError, match="Unexpected reasoning effort"):
        tok.apply_chat_template(msgs[1:2], reasoning_effort="max")
    with pytest.raises(ValueError, match="No user query"):
        render_chatml_xml([{"role": "user", "content": "<tool_response>x</tool_response>"}])
    with pytest.raises(ValueError, match="beginning"):
        render_chatml_xml([{"role": "user", "content": "q"}, {"role": "system", "content": "late"}])
    # a first tool call after an empty answer follows the think block directly
    empty = render_chatml_xml([{"role": "user", "content": "q"}, {"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "f", "arguments": {"a": 1}}}]}])
    assert "<think>\n\n</think>\n\n<tool_call>\n<function=f>\n<parameter=a>\n1\n</parameter>\n</function>\n</tool_call><|im_end|>" in empty


@pytest.mark.parametrize("specials,kind", [(["<bos>", "<|turn>", "<turn|>", "<|channel>", "<channel|>"], "gemma4"),
                                           (["<|begin_of_text|>", "<|start|>", "<|message|>", "<|eot|>"], "muse"),
                                           (["<|ifm|begin_of_text|>", "<|ifm|im_start|>", "<|ifm|im_end|>"], "k2")])
def test_template_kind_follows_the_checkpoints_special_tokens(tmp_path, specials, kind):
    hf = HFTok(models.BPE())
    hf.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(PAT), behavior="isolated", invert=False),
                                                pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    hf.decoder = decoders.ByteLevel()
    hf.train_from_iterator(CORPUS, trainers.BpeTrainer(vocab_size=400, special_tokens=specials, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                                       show_progress=False))
    hf.save(str(tmp_path / "tokenizer.json"))
    tok = Tokenizer(tmp_path)
    assert tok.template_kind() == kind
    ids = tok.encode_chat([{"role": "user", "content": "Hello"}], enable_thinking=False)
    first = hf.token_to_id(specials[0])
    assert ids[0] == first and ids.count(first) == 1               # BOS once: added for gemma4, part of the template for the others
    text = tok.apply_chat_template([{"role": "user", "content": "Hello"}], enable_thinking=False)
    assert tok.decode(ids, skip_special=False).endswith(text[-12:])
    with pytest.raises(ValueError, match="tool-call"):
        tok.apply_chat_template([{"role": "user", "content": "x"}], tools=[{"type": "function"}])
