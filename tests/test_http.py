"""Request validation and response decoding (tier T2; tests/test_http.cpp in the reference)."""
import json

import pytest

from grimoire_b200.http_request import BadRequest, ResponseDecoder, parse_completion_request, parse_xml_tool_calls


def test_defaults_and_aliases():
    r = parse_completion_request({"messages": [{"role": "user", "content": "hi"}]}, chat=True)
    assert r.max_tokens == 4096 and r.sampling.top_k == 20 and r.sampling.greedy and not r.stream and r.enable_thinking
    r = parse_completion_request({"prompt": "x", "max_completion_tokens": 7, "temperature": 0.5, "top_k": 5, "seed": 3}, chat=False)
    assert r.max_tokens == 7 and not r.sampling.greedy and r.sampling.seed == 3


@pytest.mark.parametrize("body", [
    {"messages": []}, {"messages": [{"role": "robot", "content": "x"}]}, {"messages": [{"role": "user", "content": "x"}], "n": 2},
    {"messages": [{"role": "user", "content": "x"}], "stop": ["a"]}, {"messages": [{"role": "user", "content": "x"}], "logprobs": True},
    {"messages": [{"role": "user", "content": "x"}], "response_format": {"type": "json_object"}},
    {"messages": [{"role": "user", "content": "x"}], "presence_penalty": 0.5}, {"messages": [{"role": "user", "content": "x"}], "top_k": 65},
    {"messages": [{"role": "user", "content": "x"}], "top_k": 0}, {"messages": [{"role": "user", "content": "x"}], "top_p": 0},
    {"messages": [{"role": "user", "content": "x"}], "tool_choice": "required"}, {"messages": [{"role": "user", "content": "x"}], "max_tokens": 0},
    {"messages": [{"role": "user", "content": "x"}], "temperature": "hot"},
])
def test_rejections(body):
    with pytest.raises(BadRequest):
        parse_completion_request(body, chat=True)
    with pytest.raises(BadRequest):
        parse_completion_request({"prompt": ""}, chat=False)


def test_tools_and_thinking_switch():
    tools = [{"type": "function", "function": {"name": "f"}}]
    r = parse_completion_request({"messages": [{"role": "user", "content": "x"}], "tools": tools, "tool_choice": "none",
                                  "chat_template_kwargs": {"enable_thinking": False}, "reasoning_effort": "low"}, chat=True)
    assert r.tools is None and not r.enable_thinking and r.reasoning_effort == "low"


def test_tool_call_parsing_json_and_xml_forms():
    text = 'Let me check.  \n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>'
    content, calls = parse_xml_tool_calls(text)
    assert content == "Let me check." and len(calls) == 1
    assert calls[0]["function"]["name"] == "get_weather" and json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris"}
    assert calls[0]["id"].startswith("call_") and len(calls[0]["id"]) == 21
    xml = "<tool_call>\n<function=search>\n<parameter=q>\nblackwell\n</parameter>\n<parameter=n>\n3\n</parameter>\n</function>\n</tool_call>"
    _, calls = parse_xml_tool_calls(xml)
    assert calls[0]["function"]["name"] == "search" and json.loads(calls[0]["function"]["arguments"]) == {"q": "blackwell", "n": 3}


def test_response_decoder_splits_think_and_holds_tool_calls_across_pieces():
    d = ResponseDecoder(thinking=True, tools=True, starts_in_think=True)
    pieces = ["I should", " greet.</th", "ink>\n\nHello", " there <tool_", 'call>{"name":"f","arg', 'uments":{}}</tool_call>']
    ev = []
    for p in pieces:
        ev += d.push(p)
    tail, calls = d.finish()
    ev += tail
    assert "".join(t for k, t in ev if k == "reasoning") == "I should greet."
    assert "".join(t for k, t in ev if k == "content") == "Hello there "
    assert len(calls) == 1 and calls[0]["function"]["name"] == "f"
    assert d.content == "Hello there"
