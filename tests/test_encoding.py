"""Chat encodings and the GGUF BPE tokenizer."""
import json
import os

import pytest

from deepseek_v4_2080ti_b200 import encoding
from deepseek_v4_2080ti_b200.encoding import deepseek_v4 as dsv4
from deepseek_v4_2080ti_b200.encoding.gguf_tokenizer import TOKEN_CONTROL, TOKEN_NORMAL, GGUFTokenizer, _byte_maps

TOOLS = [{"type": "function", "function": {"name": "get_weather", "description": "Weather lookup",
                                           "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]


def test_deepseek_chat_mode_and_thinking_mode_prompts():
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hi"}]
    chat = dsv4.render(msgs)
    assert chat == dsv4.BOS + "Be brief." + dsv4.USER + "Hi" + dsv4.ASSISTANT + dsv4.THINK_CLOSE
    think = dsv4.render(msgs, thinking=True, reasoning_effort="high")
    assert think.startswith(dsv4.BOS + "Reasoning Effort: Absolute maximum") and think.endswith(dsv4.ASSISTANT + dsv4.THINK_OPEN)
    assert dsv4.render(msgs, thinking=True, reasoning_effort="medium") == dsv4.render(msgs, thinking=True)
    with pytest.raises(ValueError):
        dsv4.render(msgs, thinking=True, reasoning_effort="extreme")


def test_deepseek_tool_round_trip_and_result_ordering():
    calls = [{"id": "a", "type": "function", "function": {"name": "get_weather", "arguments": json.dumps({"city": "Oslo", "days": 2})}},
             {"id": "b", "type": "function", "function": {"name": "get_weather", "arguments": json.dumps({"city": "Rome"})}}]
    msgs = [{"role": "user", "content": "Compare"},
            {"role": "assistant", "reasoning_content": "two lookups", "content": "", "tool_calls": calls},
            {"role": "tool", "tool_call_id": "b", "content": "sunny"}, {"role": "tool", "tool_call_id": "a", "content": "rain"}]
    p = dsv4.render(msgs, tools=TOOLS, thinking=True)
    assert "## Tools" in p and '"name": "get_weather"' in p
    # results are re-ordered like the calls, inside one user turn
    assert dsv4.USER + "<tool_result>rain</tool_result>\n\n<tool_result>sunny</tool_result>" + dsv4.ASSISTANT + dsv4.THINK_OPEN in p
    assert '<｜DSML｜parameter name="days" string="false">2</｜DSML｜parameter>' in p
    # parse the assistant turn back out of the prompt
    start = p.index(dsv4.ASSISTANT + dsv4.THINK_OPEN) + len(dsv4.ASSISTANT + dsv4.THINK_OPEN)
    parsed = dsv4.parse_completion(p[start:p.index(dsv4.EOS, start)], thinking=True)
    assert parsed["reasoning_content"] == "two lookups" and parsed["content"] == ""
    assert [json.loads(c["function"]["arguments"]) for c in parsed["tool_calls"]] == [{"city": "Oslo", "days": 2}, {"city": "Rome"}]


def test_deepseek_earlier_reasoning_is_dropped_without_tools():
    msgs = [{"role": "user", "content": "a"}, {"role": "assistant", "reasoning_content": "SECRET", "content": "b"},
            {"role": "user", "content": "c"}]
    p = dsv4.render(msgs, thinking=True)
    assert "SECRET" not in p and p.endswith(dsv4.USER + "c" + dsv4.ASSISTANT + dsv4.THINK_OPEN)


@pytest.mark.parametrize("case,thinking", [(1, True), (2, True), (3, True), (4, False)])
def test_deepseek_matches_reference_golden_files(case, thinking):
    # golden prompt files of the reference project (tests/fixtures/encoding there): looked for beside this repository
    # or where POCKETLLM_REFERENCE_DIR points
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    roots = [os.environ.get("POCKETLLM_REFERENCE_DIR", ""), os.path.join(os.path.dirname(here), "reference")]
    base = next((os.path.join(r, "tests", "fixtures", "encoding") for r in roots
                 if r and os.path.exists(os.path.join(r, "tests", "fixtures", "encoding", f"test_input_{case}.json"))), None)
    if base is None:
        pytest.skip("reference fixtures not mounted")
    data = json.load(open(f"{base}/test_input_{case}.json"))
    tools = None
    if isinstance(data, dict):
        tools, data = data["tools"], data["messages"]
    assert dsv4.render(data, tools=tools, thinking=thinking, add_generation_prompt=False) == open(f"{base}/test_output_{case}.txt").read()


def test_glm_and_minimax_framing():
    msgs = [{"role": "system", "content": "S"}, {"role": "user", "content": "U"}]
    g = encoding.render_chat("glm_dsa", msgs)
    assert g == "[gMASK]<sop><|system|>\nS<|user|>\nU<|assistant|>\n<think></think>\n"
    assert encoding.render_chat("glm_dsa", msgs, thinking=True).endswith("<|assistant|>\n<think>")
    m = encoding.render_chat("minimax_m2", msgs, thinking=True)
    assert m == "]~!b[]~b]system\nS[e~[\n]~b]user\nU[e~[\n]~b]ai\n<think>\n"
    out = encoding.parse_completion("glm_dsa", "why</think>ok<tool_call>f\n<arg_key>x</arg_key>\n<arg_value>3</arg_value>\n</tool_call>")
    assert out["reasoning_content"] == "why" and out["content"] == "ok"
    assert json.loads(out["tool_calls"][0]["function"]["arguments"]) == {"x": 3}
    assert encoding.family_from_architecture("glm-dsa") == "glm_dsa" and encoding.family_from_architecture("minimax-m2") == "minimax_m2"
    with pytest.raises(ValueError):
        encoding.render_chat("llama", msgs)


def _toy_tokenizer():
    enc, _ = _byte_maps()
    base = [enc[b] for b in range(256)]
    merges = ["h e", "l l", "he ll", "hell o", "Ġ w", "o r", "Ġw or", "Ġwor l", "Ġworl d"]
    toks = base + ["he", "ll", "hell", "hello", "Ġw", "or", "Ġwor", "Ġworl", "Ġworld", "<|eos|>", "<|user|>"]
    types = [TOKEN_NORMAL] * (len(toks) - 2) + [TOKEN_CONTROL, TOKEN_CONTROL]
    return GGUFTokenizer(toks, merges, types, eos_id=len(toks) - 2)


def test_gguf_bpe_tokenizer_merges_specials_and_round_trip():
    tk = _toy_tokenizer()
    ids = tk.encode("hello world")
    assert [tk.tokens[i] for i in ids] == ["hello", "Ġworld"]
    ids = tk.encode("<|user|>hello<|eos|>")
    assert ids[0] == tk.vocab["<|user|>"] and ids[-1] == tk.eos_id and len(ids) == 3
    assert tk.decode(ids) == "hello" and tk.decode(ids, skip_special=False) == "<|user|>hello<|eos|>"
    text = "héllo wörld — ok 123\n"
    assert tk.decode(tk.encode(text)) == text
    assert tk.eos_ids == {tk.eos_id}


def test_gguf_tokenizer_from_file(tmp_path):
    from deepseek_v4_2080ti_b200.formats import gguf as G
    import torch
    tk = _toy_tokenizer()
    G.write_gguf(str(tmp_path / "t.gguf"), {"general.architecture": "minimax-m2", "tokenizer.ggml.model": "gpt2",
                                            "tokenizer.ggml.tokens": tk.tokens, "tokenizer.ggml.token_type": tk.types,
                                            "tokenizer.ggml.merges": [" ".join(k) for k in tk.ranks],
                                            "tokenizer.ggml.eos_token_id": tk.eos_id},
                 [("x", G.quantize(torch.zeros(1, 32), G.GGMLType.F32), G.GGMLType.F32, (1, 32))])
    t2 = GGUFTokenizer.from_gguf(str(tmp_path / "t.gguf"))
    assert t2.encode("hello world") == tk.encode("hello world")
