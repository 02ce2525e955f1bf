"""Tool-call markup parsers and execution (rollout/generate_hub/tool_calls.py)."""
import asyncio

import pytest

from miles_b200.rollout.generate_hub.tool_calls import create_parser, execute_tool_calls

SPECS = [{"type": "function", "function": {"name": "add", "parameters": {}}}, {"type": "function", "function": {"name": "search"}}]


def test_every_markup_gives_the_same_calls():
    cases = {
        "qwen25": 'I will add.\n<tool_call>\n{"name": "add", "arguments": {"a": 1, "b": 2}}\n</tool_call>\n<tool_call>{"name": "search", "arguments": {"q": "x"}}</tool_call>',
        "llama3": 'I will add.<|python_tag|>{"name": "add", "parameters": {"a": 1, "b": 2}}; {"name": "search", "parameters": {"q": "x"}}',
        "mistral": 'I will add.[TOOL_CALLS] [{"name": "add", "arguments": {"a": 1, "b": 2}}, {"name": "search", "arguments": {"q": "x"}}]',
        "glm45": 'I will add.\n<tool_call>add\n<arg_key>a</arg_key>\n<arg_value>1</arg_value>\n<arg_key>b</arg_key>\n<arg_value>2</arg_value>\n</tool_call>\n<tool_call>search\n<arg_key>q</arg_key>\n<arg_value>x</arg_value>\n</tool_call>',
        "deepseekv3": 'I will add.<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>add\n```json\n{"a": 1, "b": 2}\n```<｜tool▁call▁end｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>search\n```json\n{"q": "x"}\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>',
    }
    for name, text in cases.items():
        plain, calls = create_parser(name, SPECS)(text)
        assert plain == "I will add.", (name, plain)
        assert [(c.name, c.arguments) for c in calls] == [("add", {"a": 1, "b": 2}), ("search", {"q": "x"})], name
        assert len({c.id for c in calls}) == 2 and all(c.error is None for c in calls)
    assert create_parser("qwen25")("no calls here") == ("no calls here", [])
    with pytest.raises(ValueError):
        create_parser("klingon")


def test_malformed_and_unknown_calls_become_error_observations():
    parse = create_parser("qwen25", SPECS)
    _, calls = parse('<tool_call>{"name": "rm_rf", "arguments": {}}</tool_call><tool_call>{"name": "add", "arguments": "not json"}</tool_call>'
                     '<tool_call>{broken</tool_call><tool_call>{"name": "add", "arguments": {"a": 2, "b": 3}}</tool_call>')
    assert [c.error is None for c in calls] == [False, False, True]  # the unterminated JSON matches nothing and swallows nothing
    seen = []

    async def execute(name, arguments):
        seen.append(name)
        if arguments.get("a") == 2:
            return str(arguments["a"] + arguments["b"])
        raise RuntimeError("boom")

    msgs = asyncio.run(execute_tool_calls(calls, execute))
    assert msgs[0]["content"].startswith("error: unknown tool") and msgs[1]["content"].startswith("error: arguments are not JSON")
    assert msgs[-1]["content"] == "5" and seen == ["add"], "only the well-formed call of a known tool runs"
    assert all(m["role"] == "tool" and m["tool_call_id"] for m in msgs)
    # a tool that raises is an observation too; a synchronous function works as well
    _, one = create_parser("hermes")('<tool_call>{"name": "add", "arguments": {"a": 1}}</tool_call>')
    assert asyncio.run(execute_tool_calls(one, execute))[0]["content"] == "error: RuntimeError: boom"
    assert asyncio.run(execute_tool_calls(one, lambda n, a: {"ok": True}))[0]["content"] == '{"ok": true}'


TOOL_SPECS = [{"type": "function", "function": {"name": "add"}}]


async def run_tool(name, arguments):
    return str(arguments["a"] + arguments["b"])


def test_multi_turn_generate_with_the_reference_flag_names():
    """--generate-execute-tool-function-path / --generate-tool-specs-path / --generate-tool-call-parser: a tool call in
    Mistral markup is executed, its result joins the context with loss mask 0, the next turn answers."""
    from types import SimpleNamespace as NS

    from miles_b200.rollout.base_types import GenerateFnInput
    from miles_b200.rollout.generate_hub import multi_turn
    from miles_b200.utils.types import Sample

    class Tok:
        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [ord(c) for c in text]}

        def decode(self, ids, **kw):
            return "".join(chr(i) for i in ids)

    texts = iter(['[TOOL_CALLS] [{"name": "add", "arguments": {"a": 2, "b": 3}}]', "the sum is 5"])
    seen = []

    class Client:
        async def generate(self, payload):
            seen.append(list(payload["input_ids"]))
            t = next(texts)
            ids = [ord(c) for c in t]
            return {"output_ids": ids, "text": t, "meta_info": {"output_token_logprobs": [(-0.5, i) for i in ids],
                                                                 "finish_reason": {"type": "stop"}, "weight_version": 1}}

    args = NS(generate_max_turns=4, generate_tool_module_path=None, generate_execute_tool_function_path="tests.test_tool_calls.run_tool",
              generate_tool_specs_path="tests.test_tool_calls.TOOL_SPECS", generate_tool_call_parser="mistral",
              generate_observation_template="[TOOL_RESULTS]{result}[/TOOL_RESULTS]", use_rollout_routing_replay=False,
              rollout_max_context_len=None)
    state = NS(args=args, client=Client(), tokenizer=Tok(), stop_strings=[])
    sample = Sample(index=0, prompt="2+3?")
    out = asyncio.run(multi_turn.generate(GenerateFnInput(state=state, sample=sample, sampling_params={"max_new_tokens": 256},
                                                          evaluation=False))).samples
    text = "".join(chr(i) for i in out.tokens)
    assert text.endswith('[TOOL_RESULTS]5[/TOOL_RESULTS]the sum is 5') and out.metadata["turns"] == 2
    obs = len("[TOOL_RESULTS]5[/TOOL_RESULTS]")
    assert out.loss_mask.count(0) == obs and len(out.loss_mask) == out.response_length == len(out.rollout_log_probs)
    assert "".join(chr(i) for i in seen[1]).endswith("[TOOL_RESULTS]5[/TOOL_RESULTS]"), "the second turn saw the observation"
