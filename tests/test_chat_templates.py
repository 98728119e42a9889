"""Chat templates, tool-call parsers, the streaming output parser and grammar constraints (CPU only)."""
import json
import random

from cuteafd_b200.loader.tokenizer import ByteTokenizer
from cuteafd_b200.serving.chat_templates import parse_completion, template_for
from cuteafd_b200.serving.constraints import ChoiceConstraint, JsonConstraint, JsonPrefix, constraint_from_request, unpack_bits

TOOLS = [{"type": "function", "function": {"name": "get_weather", "description": "weather", "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]
HISTORY = [{"role": "system", "content": "be terse"}, {"role": "user", "content": "weather in Oslo?"},
           {"role": "assistant", "content": "<think>need the tool</think>\n\nLet me check.",
            "tool_calls": [{"id": "c1", "type": "function", "function": {"name": "get_weather", "arguments": "{\"city\": \"Oslo\"}"}}]},
           {"role": "tool", "tool_call_id": "c1", "content": "-3C"}, {"role": "user", "content": "and Bergen?"}]


def test_templates_render_roles_tools_and_drop_old_reasoning():
    q = template_for("qwen3-235b").render(HISTORY, tools=TOOLS, thinking=True)
    assert q.startswith("<|im_start|>system\nbe terse") and "<tools>" in q and '"name": "get_weather"' in q
    assert "need the tool" not in q and "Let me check." in q and "<tool_response>\n-3C\n</tool_response>" in q
    assert q.endswith("<|im_start|>assistant\n<think>\n") and q.count("<|im_start|>user") == 3
    d = template_for("deepseek-v3").render(HISTORY, tools=TOOLS)
    assert d.startswith("<｜begin▁of▁sentence｜>be terse") and "<｜tool▁call▁begin｜>function<｜tool▁sep｜>get_weather" in d
    assert "<｜tool▁output▁begin｜>-3C<｜tool▁output▁end｜>" in d and d.endswith("<｜Assistant｜>") and "need the tool" not in d
    g = template_for("glm-5").render(HISTORY, tools=TOOLS)
    assert g.startswith("[gMASK]<sop>") and "<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Oslo</arg_value>" in g and "<|observation|>" in g
    c = template_for("qwen3-coder").render(HISTORY, tools=TOOLS)
    assert "<function=get_weather>\n<parameter=city>\nOslo\n</parameter>" in c
    assert template_for("something-else").render([{"role": "user", "content": "x"}]) == "<|user|>\nx\n<|assistant|>\n"


CASES = [
    ("qwen3-235b", "<think>\nplan\n</think>\n\nSure.\n<tool_call>\n{\"name\": \"get_weather\", \"arguments\": {\"city\": \"Oslo\"}}\n</tool_call><|im_end|>junk", True),
    ("qwen3-coder", "<tool_call>\n<function=get_weather>\n<parameter=city>\nOslo\n</parameter>\n</function>\n</tool_call>", False),
    ("glm-5", "Checking.<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Oslo</arg_value>\n</tool_call>", False),
    ("deepseek-v3", "ok<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>get_weather\n```json\n{\"city\": \"Oslo\"}\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>", False),
]


def test_tool_calls_parse_in_every_family_and_streaming_agrees_with_whole_text():
    for model, text, has_reasoning in CASES:
        t = template_for(model)
        whole = parse_completion(t, text)
        assert [(c["name"], c["arguments"]) for c in whole["tool_calls"]] == [("get_weather", {"city": "Oslo"})], model
        assert bool(whole["reasoning"]) == has_reasoning and "junk" not in whole["content"]
        # the same text pushed in random pieces gives the same events, and never leaks a partial tag
        cut = text.split("<|im_end|>")[0]
        for seed in range(5):
            rng, p, ev, i = random.Random(seed), t.parser(), [], 0
            while i < len(cut):
                n = rng.randrange(1, 7)
                ev += p.push(cut[i:i + n])
                i += n
            ev += p.finish()
            content = "".join(x for k, x in ev if k == "content")
            assert "<tool_call" not in content and "<think" not in content and "tool▁call▁begin" not in content
            assert [c[1]["name"] for c in ev if c[0] == "tool_call"] == ["get_weather"]
            assert "".join(x for k, x in ev if k == "reasoning") == whole["reasoning"]
    broken = parse_completion(template_for("qwen3"), "text <tool_call>\nnot json\n</tool_call> more")
    assert broken["tool_calls"] == [] and "not json" in broken["content"]          # an unparsable call stays visible as text


def test_json_prefix_automaton():
    for s in ['{"a": [1, 2.5e-3, true, null, "x\\n\\u00e9"], "b": {}}', "[]", "-0.5", '"hi"', " { } ", "[[],{}]", "1E+9"]:
        p = JsonPrefix()
        assert p.feed_text(s) and p.complete, s
        json.loads(s)
    for s in ["{a", "[1,]", "01", '{"a" 1', "1.e", "tru e", '{"a":1}}', "[1 2]", '{"a":}', '"\\x"', "-", "[1,", '{"a"']:
        p = JsonPrefix()
        assert not (p.feed_text(s) and p.complete), s
    assert not JsonPrefix("object").feed_text("[") and JsonPrefix("array").feed_text("[1")


def test_json_constraint_keeps_a_random_walk_inside_json():
    tok, rng = ByteTokenizer(), random.Random(0)
    finished = 0
    for trial in range(12):
        c, toks = JsonConstraint(tok, 258, 3, eos_id=257, top="object"), [1, 2, 3]
        for _ in range(300):
            allowed = [i for i, a in enumerate(unpack_bits(c.mask(toks), 258)) if a]
            assert allowed
            closers = [a for a in allowed if a in (257, ord("}"), ord("]"), ord('"'))]
            toks.append(rng.choice(closers) if closers and rng.random() < 0.4 else rng.choice(allowed))
            if toks[-1] == 257:
                break
        text = tok.decode([t for t in toks[3:] if t != 257])
        assert JsonPrefix("object").feed_text(text)
        if toks[-1] == 257:
            assert isinstance(json.loads(text), dict)
            finished += 1
    assert finished >= 6
    # a rolled-back speculative tail is replayed from the start
    c = JsonConstraint(tok, 258, 0, eos_id=257)
    c.mask(list(b'{"a"'))
    assert ord(":") in [i for i, a in enumerate(unpack_bits(c.mask(list(b'{"a"')), 258)) if a]
    assert ord('"') in [i for i, a in enumerate(unpack_bits(c.mask(list(b"{")), 258)) if a]


def test_choice_constraint_and_response_format_mapping():
    tok = ByteTokenizer()
    ch, t = ChoiceConstraint(tok, 258, 0, ["get_weather", "get_time"], eos_id=257), []
    for _ in range(20):
        al = [i for i, a in enumerate(unpack_bits(ch.mask(t), 258)) if a]
        t.append(al[0])
        if t[-1] == 257:
            break
    assert tok.decode(t[:-1]) in ("get_weather", "get_time") and t[-1] == 257
    assert constraint_from_request({}, tok, 258, 0, 257) is None
    assert isinstance(constraint_from_request({"response_format": {"type": "json_object"}}, tok, 258, 0, 257), JsonConstraint)
    c = constraint_from_request({"response_format": {"type": "json_schema", "json_schema": {"schema": {"type": "array"}}}}, tok, 258, 0, 257)
    assert c.top == "array"
    e = constraint_from_request({"response_format": {"type": "json_schema", "json_schema": {"schema": {"enum": ["a", "b"]}}}}, tok, 258, 0, 257)
    assert isinstance(e, ChoiceConstraint) and e.choices == ['"a"', '"b"']


def test_hf_tokenizer_reads_end_of_sequence_ids_from_the_snapshot(tmp_path):
    import pytest
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, models, pre_tokenizers
    from cuteafd_b200.loader.tokenizer import load_tokenizer
    vocab = {"<|endoftext|>": 0, "<|im_end|>": 1, "a": 2, "b": 3, "[UNK]": 4}
    tk = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tk.pre_tokenizer = pre_tokenizers.Whitespace()
    tk.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [1, 0]}))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"eos_token": {"content": "<|im_end|>"}}))
    t = load_tokenizer(str(tmp_path))
    assert t.eos_id == 1 and t.stop_ids == (0,) and t.encode("a b") == [2, 3]


SCHEMA = {"type": "object", "additionalProperties": False, "required": ["city", "days"],
          "properties": {"city": {"type": "string"}, "days": {"type": "integer"}, "unit": {"enum": ["C", "F"]},
                         "tags": {"type": "array", "items": {"type": "string"}},
                         "geo": {"type": "object", "properties": {"lat": {"type": "number"}}, "required": ["lat"]}}}


def test_schema_prefix_enforces_types_required_closed_objects_items_and_enums():
    from cuteafd_b200.serving.constraints import SchemaPrefix
    good = ['{"city": "Oslo", "days": 3}', '{"days":2,"city":"x","unit":"F","tags":["a","b"],"geo":{"lat":1.5}}', ' { "city" : "a" , "days" : -1 } ']
    bad = ['{"city": "Oslo"}', '{"city": 1, "days": 2}', '{"city":"a","days":2.5}', '{"city":"a","days":2,"x":1}', '{"city":"a","days":2,"unit":"K"}',
           '{"city":"a","days":2,"tags":[1]}', '{"city":"a","days":2,"geo":{}}', "[1]", '{"city":"a","city":"b","days":1}']
    for t in good:
        p = SchemaPrefix(SCHEMA)
        assert p.feed_text(t) and p.complete, t
    for t in bad:
        p = SchemaPrefix(SCHEMA)
        assert not (p.feed_text(t) and p.complete), t


def test_schema_constrained_random_walk_yields_valid_documents():
    tok, rng, done = ByteTokenizer(), random.Random(1), 0
    for _ in range(10):
        c, toks = JsonConstraint(tok, 258, 0, eos_id=257, schema=SCHEMA), []
        for _ in range(400):
            allowed = [i for i, a in enumerate(unpack_bits(c.mask(toks), 258)) if a]
            assert allowed
            closers = [a for a in allowed if a in (257, ord("}"), ord("]"), ord('"'), ord(","), ord(":"))]
            toks.append(rng.choice(closers) if closers and rng.random() < 0.6 else rng.choice(allowed))
            if toks[-1] == 257:
                break
        if toks[-1] == 257:
            v = json.loads(tok.decode(toks[:-1]))
            assert isinstance(v["city"], str) and isinstance(v["days"], int) and set(v) <= set(SCHEMA["properties"])
            done += 1
    assert done >= 1
    c = constraint_from_request({"response_format": {"type": "json_schema", "json_schema": {"schema": SCHEMA}}}, tok, 258, 0, 257)
    assert c.schema is SCHEMA


def test_forced_tool_call_grammar_names_a_tool_and_checks_its_arguments():
    from cuteafd_b200.serving.constraints import ToolCallPrefix, tool_choice_constraint
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {"city": {"type": "string"}},
                                                                                     "required": ["city"], "additionalProperties": False}}},
             {"type": "function", "function": {"name": "get_time", "parameters": {"type": "object", "properties": {"tz": {"enum": ["UTC", "CET"]}},
                                                                                  "required": ["tz"], "additionalProperties": False}}}]
    schemas = {t["function"]["name"]: t["function"]["parameters"] for t in tools}
    good = '<tool_call>\n{"name": "get_time", "arguments": {"tz": "CET"}}\n</tool_call>'
    p = ToolCallPrefix(schemas)
    assert p.feed_text(good) and p.complete
    for bad in ('<tool_call>\n{"name": "nope"', '<tool_call>\n{"name": "get_time", "arguments": {"tz": "PST"', "Sure", good + "x",
                '<tool_call>\n{"name": "get_weather", "arguments": {}}'):
        assert not ToolCallPrefix(schemas).feed_text(bad), bad
    tok, t, rng = ByteTokenizer(), template_for("qwen3"), random.Random(0)
    for choice in ("required", {"type": "function", "function": {"name": "get_time"}}):
        c, toks = tool_choice_constraint({"tools": tools, "tool_choice": choice}, t, tok, 258, 0, 257), []
        for _ in range(300):
            allowed = [i for i, a in enumerate(unpack_bits(c.mask(toks), 258)) if a]
            closers = [a for a in allowed if a in (257, ord("}"), ord('"'))]
            toks.append(rng.choice(closers) if closers and rng.random() < 0.7 else rng.choice(allowed))
            if toks[-1] == 257:
                break
        assert toks[-1] == 257
        calls = parse_completion(t, tok.decode(toks[:-1]))["tool_calls"]
        assert len(calls) == 1 and calls[0]["name"] in schemas and (calls[0]["name"] != "get_time" or calls[0]["arguments"]["tz"] in ("UTC", "CET"))
    assert tool_choice_constraint({"tools": tools, "tool_choice": "auto"}, t, tok, 258, 0, 257) is None
    assert tool_choice_constraint({"tools": tools, "tool_choice": "required"}, template_for("glm-5"), tok, 258, 0, 257) is None


def test_template_round_trip_of_assistant_tool_calls():
    """What a template writes for an assistant turn with tool calls parses back to the same calls (every family)."""
    call = {"id": "c1", "type": "function", "function": {"name": "get_weather", "arguments": json.dumps({"city": "Oslo", "days": 3, "units": ["C", "F"]})}}
    msgs = [{"role": "user", "content": "q"}, {"role": "assistant", "content": "Looking it up.", "tool_calls": [call]}, {"role": "user", "content": "next"}]
    for model, start, end in (("qwen3-235b", "<|im_start|>assistant\n", "<|im_end|>"), ("qwen3-coder", "<|im_start|>assistant\n", "<|im_end|>"),
                              ("deepseek-v3", "<｜Assistant｜>", "<｜end▁of▁sentence｜>"), ("glm-5", "<|assistant|>\n", "<|user|>")):
        t = template_for(model)
        text = t.render(msgs, tools=TOOLS)
        seg = text.split(start, 1)[1].split(end, 1)[0]
        got = parse_completion(t, seg)
        assert [(c["name"], c["arguments"]) for c in got["tool_calls"]] == [("get_weather", {"city": "Oslo", "days": 3, "units": ["C", "F"]})], model
        assert got["content"].strip() == "Looking it up.", model


REF_SCHEMA = {"type": "object", "additionalProperties": False, "required": ["v"],
              "properties": {"v": {"anyOf": [{"type": "integer"}, {"type": "string", "pattern": "^[a-c]+$"}, {"type": "null"}]},
                             "kind": {"const": "leaf"}, "node": {"$ref": "#/$defs/n"}},
              "$defs": {"n": {"type": "object", "additionalProperties": False,
                              "properties": {"next": {"$ref": "#/$defs/n"}, "tag": {"oneOf": [{"type": "boolean"}, {"type": "string", "enum": ["x", "yy"]}]}}}}}


def test_schema_refs_unions_const_and_patterns():
    """`$ref` (recursive), `anyOf` / `oneOf`, `const` and string `pattern` are enforced; prefixes are judged character by character."""
    from cuteafd_b200.serving.constraints import SchemaSet

    def run(text):
        s = SchemaSet(REF_SCHEMA)
        return s.feed_text(text), s.complete
    assert run('{"v": 12}') == (True, True) and run('{"v": null}') == (True, True) and run('{"v": "abca"}') == (True, True)
    assert run('{"v": "ab')[0] and not run('{"v": "abd')[0] and not run('{"v": 1.5')[0] and not run('{"v": tr')[0]
    assert run('{"v": 3, "kind": "leaf"}') == (True, True) and not run('{"v": 3, "kind": "lead')[0] and not run('{"v": 3, "kind": 1')[0]
    assert run('{"v": 3, "node": {"next": {"next": {"tag": "yy"}}, "tag": true}}') == (True, True)
    assert not run('{"v": 3, "node": {"next": {"nex": ')[0] and not run('{"v": 3, "node": {"tag": "z')[0] and not run('{"v": 3, "node": {"tag": 7')[0]
    assert not run('{"node": {}}')[0]                       # required key missing at the close


def test_union_schema_random_walk_and_whole_text_regex():
    tok, rng, done = ByteTokenizer(), random.Random(5), 0
    for _ in range(12):
        c, toks = JsonConstraint(tok, 258, 0, eos_id=257, schema=REF_SCHEMA), []
        for _ in range(500):
            allowed = [i for i, a in enumerate(unpack_bits(c.mask(toks), 258)) if a]
            assert allowed
            closers = [a for a in allowed if a in (257, ord("}"), ord("]"), ord('"'), ord(","), ord(":"))]
            toks.append(rng.choice(closers) if closers and rng.random() < 0.7 else rng.choice(allowed))
            if toks[-1] == 257:
                break
        if toks[-1] == 257:
            v = json.loads(tok.decode(toks[:-1]))
            assert "v" in v and (v["v"] is None or isinstance(v["v"], int) or set(v["v"]) <= set("abc")) and v.get("kind", "leaf") == "leaf"
            done += 1
    assert done >= 1
    # the completion as a whole matches a regular expression
    c = constraint_from_request({"guided_regex": r"(yes|no), \d{2}"}, tok, 258, 0, 257)
    toks = []
    for _ in range(20):
        allowed = [i for i, a in enumerate(unpack_bits(c.mask(toks), 258)) if a]
        toks.append(rng.choice(allowed))
        if toks[-1] == 257:
            break
    import re
    assert toks[-1] == 257 and re.fullmatch(r"(yes|no), \d{2}", tok.decode(toks[:-1]))
