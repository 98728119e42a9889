"""Chat templates, tool-call formats and the streaming output parser of the model families the server speaks.

A template turns OpenAI-style messages (+ optional tool definitions) into the prompt text of a family and knows how
that family writes reasoning and tool calls in its output:

  * `chatml` (Qwen): `<|im_start|>role\\n...<|im_end|>`, tools listed in the system turn inside `<tools>`, calls as
    `<tool_call>{"name":..,"arguments":..}</tool_call>` (JSON) or the Qwen3-Coder XML form
    `<tool_call><function=NAME><parameter=KEY>VALUE</parameter></function></tool_call>`, results in a user turn inside
    `<tool_response>`; reasoning inside `<think>...</think>`, dropped from earlier assistant turns when re-rendered.
  * `deepseek`: `<｜begin▁of▁sentence｜>system<｜User｜>...<｜Assistant｜>`, calls inside
    `<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>NAME\\n```json\\n{..}\\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>`,
    results inside `<｜tool▁outputs▁begin｜><｜tool▁output▁begin｜>..<｜tool▁output▁end｜><｜tool▁outputs▁end｜>`.
  * `glm`: `[gMASK]<sop><|system|>\\n..<|user|>\\n..<|assistant|>\\n`, calls as
    `<tool_call>NAME\\n<arg_key>K</arg_key>\\n<arg_value>V</arg_value>\\n</tool_call>`, results after `<|observation|>`.
  * `plain`: role-tagged text for models without a template (and the byte tokenizer of the tests).

`StreamParser` consumes decoded text increments and yields ("reasoning" | "content", text) and ("tool_call", dict)
events; text that could still turn into a tag is held back so a tag is never half-emitted.

Reference: cuteafd-api/src/openai/chat/ (deepseek/parser.rs streaming parser, v41_turns.rs thinking-history rule,
glm5/*.rs template + XML tool parser, qwen4/*.rs template + Qwen3-Coder XML parser), openai/tools.rs.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field


def _text(content) -> str:
    if content is None:
        return ""
    if isinstance(content, list):
        return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type", "text") == "text")
    return str(content)


def _strip_reasoning(text: str) -> str:
    """Earlier assistant turns are re-rendered without their reasoning (only the final answer is history)."""
    end = text.rfind("</think>")
    return text[end + len("</think>"):].lstrip("\n") if end >= 0 else text


def _tool_specs(tools) -> list[dict]:
    out = []
    for t in tools or []:
        f = t.get("function", t) if isinstance(t, dict) else None
        if f and f.get("name"):
            out.append({"type": "function", "function": {"name": f["name"], "description": f.get("description", ""),
                                                        "parameters": f.get("parameters") or f.get("input_schema") or {"type": "object", "properties": {}}}})
    return out


def _calls_of(msg: dict) -> list[dict]:
    out = []
    for c in msg.get("tool_calls") or []:
        f = c.get("function", c)
        args = f.get("arguments", {})
        if isinstance(args, str):
            try:
                args = json.loads(args) if args.strip() else {}
            except json.JSONDecodeError:
                args = {"_raw": args}
        out.append({"name": f.get("name", ""), "arguments": args})
    return out


@dataclass
class ChatTemplate:
    name: str = "plain"
    think_open: str = "<think>"
    think_close: str = "</think>"
    call_open: str = "<tool_call>"
    call_close: str = "</tool_call>"
    stop_strings: tuple = ()

    # -------------------------------------------------------------- prompt side
    def render(self, messages: list[dict], tools=None, system: str | None = None, thinking: bool = False) -> str:
        parts = []
        if system:
            parts.append(f"<|system|>\n{system}\n")
        for m in messages:
            parts.append(f"<|{m.get('role', 'user')}|>\n{_text(m.get('content'))}\n")
        parts.append("<|assistant|>\n")
        return "".join(parts)

    # -------------------------------------------------------------- output side
    def parse_call(self, body: str) -> dict | None:
        """One call from the text between `call_open` and `call_close`."""
        return parse_json_call(body)

    def parser(self, thinking: bool = False) -> "StreamParser":
        return StreamParser(self, in_reasoning=thinking)


def parse_json_call(body: str) -> dict | None:
    try:
        d = json.loads(body.strip())
    except json.JSONDecodeError:
        return None
    if not isinstance(d, dict) or "name" not in d:
        return None
    return {"name": d["name"], "arguments": d.get("arguments", d.get("parameters", {}))}


def _coerce(v: str):
    """XML-style parameter values are text; numbers, booleans, null and JSON containers are recovered."""
    s = v.strip()
    if s and (s[0] in "[{\"" or s in ("true", "false", "null") or re.fullmatch(r"-?\d+(\.\d+)?([eE][+-]?\d+)?", s)):
        try:
            return json.loads(s)
        except json.JSONDecodeError:
            pass
    return v.strip("\n")


_QWEN_FN = re.compile(r"<function=([^>\s]+)>(.*?)</function>", re.S)
_QWEN_PARAM = re.compile(r"<parameter=([^>\s]+)>(.*?)</parameter>", re.S)


def parse_qwen_xml_call(body: str) -> dict | None:
    m = _QWEN_FN.search(body)
    if not m:
        return None
    return {"name": m.group(1), "arguments": {k: _coerce(v) for k, v in _QWEN_PARAM.findall(m.group(2))}}


_GLM_ARG = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)


def parse_glm_call(body: str) -> dict | None:
    name = body.strip().split("\n", 1)[0].split("<arg_key>", 1)[0].strip()
    if not name:
        return None
    return {"name": name, "arguments": {k.strip(): _coerce(v) for k, v in _GLM_ARG.findall(body)}}


# ---------------------------------------------------------------------------------------------- families
class ChatMLTemplate(ChatTemplate):
    """Qwen family."""

    def __init__(self, xml_calls: bool = False):
        super().__init__(name="chatml", stop_strings=("<|im_end|>",))
        self.xml_calls = xml_calls

    def _tools_block(self, tools) -> str:
        lines = "\n".join(json.dumps(t, ensure_ascii=False) for t in _tool_specs(tools))
        if self.xml_calls:
            how = ("<tool_call>\n<function=example_function_name>\n<parameter=example_parameter_1>\nvalue_1\n</parameter>\n"
                   "</function>\n</tool_call>")
        else:
            how = '<tool_call>\n{"name": <function-name>, "arguments": <args-json-object>}\n</tool_call>'
        return ("# Tools\n\nYou may call one or more functions to assist with the user query.\n\nYou are provided with function "
                f"signatures within <tools></tools> XML tags:\n<tools>\n{lines}\n</tools>\n\nFor each function call, return:\n{how}")

    def _call_text(self, c: dict) -> str:
        if self.xml_calls:
            ps = "".join(f"<parameter={k}>\n{v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)}\n</parameter>\n"
                         for k, v in c["arguments"].items())
            return f"<tool_call>\n<function={c['name']}>\n{ps}</function>\n</tool_call>"
        return "<tool_call>\n" + json.dumps({"name": c["name"], "arguments": c["arguments"]}, ensure_ascii=False) + "\n</tool_call>"

    def render(self, messages, tools=None, system=None, thinking=False) -> str:
        msgs = list(messages)
        sys_text = system or ""
        if msgs and msgs[0].get("role") == "system":
            sys_text = (sys_text + "\n\n" if sys_text else "") + _text(msgs.pop(0).get("content"))
        if _tool_specs(tools):
            sys_text = (sys_text + "\n\n" if sys_text else "") + self._tools_block(tools)
        out = [f"<|im_start|>system\n{sys_text}<|im_end|>\n"] if sys_text else []
        last_user = max((i for i, m in enumerate(msgs) if m.get("role") == "user"), default=-1)
        i = 0
        while i < len(msgs):
            m = msgs[i]
            role = m.get("role", "user")
            if role == "tool":
                block = []
                while i < len(msgs) and msgs[i].get("role") == "tool":       # consecutive results share one user turn
                    block.append(f"<tool_response>\n{_text(msgs[i].get('content'))}\n</tool_response>")
                    i += 1
                out.append("<|im_start|>user\n" + "\n".join(block) + "<|im_end|>\n")
                continue
            body = _text(m.get("content"))
            if role == "assistant":
                if i < last_user:
                    body = _strip_reasoning(body)
                calls = "\n".join(self._call_text(c) for c in _calls_of(m))
                body = body + ("\n" if body and calls else "") + calls
            out.append(f"<|im_start|>{role}\n{body}<|im_end|>\n")
            i += 1
        out.append("<|im_start|>assistant\n" + ("<think>\n" if thinking else ""))
        return "".join(out)

    def parse_call(self, body):
        return parse_qwen_xml_call(body) or parse_json_call(body)


class DeepSeekTemplate(ChatTemplate):
    BOS, USER, ASSISTANT, EOS = "<｜begin▁of▁sentence｜>", "<｜User｜>", "<｜Assistant｜>", "<｜end▁of▁sentence｜>"

    def __init__(self):
        super().__init__(name="deepseek", call_open="<｜tool▁call▁begin｜>", call_close="<｜tool▁call▁end｜>", stop_strings=(self.EOS,))

    def render(self, messages, tools=None, system=None, thinking=False) -> str:
        msgs = list(messages)
        sys_text = system or ""
        if msgs and msgs[0].get("role") == "system":
            sys_text = (sys_text + "\n\n" if sys_text else "") + _text(msgs.pop(0).get("content"))
        specs = _tool_specs(tools)
        if specs:
            listing = "\n\n".join(f"### {t['function']['name']}\nDescription: {t['function']['description']}\n\nParameters: "
                                  f"{json.dumps(t['function']['parameters'], ensure_ascii=False)}" for t in specs)
            sys_text = (sys_text + "\n\n" if sys_text else "") + "## Tools\nYou have access to the following tools:\n\n" + listing
        out = [self.BOS + sys_text]
        last_user = max((i for i, m in enumerate(msgs) if m.get("role") == "user"), default=-1)
        i = 0
        while i < len(msgs):
            m = msgs[i]
            role = m.get("role", "user")
            if role == "user":
                out.append(self.USER + _text(m.get("content")))
            elif role == "assistant":
                body = _text(m.get("content"))
                if i < last_user:
                    body = _strip_reasoning(body)
                calls = _calls_of(m)
                if calls:
                    body += "<｜tool▁calls▁begin｜>" + "".join(
                        f"<｜tool▁call▁begin｜>function<｜tool▁sep｜>{c['name']}\n```json\n{json.dumps(c['arguments'], ensure_ascii=False)}\n```<｜tool▁call▁end｜>"
                        for c in calls) + "<｜tool▁calls▁end｜>"
                out.append(self.ASSISTANT + body + self.EOS)
            elif role == "tool":
                block = []
                while i < len(msgs) and msgs[i].get("role") == "tool":
                    block.append(f"<｜tool▁output▁begin｜>{_text(msgs[i].get('content'))}<｜tool▁output▁end｜>")
                    i += 1
                out.append("<｜tool▁outputs▁begin｜>" + "".join(block) + "<｜tool▁outputs▁end｜>")
                continue
            i += 1
        out.append(self.ASSISTANT + ("<think>\n" if thinking else ""))
        return "".join(out)

    def parse_call(self, body):
        head, _, rest = body.partition("<｜tool▁sep｜>")
        name, _, args = (rest if _ else head).partition("\n")
        m = re.search(r"```(?:json)?\s*(.*?)\s*```", args, re.S)
        raw = m.group(1) if m else args.strip()
        try:
            return {"name": name.strip(), "arguments": json.loads(raw) if raw else {}}
        except json.JSONDecodeError:
            return None


class GlmTemplate(ChatTemplate):
    def __init__(self):
        super().__init__(name="glm", stop_strings=("<|user|>", "<|observation|>", "<|endoftext|>"))

    def render(self, messages, tools=None, system=None, thinking=False) -> str:
        msgs = list(messages)
        out = ["[gMASK]<sop>"]
        specs = _tool_specs(tools)
        if specs:
            out.append("<|system|>\n# Tools\n\nYou may call one or more functions to assist with the user query.\n\n<tools>\n"
                       + "\n".join(json.dumps(t["function"], ensure_ascii=False) for t in specs)
                       + "\n</tools>\n\nFor each function call, output the function name and arguments within the following XML format:\n"
                         "<tool_call>{function-name}\n<arg_key>{arg-key-1}</arg_key>\n<arg_value>{arg-value-1}</arg_value>\n...\n</tool_call>")
        if system:
            out.append(f"<|system|>\n{system}")
        last_user = max((i for i, m in enumerate(msgs) if m.get("role") == "user"), default=-1)
        for i, m in enumerate(msgs):
            role, body = m.get("role", "user"), _text(m.get("content"))
            if role == "tool":
                out.append(f"<|observation|>\n<tool_response>\n{body}\n</tool_response>")
                continue
            if role == "assistant":
                if i < last_user:
                    body = _strip_reasoning(body)
                for c in _calls_of(m):
                    args = "".join(f"<arg_key>{k}</arg_key>\n<arg_value>{v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)}</arg_value>\n"
                                   for k, v in c["arguments"].items())
                    body += f"\n<tool_call>{c['name']}\n{args}</tool_call>"
            out.append(f"<|{role}|>\n{body}")
        out.append("<|assistant|>\n" + ("<think>" if thinking else ""))
        return "".join(out)

    def parse_call(self, body):
        return parse_glm_call(body)


def template_for(model: str | None) -> ChatTemplate:
    """Template by model / family name (`qwen3-235b`, `deepseek-v3`, `glm-5`, ...); unknown names get the plain one."""
    n = (model or "").lower()
    if "coder" in n and "qwen" in n:
        return ChatMLTemplate(xml_calls=True)
    if "qwen" in n or "chatml" in n or "mimo" in n:
        return ChatMLTemplate()
    if "deepseek" in n or "dsv" in n:
        return DeepSeekTemplate()
    if "glm" in n:
        return GlmTemplate()
    return ChatTemplate()


# ---------------------------------------------------------------------------------------------- streaming output parser
class StreamParser:
    """Splits a streamed completion into reasoning, content and tool calls.

    `push(text)` returns the events that are final given the text so far; a suffix that is a proper prefix of one of
    the tags being watched is held back until it is resolved.  `finish()` flushes what is left (an unterminated call
    is returned as content, an unterminated reasoning block as reasoning)."""

    def __init__(self, template: ChatTemplate, in_reasoning: bool = False):
        self.t = template
        self.mode = "reasoning" if in_reasoning else "content"
        self.buf = ""
        self.calls: list[dict] = []

    def _tags(self):
        if self.mode == "reasoning":
            return [self.t.think_close]
        if self.mode == "call":
            return [self.t.call_close]
        return [self.t.think_open, self.t.call_open]

    def push(self, text: str) -> list[tuple]:
        self.buf += text
        events = []
        while True:
            tags = self._tags()
            hits = [(self.buf.find(tag), tag) for tag in tags if tag in self.buf]
            if hits:
                pos, tag = min(hits)
                before, self.buf = self.buf[:pos], self.buf[pos + len(tag):]
                if self.mode == "call":
                    call = self.t.parse_call(before)
                    if call is not None:
                        call = dict(call, id="call_" + uuid.uuid4().hex[:12])
                        self.calls.append(call)
                        events.append(("tool_call", call))
                    else:
                        events.append(("content", self.t.call_open + before + tag))
                    self.mode = "content"
                else:
                    if before:
                        events.append((self.mode, before))
                    self.mode = {self.t.think_open: "reasoning", self.t.think_close: "content", self.t.call_open: "call"}[tag]
                    if self.mode == "content":
                        self.buf = self.buf.lstrip("\n")
                continue
            if self.mode == "call":
                return events                                  # a call is only emitted whole
            hold = 0
            for tag in tags:                                    # longest suffix of the buffer that may still become a tag
                for k in range(min(len(tag) - 1, len(self.buf)), 0, -1):
                    if self.buf.endswith(tag[:k]):
                        hold = max(hold, k)
                        break
            cut = len(self.buf) - hold
            if cut > 0:
                events.append((self.mode, self.buf[:cut]))
                self.buf = self.buf[cut:]
            return events

    def finish(self) -> list[tuple]:
        events = []
        if self.buf:
            events.append(("content", self.t.call_open + self.buf) if self.mode == "call" else (self.mode, self.buf))
        self.buf = ""
        return events


def parse_completion(template: ChatTemplate, text: str, thinking: bool = False) -> dict:
    """Whole-completion form of the parser: {"content", "reasoning", "tool_calls"} with stop strings removed."""
    for s in template.stop_strings:
        cut = text.find(s)
        if cut >= 0:
            text = text[:cut]
    p = template.parser(thinking)
    ev = p.push(text) + p.finish()
    join = lambda kind: "".join(x for k, x in ev if k == kind)
    skip = ("<｜tool▁calls▁begin｜>", "<｜tool▁calls▁end｜>")
    content = join("content")
    for s in skip:
        content = content.replace(s, "")
    return {"content": content.strip("\n") if p.calls else content, "reasoning": join("reasoning"), "tool_calls": p.calls}


# ---------------------------------------------------------------------------------------------- round-trip check
_ASSISTANT_SPAN = {"ChatMLTemplate": ("<|im_start|>assistant\n", "<|im_end|>"), "DeepSeekTemplate": ("<｜Assistant｜>", "<｜end▁of▁sentence｜>"),
                   "GlmTemplate": ("<|assistant|>\n", "<|user|>")}


def template_round_trip(model: str | None) -> bool:
    """Quality gate of the baseline card: an assistant turn with text and a tool call, rendered by the model's template, parses
    back to the same text and the same call (reference: the chat-template round trip of cuteafd-bench/src/baseline.rs:1-6).
    Families without a tool-call syntax (the plain template) pass when the text survives."""
    import json
    t = template_for(model)
    args = {"city": "Oslo", "days": 3, "units": ["C", "F"]}
    tools = [{"type": "function", "function": {"name": "get_weather", "description": "weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}, "units": {"type": "array", "items": {"type": "string"}}}}}}]
    call = {"id": "c1", "type": "function", "function": {"name": "get_weather", "arguments": json.dumps(args)}}
    msgs = [{"role": "user", "content": "q"}, {"role": "assistant", "content": "Looking it up.", "tool_calls": [call]}, {"role": "user", "content": "next"}]
    span = _ASSISTANT_SPAN.get(type(t).__name__)
    if span is None:
        return "Looking it up." in t.render(msgs[:1] + [{"role": "assistant", "content": "Looking it up."}])
    text = t.render(msgs, tools=tools)
    if span[0] not in text:
        return False
    seg = text.split(span[0], 1)[1].split(span[1], 1)[0]
    got = parse_completion(t, seg)
    return [(c["name"], c["arguments"]) for c in got["tool_calls"]] == [("get_weather", args)] and got["content"].strip() == "Looking it up."
