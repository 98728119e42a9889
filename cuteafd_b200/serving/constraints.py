"""Structured output: token masks that keep a completion inside a grammar.

A constraint object has `mask(tokens) -> int32 bit words [ceil(vocab / 32)] | None` (bit set = token allowed), which is
what the runner hands to the masked argmax / sampler kernels for rows that carry one.  Two grammars are built in:

  * `JsonConstraint`: the completion must be one JSON value (optionally an object / array at the top, for
    `response_format = json_object`), or follow a `json_schema` in the subset `SchemaPrefix` / `SchemaSet` enforce (types,
    properties, required, closed objects, items, string enums and `const`, string `pattern`, local `$ref` incl. recursive
    schemas, `anyOf` / `oneOf` unions), or match a regular expression as a whole (`guided_regex`), then end of sequence;
  * `ChoiceConstraint`: the completion must be exactly one of a list of strings (tool_choice by name, enums).

Both work on the decoded text of single tokens, so they run with any tokenizer that can decode one id at a time.  The
JSON automaton is a character-level pushdown recogniser of JSON *prefixes*; masks are cached per automaton state, so a
long string or number costs one vocabulary scan, not one per token.

Reference: cuteafd-api/src/openai/constraints.rs (grammar specs handed to the sampler as per-row token masks),
shared/constraints.rs (`SelectBatch` masks).
"""
from __future__ import annotations

import torch

WS = " \t\n\r"


class JsonPrefix:
    """Recogniser of prefixes of one JSON value.  `feed(ch)` returns False when `ch` cannot follow."""
    __slots__ = ("stack", "mode", "lit", "lit_pos", "hex_left", "num", "done", "top", "ws_run")
    MAX_WS = 2                          # consecutive whitespace characters between tokens (a model must not stall on blanks)

    def __init__(self, top: str | None = None):
        self.stack: list[str] = []      # "{" / "[" frames; the mode says where in the frame we are
        self.mode = "value"             # value | string | key | escape | kescape | hex | khex | number | literal | after | key_start | key_or_end | colon | value_or_end
        self.lit, self.lit_pos, self.hex_left, self.num = "", 0, 0, ""
        self.done = False
        self.top = top                  # None | "object" | "array"
        self.ws_run = 0

    def copy(self) -> "JsonPrefix":
        c = JsonPrefix(self.top)
        c.stack, c.mode, c.lit, c.lit_pos, c.hex_left, c.num, c.done = list(self.stack), self.mode, self.lit, self.lit_pos, self.hex_left, self.num, self.done
        c.ws_run = self.ws_run
        return c

    def signature(self):
        return (tuple(self.stack), self.mode, self.lit, self.lit_pos, self.hex_left, self._num_class(), self.done, self.ws_run)

    # -------------------------------------------------------------- numbers: -?(0|[1-9]\d*)(\.\d+)?([eE][+-]?\d+)?
    def _num_class(self) -> str:
        n = self.num
        if not n:
            return ""
        if n == "-":
            return "sign"
        if "e" in n or "E" in n:
            tail = n.replace("E", "e").split("e", 1)[1]
            return "exp0" if tail == "" else ("expsign" if tail in "+-" else "exp")
        if "." in n:
            return "frac0" if n.endswith(".") else "frac"
        return "zero" if n.lstrip("-") == "0" else "int"

    def _num_can_end(self) -> bool:
        return self._num_class() in ("zero", "int", "frac", "exp")

    def _num_feed(self, ch: str) -> bool:
        c = self._num_class()
        if ch.isdigit() and ch.isascii():
            if c == "zero":
                return False
            self.num += ch
            return True
        if ch == "." and c in ("zero", "int"):
            self.num += ch
            return True
        if ch in "eE" and c in ("zero", "int", "frac"):
            self.num += ch
            return True
        if ch in "+-" and c == "exp0":
            self.num += ch
            return True
        return False

    # -------------------------------------------------------------- transitions
    def _value_done(self):
        if not self.stack:
            self.done, self.mode = True, "after"
        else:
            self.mode = "after"

    def _start_value(self, ch: str) -> bool:
        if not self.stack and self.top and not self.done:
            if (self.top == "object" and ch != "{") or (self.top == "array" and ch != "["):
                return False
        if ch == "{":
            self.stack.append("{"); self.mode = "key_or_end"; return True
        if ch == "[":
            self.stack.append("["); self.mode = "value_or_end"; return True
        if ch == '"':
            self.mode = "string"; return True
        if ch == "-" or (ch.isdigit() and ch.isascii()):
            self.num, self.mode = ch, "number"; return True
        for lit in ("true", "false", "null"):
            if ch == lit[0]:
                self.lit, self.lit_pos, self.mode = lit, 1, "literal"; return True
        return False

    def feed(self, ch: str) -> bool:
        m = self.mode
        if m in ("string", "key"):
            if ch == '"':
                if m == "key":
                    self.mode = "colon"
                else:
                    self._value_done()
                return True
            if ch == "\\":
                self.mode = "escape" if m == "string" else "kescape"
                return True
            return ch >= " "
        if m in ("escape", "kescape"):
            back = "string" if m == "escape" else "key"
            if ch in '"\\/bfnrt':
                self.mode = back; return True
            if ch == "u":
                self.hex_left, self.mode = 4, "hex" if m == "escape" else "khex"; return True
            return False
        if m in ("hex", "khex"):
            if ch not in "0123456789abcdefABCDEF":
                return False
            self.hex_left -= 1
            if self.hex_left == 0:
                self.mode = "string" if m == "hex" else "key"
            return True
        if m == "literal":
            if ch != self.lit[self.lit_pos]:
                return False
            self.lit_pos += 1
            if self.lit_pos == len(self.lit):
                self._value_done()
            return True
        if m == "number":
            if self._num_feed(ch):
                return True
            if not self._num_can_end():
                return False
            self.num = ""
            self._value_done()
            return self.feed(ch)
        if ch in WS:
            self.ws_run += 1
            return self.ws_run <= self.MAX_WS
        self.ws_run = 0
        if m == "value":
            return (not self.done) and self._start_value(ch)
        if m == "value_or_end":
            if ch == "]":
                self.stack.pop(); self._value_done(); return True
            return self._start_value(ch)
        if m == "key_or_end":
            if ch == "}":
                self.stack.pop(); self._value_done(); return True
            if ch == '"':
                self.mode = "key"; return True
            return False
        if m == "key_start":
            if ch == '"':
                self.mode = "key"; return True
            return False
        if m == "colon":
            if ch == ":":
                self.mode = "value"; return True
            return False
        if m == "after":
            if not self.stack:
                return False
            if ch == ",":
                self.mode = "key_start" if self.stack[-1] == "{" else "value"; return True
            if ch == "}" and self.stack[-1] == "{" or ch == "]" and self.stack[-1] == "[":
                self.stack.pop(); self._value_done(); return True
            return False
        return False

    @property
    def complete(self) -> bool:
        """The text so far is a whole value (a top-level number also counts once it can end)."""
        return (self.done and self.mode == "after" and not self.stack) or (not self.stack and self.mode == "number" and self._num_can_end())

    def feed_text(self, text: str) -> bool:
        for ch in text:
            if not self.feed(ch):
                return False
        return True

    def finished(self) -> bool:
        return self.complete and not self.stack and self.mode == "after"


_FIRST = {"object": "{", "array": "[", "string": '"', "number": "-0123456789", "integer": "-0123456789", "boolean": "tf", "null": "n"}


def _int_bounds(schema: dict):
    """(lowest, highest) integer a schema's minimum / maximum / exclusive bounds allow, None for an open side."""
    import math
    lo = hi = None
    for key, excl in (("minimum", False), ("exclusiveMinimum", True)):
        v = schema.get(key)
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            b = math.floor(v) + 1 if excl else math.ceil(v)
            lo = b if lo is None else max(lo, b)
    for key, excl in (("maximum", False), ("exclusiveMaximum", True)):
        v = schema.get(key)
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            b = math.ceil(v) - 1 if excl else math.floor(v)
            hi = b if hi is None else min(hi, b)
    return lo, hi


def _num_bounds(schema: dict):
    """(low, low is exclusive, high, high is exclusive) of a `number` schema, None for an open side."""
    lo = hi = None
    lo_x = hi_x = False
    for key, excl in (("minimum", False), ("exclusiveMinimum", True)):
        v = schema.get(key)
        if isinstance(v, (int, float)) and not isinstance(v, bool) and (lo is None or v > lo or (v == lo and excl)):
            lo, lo_x = float(v), excl
    for key, excl in (("maximum", False), ("exclusiveMaximum", True)):
        v = schema.get(key)
        if isinstance(v, (int, float)) and not isinstance(v, bool) and (hi is None or v < hi or (v == hi and excl)):
            hi, hi_x = float(v), excl
    return lo, lo_x, hi, hi_x


def _num_in(v: float, b) -> bool:
    lo, lo_x, hi, hi_x = b
    return not (lo is not None and (v < lo or (lo_x and v == lo))) and not (hi is not None and (v > hi or (hi_x and v == hi)))


def _num_prefix_ok(text: str, b) -> bool:
    """Can a decimal typed so far (no exponent) still end inside the bounds?  With k fraction digits typed the values it can grow
    into lie within one unit of the last place of the typed value, away from zero."""
    import math
    lo, lo_x, hi, hi_x = b
    neg = text.startswith("-")
    if neg and lo is not None and (lo > 0 or (lo == 0 and lo_x)):          # a minus sign writes a value <= 0
        return False
    if not neg and hi is not None and (hi < 0 or (hi == 0 and hi_x)):
        return False
    if "." not in text:
        ilo = None if lo is None else math.trunc(lo)
        ihi = None if hi is None else math.trunc(hi)
        return _int_prefix_ok(text, ilo, ihi) or (neg and text in ("-", "-0") and (lo is None or lo < 0) and (hi is None or hi > -1))
    frac = text.split(".", 1)[1]
    v = float(text + "0")
    ulp = 10.0 ** -len(frac)
    if neg:                                               # reachable values: (v - ulp, v]
        return not (hi is not None and v - ulp >= hi) and not (lo is not None and v < lo)
    return not (hi is not None and v > hi) and not (lo is not None and v + ulp <= lo)          # reachable values: [v, v + ulp)


def _int_prefix_ok(text: str, lo, hi) -> bool:
    """Can the digits typed so far (optionally after a minus sign) still grow into an integer inside [lo, hi]?"""
    neg = text.startswith("-")
    d = text[1:] if neg else text
    if not d:
        return lo is None or lo <= 0                      # "-" so far: "-0" or a negative number must be allowed
    base = int(d)
    for extra in range(0, 24):
        a, b = base * 10 ** extra, base * 10 ** extra + 10 ** extra - 1
        if neg:
            a, b = -b, -a
        if (hi is None or a <= hi) and (lo is None or b >= lo):
            return True
        if d == "0" or (not neg and hi is not None and a > hi) or (neg and lo is not None and b < lo):
            break                                         # a leading zero cannot grow; longer numbers only move further out
    return False


class SchemaPrefix:
    """`JsonPrefix` plus a cursor into a JSON schema, for the subset that covers tool arguments and typical
    `response_format` schemas: `type` (also a list of types), `properties`, `required`, `additionalProperties: false`,
    `items`, `minItems` / `maxItems`, string `enum`, `minLength` / `maxLength` (in code points, escapes counted once), `integer` vs
    `number`, `minimum` / `maximum` (also exclusive) of integers and of numbers (bounded numbers are written without an exponent and
    pruned digit by digit, so a value that cannot end inside its bounds is refused at the first digit that rules it out).
    Anything else in a schema is ignored (not enforced)."""

    def __init__(self, schema: dict, root: dict | None = None):
        self.j = JsonPrefix()
        self.frames: list = []            # [schema, kind, seen keys, key being typed or None]
        self.root = root if root is not None else (schema if isinstance(schema, dict) else {})
        self.cur = resolve_ref(schema if isinstance(schema, dict) else {}, self.root)
        self.enum: list | None = None     # inside a string value restricted to choices: [choices, typed so far]
        self.pattern: list | None = None  # inside a string value restricted by `pattern`: [compiled regex, typed so far]
        self.integer = False
        self.irange = None                # inside an integer with bounds: [lowest, highest, digits typed so far]
        self.nrange = None                # inside a number with bounds: [bounds, text typed so far]
        self.strlen = None                # inside a string with minLength / maxLength: [min, max, code points so far, escape state]

    def copy(self) -> "SchemaPrefix":
        c = SchemaPrefix.__new__(SchemaPrefix)
        c.j, c.cur, c.integer, c.root = self.j.copy(), self.cur, self.integer, self.root
        c.irange = None if self.irange is None else list(self.irange)
        c.nrange = None if self.nrange is None else list(self.nrange)
        c.strlen = None if self.strlen is None else list(self.strlen)
        c.frames = [[f[0], f[1], set(f[2]), f[3]] for f in self.frames]
        c.enum = None if self.enum is None else [self.enum[0], self.enum[1]]
        c.pattern = None if self.pattern is None else [self.pattern[0], self.pattern[1]]
        return c

    def signature(self):
        return (self.j.signature(), tuple((id(f[0]), f[1], frozenset(f[2]), f[3]) for f in self.frames), id(self.cur),
                None if self.enum is None else self.enum[1], None if self.pattern is None else self.pattern[1], self.integer,
                None if self.irange is None else tuple(self.irange), None if self.nrange is None else self.nrange[1],
                None if self.strlen is None else tuple(self.strlen[2:]))

    def finished(self) -> bool:
        return self.j.complete and not self.j.stack and self.j.mode == "after"

    def _sub(self, schema) -> dict:
        return resolve_ref(schema if isinstance(schema, dict) else {}, self.root)

    def alternatives(self):
        """At the start of a value whose schema is a union (`anyOf` / `oneOf`): one copy of this state per branch."""
        if self.j.mode not in ("value", "value_or_end"):
            return None
        alts = self.cur.get("anyOf") or self.cur.get("oneOf")
        if not isinstance(alts, list) or not alts:
            return None
        out = []
        for a in alts:
            c = self.copy()
            c.cur = self._sub(a)
            out.append(c)
        return out

    @property
    def stack(self):
        return self.j.stack

    @property
    def mode(self):
        return self.j.mode

    @property
    def complete(self) -> bool:
        if self.j.complete and self.irange is not None:       # a top-level integer that may end here: only inside its bounds
            lo, hi, typed = self.irange
            if typed in ("", "-") or (lo is not None and int(typed) < lo) or (hi is not None and int(typed) > hi):
                return False
        if self.j.complete and self.nrange is not None:
            try:
                if not _num_in(float(self.nrange[1]), self.nrange[0]):
                    return False
            except ValueError:
                return False
        return self.j.complete

    @staticmethod
    def _types(schema: dict):
        t = schema.get("type")
        if isinstance(schema.get("enum"), list) and schema["enum"] and all(isinstance(e, str) for e in schema["enum"]):
            return ["string"]
        return [t] if isinstance(t, str) else (list(t) if isinstance(t, list) else [])

    def _start_ok(self, ch: str) -> bool:
        types = self._types(self.cur)
        if types and not any(ch in _FIRST.get(t, "") for t in types):
            return False
        if "const" in self.cur and isinstance(self.cur["const"], str) and ch != '"':
            return False
        if ch == "{":
            self.frames.append([self.cur, "{", set(), None])
        elif ch == "[":
            self.frames.append([self.cur, "[", set(), 0])        # arrays: the last slot counts the items
            self.cur = self._sub(self.cur.get("items"))
        elif ch == '"':
            e = self.cur.get("enum")
            if "const" in self.cur and isinstance(self.cur["const"], str):
                e = [self.cur["const"]]
            self.enum = [[x for x in e if isinstance(x, str)], ""] if isinstance(e, list) and e else None
            pat = self.cur.get("pattern")
            self.pattern = None
            if self.enum is None and isinstance(pat, str):
                self.pattern = [_compile_pattern(pat), ""]
            self.strlen = None
            lo_n, hi_n = self.cur.get("minLength"), self.cur.get("maxLength")
            if self.enum is None and self.pattern is None and (isinstance(lo_n, int) or isinstance(hi_n, int)):
                self.strlen = [lo_n if isinstance(lo_n, int) else 0, hi_n if isinstance(hi_n, int) else None, 0, 0]
        elif ch in "-0123456789":
            self.integer = "integer" in types and "number" not in types
            self.irange = None
            if self.integer:
                lo, hi = _int_bounds(self.cur)
                if lo is not None or hi is not None:
                    self.irange = [lo, hi, ch]
                    if not _int_prefix_ok(ch, lo, hi):
                        return False
            self.nrange = None
            if not self.integer:
                b = _num_bounds(self.cur)
                if b[0] is not None or b[2] is not None:
                    self.nrange = [b, ch]
                    if not _num_prefix_ok(ch, b):
                        return False
        return True

    def _close_ok(self, ch: str) -> bool:
        if not self.frames:
            return True
        schema, kind, seen, _ = self.frames[-1]
        if ch == "}" and kind == "{":
            if any(r not in seen for r in schema.get("required", []) or []):
                return False
            self.frames.pop()
        elif ch == "]" and kind == "[":
            if isinstance(schema.get("minItems"), int) and self.frames[-1][3] < schema["minItems"]:
                return False
            self.frames.pop()
        elif ch == "," and kind == "[":
            if isinstance(schema.get("maxItems"), int) and self.frames[-1][3] >= schema["maxItems"]:
                return False
            self.frames[-1][3] += 1
            self.cur = self._sub(schema.get("items"))
        elif ch == "," and kind == "{":
            props = schema.get("properties") if isinstance(schema.get("properties"), dict) else None
            if props is not None and schema.get("additionalProperties") is False and all(k in seen for k in props):
                return False                # a closed object with every property written: nothing can follow a comma
        return True

    def feed(self, ch: str) -> bool:
        m = self.j.mode
        if m == "number" and not (ch.isdigit() or ch in ".eE+-"):
            m = "after"                                         # the number ends here; `ch` is judged as what follows a value
            if self.irange is not None:
                lo, hi, typed = self.irange
                self.irange = None
                if typed in ("", "-") or (lo is not None and int(typed) < lo) or (hi is not None and int(typed) > hi):
                    return False
            if self.nrange is not None:
                b, typed = self.nrange
                self.nrange = None
                try:
                    if not _num_in(float(typed), b):
                        return False
                except ValueError:
                    return False
        if m == "number" and self.integer and ch in ".eE":
            return False
        if m == "number" and self.nrange is not None:
            if ch in "eE+":                                      # bounded numbers are written without an exponent
                return False
            self.nrange[1] += ch
            if not _num_prefix_ok(self.nrange[1], self.nrange[0]):
                return False
        if m == "number" and self.irange is not None and ch.isdigit():
            self.irange[2] += ch
            if not _int_prefix_ok(self.irange[2], self.irange[0], self.irange[1]):
                return False
        if m == "key":
            f = self.frames[-1]
            props = f[0].get("properties") if isinstance(f[0].get("properties"), dict) else None
            closed = props is not None and f[0].get("additionalProperties") is False
            if ch == '"':
                key = f[3] or ""
                if key in f[2] or (closed and key not in props):
                    return False
                f[2].add(key)
                self.cur = self._sub((props or {}).get(key, {}))
                f[3] = None
            else:
                if closed and ch == "\\":
                    return False
                f[3] = (f[3] or "") + ch
                if closed and not any(k.startswith(f[3]) and k not in f[2] for k in props):
                    return False
        elif m == "string" and self.enum is not None:
            if ch == '"':
                if self.enum[1] not in self.enum[0]:
                    return False
                self.enum = None
            else:
                self.enum[1] += ch
                if ch == "\\" or not any(c.startswith(self.enum[1]) for c in self.enum[0]):
                    return False
        elif m == "string" and self.pattern is not None:
            rx, typed = self.pattern
            if ch == '"':
                if rx is not None and rx.fullmatch(typed) is None:
                    return False
                self.pattern = None
            else:
                typed += ch
                if ch == "\\" or (rx is not None and rx.fullmatch(typed, partial=True) is None):
                    return False
                self.pattern[1] = typed
        elif m in ("string", "escape", "hex") and self.strlen is not None:
            lo_n, hi_n, n, esc = self.strlen
            if esc == 1:                                         # the character after a backslash
                esc = 14 if ch == "u" else 0
                n += 0 if ch == "u" else 1
            elif esc > 10:                                       # hex digits of a \u escape
                esc = 0 if esc == 11 else esc - 1
                n += 1 if esc == 0 else 0
            elif ch == "\\":
                esc = 1
            elif ch == '"':
                if n < lo_n:
                    return False
                self.strlen = None
                return self.j.feed(ch)
            else:
                n += 1
            if hi_n is not None and n > hi_n:
                return False
            self.strlen[2], self.strlen[3] = n, esc
        elif ch not in WS:
            if m in ("value", "value_or_end") and not (m == "value_or_end" and ch == "]"):
                if m == "value_or_end" and self.frames and self.frames[-1][1] == "[":       # the first item of an array
                    if self.frames[-1][0].get("maxItems") == 0:
                        return False
                    self.frames[-1][3] = 1
                if not self._start_ok(ch):
                    return False
            elif m == "value_or_end" or (m in ("after", "key_or_end") and ch in "}],"):
                if not self._close_ok(ch):
                    return False
        return self.j.feed(ch)

    def feed_text(self, text: str) -> bool:
        for ch in text:
            if not self.feed(ch):
                return False
        return True


def resolve_ref(schema: dict, root: dict, depth: int = 0) -> dict:
    """Follows local `$ref`s (`#/$defs/name`, `#/definitions/name`, `#`) to the schema they name; recursive schemas resolve
    lazily because only the node being entered is resolved."""
    while isinstance(schema, dict) and isinstance(schema.get("$ref"), str) and depth < 32:
        ref, node = schema["$ref"], root
        if not ref.startswith("#"):
            return {}
        for part in [p for p in ref[1:].split("/") if p]:
            node = node.get(part.replace("~1", "/").replace("~0", "~")) if isinstance(node, dict) else None
            if node is None:
                return {}
        schema, depth = node, depth + 1
    return schema if isinstance(schema, dict) else {}


_PATTERNS: dict = {}


def _compile_pattern(pat: str):
    """Compiled `pattern` of a string schema (JSON-schema patterns search unless anchored: an unanchored side may be anything).
    Prefix decisions use the `regex` module's partial matching.  An invalid pattern is not enforced."""
    if pat not in _PATTERNS:
        try:
            import regex
            body = pat
            body = body[1:] if body.startswith("^") else "(?s:.*?)" + body
            body = body[:-1] if body.endswith("$") and not body.endswith("\\$") else body + "(?s:.*)"
            _PATTERNS[pat] = regex.compile(body)
        except Exception:
            _PATTERNS[pat] = None
    return _PATTERNS[pat]


class SchemaSet:
    """Several `SchemaPrefix` states followed at once: a schema with `anyOf` / `oneOf` forks one state per branch where the
    value starts and keeps the branches the text still fits.  Same interface as a single state."""

    def __init__(self, schema: dict | None = None, states: list | None = None):
        self.states = states if states is not None else [SchemaPrefix(schema)]
        self._expand()

    def _expand(self):
        todo, out, guard = list(self.states), [], 0
        while todo and guard < 256:
            st = todo.pop()
            alts = st.alternatives()
            guard += 1
            if alts is None:
                out.append(st)
            else:
                todo.extend(alts)
        uniq = {}
        for st in out:
            uniq.setdefault(st.signature(), st)
        self.states = list(uniq.values())

    def copy(self) -> "SchemaSet":
        c = SchemaSet.__new__(SchemaSet)
        c.states = [st.copy() for st in self.states]
        return c

    def signature(self):
        return tuple(sorted((repr(st.signature()) for st in self.states)))

    def feed(self, ch: str) -> bool:
        self.states = [st for st in self.states if st.feed(ch)]
        self._expand()
        return bool(self.states)

    def feed_text(self, text: str) -> bool:
        for ch in text:
            if not self.feed(ch):
                return False
        return True

    @property
    def complete(self) -> bool:
        return any(st.complete for st in self.states)

    def finished(self) -> bool:
        return bool(self.states) and all(st.finished() for st in self.states)


class RegexPrefix:
    """The completion must match a regular expression as a whole (`guided_regex`-style requests)."""

    def __init__(self, pattern: str):
        import regex
        self.rx, self.text = regex.compile(pattern), ""

    def copy(self):
        c = RegexPrefix.__new__(RegexPrefix)
        c.rx, c.text = self.rx, self.text
        return c

    def signature(self):
        return self.text

    def feed_text(self, text: str) -> bool:
        self.text += text
        return self.rx.fullmatch(self.text, partial=True) is not None

    @property
    def complete(self) -> bool:
        return self.rx.fullmatch(self.text) is not None

    def finished(self) -> bool:
        return False                    # a longer match may exist; the end of sequence token is allowed once `complete`


def _pack_bits(allowed: list[bool]) -> torch.Tensor:
    n = len(allowed)
    words = torch.zeros((n + 31) // 32, dtype=torch.int64)
    idx = torch.tensor([i for i, a in enumerate(allowed) if a], dtype=torch.int64)
    if idx.numel():
        words.index_put_((idx >> 5,), torch.ones_like(idx) << (idx & 31), accumulate=True)   # distinct bits: add == or
    words = torch.where(words >= (1 << 31), words - (1 << 32), words)
    return words.to(torch.int32)


class _TextConstraint:
    """Shared part: the decoded text of every token id and the prompt length (only generated tokens are constrained)."""

    def __init__(self, tokenizer, vocab_size: int, prompt_len: int, eos_id: int | None):
        self.vocab_size, self.prompt_len, self.eos_id = vocab_size, prompt_len, eos_id
        self.pieces = token_pieces(tokenizer, vocab_size)

    def _text_of(self, ids) -> str:
        return "".join(self.pieces[i] or "" for i in ids if 0 <= i < self.vocab_size)


_PIECE_CACHE: dict = {}


def token_pieces(tokenizer, vocab_size: int) -> list:
    """Decoded text per token id (None for ids that decode to nothing: specials, padding)."""
    key = (id(tokenizer), vocab_size)
    if key not in _PIECE_CACHE:
        out = []
        for i in range(vocab_size):
            try:
                s = tokenizer.decode([i])
            except Exception:
                s = ""
            out.append(s if s and "�" not in s else None)
        _PIECE_CACHE[key] = out
    return _PIECE_CACHE[key]


class JsonConstraint(_TextConstraint):
    def __init__(self, tokenizer, vocab_size: int, prompt_len: int, eos_id: int | None = None, top: str | None = "object",
                 schema: dict | None = None, regex: str | None = None, grammar=None):
        super().__init__(tokenizer, vocab_size, prompt_len, eos_id)
        self.top, self.schema, self.regex, self.grammar = top, schema, regex, grammar
        self.state, self.seen = self._fresh(), 0
        self.cache: dict = {}

    def _fresh(self):
        if self.grammar is not None:
            from .grammar import GrammarPrefix
            return GrammarPrefix(self.grammar)
        if self.regex:
            return RegexPrefix(self.regex)
        return SchemaSet(self.schema) if self.schema else JsonPrefix(self.top)

    def _advance(self, tokens):
        gen = tokens[self.prompt_len:]
        if len(gen) < self.seen:                       # a speculative tail was rolled back: replay
            self.state, self.seen = self._fresh(), 0
        for t in gen[self.seen:]:
            if t != self.eos_id:
                self.state.feed_text(self.pieces[t] or "")
        self.seen = len(gen)

    def mask(self, tokens):
        self._advance(tokens)
        sig = self.state.signature()
        m = self.cache.get(sig)
        if m is None:
            done = self.state.finished()
            allowed = [False] * self.vocab_size
            if not done:
                for i, piece in enumerate(self.pieces):
                    if piece and self.state.copy().feed_text(piece):
                        allowed[i] = True
            if self.eos_id is not None and 0 <= self.eos_id < self.vocab_size:
                allowed[self.eos_id] = self.state.complete
            if not any(allowed) and self.eos_id is not None:
                allowed[self.eos_id] = True            # never hand the sampler an empty set
            m = self.cache[sig] = _pack_bits(allowed)
        return m


class ChoiceConstraint(_TextConstraint):
    """The completion must spell exactly one of `choices`."""

    def __init__(self, tokenizer, vocab_size: int, prompt_len: int, choices: list[str], eos_id: int | None = None):
        super().__init__(tokenizer, vocab_size, prompt_len, eos_id)
        self.choices = list(choices)

    def mask(self, tokens):
        text = self._text_of(t for t in tokens[self.prompt_len:] if t != self.eos_id)
        live = [c for c in self.choices if c.startswith(text)]
        allowed = [False] * self.vocab_size
        for i, piece in enumerate(self.pieces):
            if piece and any(c.startswith(text + piece) for c in live):
                allowed[i] = True
        if self.eos_id is not None and (text in self.choices or not any(allowed)):
            allowed[self.eos_id] = True
        return _pack_bits(allowed)


class ToolCallPrefix:
    """Automaton of one forced tool call in the JSON call format:
    `OPEN\n{"name": "` NAME `", "arguments": ` ARGUMENTS `}\nCLOSE`, where NAME is one of the offered functions and
    ARGUMENTS follows that function's parameter schema (`SchemaPrefix`)."""

    def __init__(self, tools: dict, call_open: str = "<tool_call>", call_close: str = "</tool_call>"):
        self.tools = tools                               # name -> parameters schema
        self.head = call_open + '\n{"name": "'
        self.mid = '", "arguments": '
        self.tail = "}\n" + call_close
        self.phase, self.pos, self.name, self.args = 0, 0, "", None

    def copy(self):
        c = ToolCallPrefix.__new__(ToolCallPrefix)
        c.tools, c.head, c.mid, c.tail = self.tools, self.head, self.mid, self.tail
        c.phase, c.pos, c.name = self.phase, self.pos, self.name
        c.args = self.args.copy() if self.args is not None else None
        return c

    def signature(self):
        return (self.phase, self.pos, self.name, self.args.signature() if self.args is not None else None)

    # the interface JsonConstraint.mask relies on
    stack = ()

    @property
    def mode(self):
        return "after" if self.phase == 5 else "call"

    @property
    def complete(self) -> bool:
        return self.phase == 5

    def finished(self) -> bool:
        return self.phase == 5

    def _literal(self, lit: str, ch: str, nxt: int) -> bool:
        if ch != lit[self.pos]:
            return False
        self.pos += 1
        if self.pos == len(lit):
            self.phase, self.pos = nxt, 0
        return True

    def feed(self, ch: str) -> bool:
        if self.phase == 0:
            return self._literal(self.head, ch, 1)
        if self.phase == 1:                              # function name, ended by the quote
            if ch == '"':
                if self.name not in self.tools:
                    return False
                schema = self.tools[self.name] if isinstance(self.tools[self.name], dict) else {}
                self.args = SchemaSet(dict(schema, type="object"))      # tool parameter schemas may use $ref / anyOf too
                self.phase, self.pos = 2, 1              # the quote is the first character of `mid`
                return True
            self.name += ch
            return any(n.startswith(self.name) for n in self.tools)
        if self.phase == 2:
            return self._literal(self.mid, ch, 3)
        if self.phase == 3:
            if not self.args.feed(ch):
                return False
            if self.args.finished():
                self.phase = 4
            return True
        if self.phase == 4:
            return self._literal(self.tail, ch, 5)
        return False

    def feed_text(self, text: str) -> bool:
        for ch in text:
            if not self.feed(ch):
                return False
        return True


def tool_choice_constraint(body: dict, template, tokenizer, vocab_size: int, prompt_len: int, eos_id: int | None):
    """`tool_choice: "required"` or a named function -> a constraint that forces exactly one tool call (templates
    whose calls are JSON inside `call_open` / `call_close`; other call formats are not forced)."""
    choice = body.get("tool_choice")
    tools = {}
    for t in body.get("tools") or []:
        f = t.get("function", t) if isinstance(t, dict) else None
        if f and f.get("name"):
            tools[f["name"]] = f.get("parameters") or f.get("input_schema") or {}
    if isinstance(choice, dict):
        name = (choice.get("function") or {}).get("name") or choice.get("name")
        tools = {name: tools[name]} if name in tools else {}
    elif choice not in ("required", "any"):
        return None
    if not tools or getattr(template, "name", "") != "chatml" or getattr(template, "xml_calls", False):
        return None
    c = JsonConstraint(tokenizer, vocab_size, prompt_len, eos_id, top=None)
    c._fresh = lambda: ToolCallPrefix(tools, template.call_open, template.call_close)
    c.state = c._fresh()
    return c


def constraint_from_request(body: dict, tokenizer, vocab_size: int, prompt_len: int, eos_id: int | None):
    """OpenAI `response_format` -> constraint (None when the request asks for plain text)."""
    rf = body.get("response_format") or {}
    kind = rf.get("type") if isinstance(rf, dict) else None
    if kind == "json_object":
        return JsonConstraint(tokenizer, vocab_size, prompt_len, eos_id, top="object")
    if kind == "json_schema":
        schema = (rf.get("json_schema") or {}).get("schema") or {}
        if isinstance(schema.get("enum"), list) and all(isinstance(e, str) for e in schema["enum"]):
            import json
            return ChoiceConstraint(tokenizer, vocab_size, prompt_len, [json.dumps(e) for e in schema["enum"]], eos_id)
        top = {"object": "object", "array": "array"}.get(schema.get("type"))
        enforce = any(k in schema for k in ("properties", "items", "required", "type", "anyOf", "oneOf", "$ref", "const", "pattern"))
        return JsonConstraint(tokenizer, vocab_size, prompt_len, eos_id, top=top, schema=schema if enforce else None)
    if kind == "grammar" or isinstance(body.get("guided_grammar"), str):
        # the completion must be a sentence of an EBNF grammar (vLLM-style `guided_grammar`, or response_format.type = "grammar")
        text = body.get("guided_grammar") or (rf.get("grammar") if isinstance(rf, dict) else None)
        if isinstance(text, str) and text.strip():
            from .grammar import Grammar
            return JsonConstraint(tokenizer, vocab_size, prompt_len, eos_id, grammar=Grammar(text))      # compiled once per request; GrammarError -> 400
    if kind == "regex" or isinstance(body.get("guided_regex"), str):
        # the completion as a whole must match a regular expression (vLLM-style `guided_regex`, or response_format.type = "regex")
        pattern = body.get("guided_regex") or (rf.get("regex") or rf.get("pattern") if isinstance(rf, dict) else None)
        if isinstance(pattern, str) and pattern:
            return JsonConstraint(tokenizer, vocab_size, prompt_len, eos_id, regex=pattern)
    return None


def unpack_bits(words: torch.Tensor, vocab_size: int) -> list[bool]:
    w = words.to(torch.int64) & 0xFFFFFFFF
    return [bool((int(w[i >> 5]) >> (i & 31)) & 1) for i in range(vocab_size)]
