"""Context-free grammars for constrained decoding: an EBNF dialect compiled to a character-level pushdown recogniser.

Grammar text (the GBNF / xgrammar-EBNF dialect: one rule per `name ::= ...`, the start rule is `root`):

    root   ::= "SELECT " column (", " column)* " FROM " ident ";"
    column ::= ident | "*"
    ident  ::= [a-zA-Z_] [a-zA-Z0-9_]*

Elements: "literals" (escapes \\n \\t \\r \\" \\\\ \\xHH \\uHHHH), character classes `[a-z0-9_]` / `[^"\\\\]`, `.` (any character), rule
names, groups `( ... )`, alternation `|`, postfix `*` `+` `?` and `{m}` / `{m,}` / `{m,n}`; `#` starts a comment.  Rules may span
lines; a new rule starts at `name ::=`.

The recogniser keeps the set of parse stacks that are consistent with the text so far (each stack a tuple of positions inside rule
alternatives, expanded until its top is a terminal), so ambiguity and nesting are exact; left recursion is rejected at compile time.
`GrammarPrefix` has the interface of the other prefix automata of `serving.constraints` (copy / signature / feed_text / complete /
finished), so token masks, caching by state and rollback come from `JsonConstraint`.

Reference: native/shared/src/xgrammar_adapter.cc (EBNF / regex / JSON-schema grammars compiled by the xgrammar library and applied
as token bitmasks); the grammar engine here is this repository's own.
"""
from __future__ import annotations

MAX_STACK = 256          # parse stacks deeper than this are dropped (runaway recursion on pathological input)
MAX_STATES = 4096        # and a text that keeps more alternatives than this alive is refused


class GrammarError(ValueError):
    pass


# element kinds inside an alternative: ("c", frozenset of code points | None, ranges tuple, negated) | ("r", rule index)
def _lit(ch: str):
    return ("c", frozenset((ord(ch),)), (), False)


class _Parser:
    def __init__(self, text: str):
        self.s, self.i = text, 0
        self.rules: list[list[list[tuple]]] = []        # rule -> alternatives -> elements
        self.names: dict[str, int] = {}
        self.pending: list[tuple[str, int]] = []         # (name, position) of references, checked at the end

    # ---- lexical helpers
    def _ws(self, newlines: bool = True):
        s = self.s
        while self.i < len(s):
            c = s[self.i]
            if c == "#":
                while self.i < len(s) and s[self.i] != "\n":
                    self.i += 1
            elif c in " \t\r" or (newlines and c == "\n"):
                self.i += 1
            else:
                break

    def _name(self) -> str | None:
        s, j = self.s, self.i
        if j < len(s) and (s[j].isalpha() or s[j] == "_"):
            while j < len(s) and (s[j].isalnum() or s[j] in "_-"):
                j += 1
            name, self.i = s[self.i:j], j
            return name
        return None

    def _rule_id(self, name: str) -> int:
        if name not in self.names:
            self.names[name] = len(self.rules)
            self.rules.append(None)
        return self.names[name]

    def _new_rule(self, alts) -> int:
        self.rules.append(alts)
        return len(self.rules) - 1

    def _escape(self) -> str:
        s = self.s
        c = s[self.i]
        self.i += 1
        if c != "\\":
            return c
        if self.i >= len(s):
            raise GrammarError("dangling backslash")
        e = s[self.i]
        self.i += 1
        if e in "nrt":
            return {"n": "\n", "r": "\r", "t": "\t"}[e]
        if e in "xuU":
            n = {"x": 2, "u": 4, "U": 8}[e]
            h = s[self.i:self.i + n]
            if len(h) != n or any(ch not in "0123456789abcdefABCDEF" for ch in h):
                raise GrammarError(f"bad \\{e} escape at {self.i}")
            self.i += n
            return chr(int(h, 16))
        return e                                             # \" \\ \[ \] \- and friends stand for themselves

    # ---- grammar
    def parse(self):
        self._ws()
        while self.i < len(self.s):
            name = self._name()
            if name is None:
                raise GrammarError(f"rule name expected at offset {self.i}")
            self._ws(newlines=False)
            if not self.s.startswith("::=", self.i):
                raise GrammarError(f"'::=' expected after {name!r}")
            self.i += 3
            rid = self._rule_id(name)
            if self.rules[rid] is not None:
                raise GrammarError(f"rule {name!r} defined twice")
            self.rules[rid] = self._alternatives(top=True)
            self._ws()
        for name, rid in self.names.items():
            if self.rules[rid] is None:
                raise GrammarError(f"rule {name!r} is used but never defined")
        if "root" not in self.names:
            raise GrammarError("the grammar needs a rule named 'root'")
        return self.rules, self.names["root"]

    def _at_rule_start(self) -> bool:
        """Is the parser looking at `name ::=` (the start of the next rule)?"""
        save = self.i
        name = self._name()
        ok = False
        if name is not None:
            self._ws(newlines=False)
            ok = self.s.startswith("::=", self.i)
        self.i = save
        return ok

    def _alternatives(self, top: bool = False):
        alts = [self._sequence(top)]
        while True:
            self._ws(newlines=True)
            if self.i < len(self.s) and self.s[self.i] == "|":
                self.i += 1
                alts.append(self._sequence(top))
            else:
                return alts

    def _sequence(self, top: bool):
        seq: list[tuple] = []
        while True:
            self._ws(newlines=True)
            if self.i >= len(self.s) or self.s[self.i] in "|)":
                return seq
            if top and self._at_rule_start():
                return seq
            start = len(seq)
            c = self.s[self.i]
            if c == '"':
                self.i += 1
                while True:
                    if self.i >= len(self.s):
                        raise GrammarError("unterminated string literal")
                    if self.s[self.i] == '"':
                        self.i += 1
                        break
                    seq.append(_lit(self._escape()))
            elif c == "[":
                seq.append(self._char_class())
            elif c == ".":
                self.i += 1
                seq.append(("c", None, (), True))              # everything but nothing = any character
            elif c == "(":
                self.i += 1
                alts = self._alternatives()
                self._ws()
                if self.i >= len(self.s) or self.s[self.i] != ")":
                    raise GrammarError("')' expected")
                self.i += 1
                seq.append(("r", self._new_rule(alts)))
            else:
                name = self._name()
                if name is None:
                    raise GrammarError(f"unexpected {c!r} at offset {self.i}")
                seq.append(("r", self._rule_id(name)))
            self._postfix(seq, start)

    def _char_class(self):
        self.i += 1
        neg = self.i < len(self.s) and self.s[self.i] == "^"
        if neg:
            self.i += 1
        singles, ranges = set(), []
        while True:
            if self.i >= len(self.s):
                raise GrammarError("unterminated character class")
            if self.s[self.i] == "]":
                self.i += 1
                break
            lo = self._escape()
            if self.i + 1 < len(self.s) and self.s[self.i] == "-" and self.s[self.i + 1] != "]":
                self.i += 1
                hi = self._escape()
                if ord(hi) < ord(lo):
                    raise GrammarError(f"reversed range {lo}-{hi}")
                ranges.append((ord(lo), ord(hi)))
            else:
                singles.add(ord(lo))
        return ("c", frozenset(singles), tuple(ranges), neg)

    def _postfix(self, seq: list, start: int):
        """Applies * + ? {m,n} to the element(s) appended since `start` (a multi-character literal repeats as a whole)."""
        while self.i < len(self.s) and self.s[self.i] in "*+?{":
            op = self.s[self.i]
            item = seq[start:]
            del seq[start:]
            unit = item if len(item) != 1 else item
            if op == "{":
                j = self.s.find("}", self.i)
                if j < 0:
                    raise GrammarError("unterminated repetition")
                body = self.s[self.i + 1:j].replace(" ", "")
                self.i = j + 1
                try:
                    if "," in body:
                        lo_s, hi_s = body.split(",", 1)
                        lo, hi = int(lo_s or 0), (int(hi_s) if hi_s else None)
                    else:
                        lo = hi = int(body)
                except ValueError:
                    raise GrammarError(f"bad repetition {{{body}}}") from None
                if hi is not None and hi < lo:
                    raise GrammarError(f"bad repetition {{{body}}}")
                out = list(unit) * lo
                if hi is None:
                    out.append(("r", self._star(unit)))
                else:
                    opt = None                                 # nested optionals: (x (x (x)?)?)?
                    for _ in range(hi - lo):
                        inner = list(unit) + ([("r", opt)] if opt is not None else [])
                        opt = self._new_rule([inner, []])
                    if opt is not None:
                        out.append(("r", opt))
                seq.extend(out)
            else:
                self.i += 1
                if op == "*":
                    seq.append(("r", self._star(unit)))
                elif op == "+":
                    seq.extend(list(unit) + [("r", self._star(unit))])
                else:
                    seq.append(("r", self._new_rule([list(unit), []])))

    def _star(self, unit) -> int:
        rid = self._new_rule(None)
        self.rules[rid] = [list(unit) + [("r", rid)], []]
        return rid


def _nullable_and_left(rules):
    """Nullable rules, and a check that no rule can reach itself without consuming a character."""
    nullable = [False] * len(rules)
    changed = True
    while changed:
        changed = False
        for r, alts in enumerate(rules):
            if not nullable[r] and any(all(e[0] == "r" and nullable[e[1]] for e in alt) for alt in alts):
                nullable[r] = changed = True
    first: list[set] = [set() for _ in rules]               # rules reachable at the left edge
    for r, alts in enumerate(rules):
        for alt in alts:
            for e in alt:
                if e[0] != "r":
                    break
                first[r].add(e[1])
                if not nullable[e[1]]:
                    break
    for r in range(len(rules)):
        seen, todo = set(), list(first[r])
        while todo:
            x = todo.pop()
            if x == r:
                raise GrammarError("left-recursive rule (a rule reaches itself before consuming a character)")
            if x not in seen:
                seen.add(x)
                todo.extend(first[x])


class Grammar:
    """A compiled grammar: immutable, shared by every `GrammarPrefix` of a request."""

    def __init__(self, text: str):
        self.rules, self.root = _Parser(text).parse()
        _nullable_and_left(self.rules)

    def start(self) -> frozenset:
        out: set = set()
        for a in range(len(self.rules[self.root])):
            self._expand(((self.root, a, 0),), out, set())
        return frozenset(out)

    def _expand(self, stack: tuple, out: set, seen: set):
        """Adds to `out` every stack reachable from `stack` without consuming input whose top is a terminal (or that is empty)."""
        if stack in seen or len(stack) > MAX_STACK:
            return
        seen.add(stack)
        if not stack:
            out.add(stack)
            return
        r, a, i = stack[-1]
        alt = self.rules[r][a]
        if i == len(alt):
            self._expand(stack[:-1], out, seen)
            return
        e = alt[i]
        if e[0] == "r":
            base = stack[:-1] + (((r, a, i + 1),) if i + 1 < len(alt) else ())      # a finished parent leaves the stack now (tail call)
            for a2 in range(len(self.rules[e[1]])):
                self._expand(base + ((e[1], a2, 0),), out, seen)
        else:
            out.add(stack)

    @staticmethod
    def _matches(e: tuple, cp: int) -> bool:
        _, singles, ranges, neg = e
        if singles is None:
            return True
        hit = cp in singles or any(lo <= cp <= hi for lo, hi in ranges)
        return hit != neg

    def step(self, states: frozenset, ch: str) -> frozenset:
        cp, out, seen = ord(ch), set(), set()
        for stack in states:
            if not stack:
                continue
            r, a, i = stack[-1]
            alt = self.rules[r][a]
            if self._matches(alt[i], cp):
                nxt = stack[:-1] + (((r, a, i + 1),) if i + 1 < len(alt) else ())
                self._expand(nxt, out, seen)
        if len(out) > MAX_STATES:
            raise GrammarError("the grammar keeps too many alternatives alive on this text")
        return frozenset(out)


class GrammarPrefix:
    """The completion must be a sentence of the grammar (`guided_grammar` requests, `response_format.type == "grammar"`)."""

    def __init__(self, grammar: "Grammar | str"):
        self.g = grammar if isinstance(grammar, Grammar) else Grammar(grammar)
        self.states = self.g.start()

    def copy(self):
        c = GrammarPrefix.__new__(GrammarPrefix)
        c.g, c.states = self.g, self.states
        return c

    def signature(self):
        return self.states

    def feed_text(self, text: str) -> bool:
        for ch in text:
            if not self.states:
                return False
            self.states = self.g.step(self.states, ch)
        return bool(self.states)

    @property
    def complete(self) -> bool:
        return () in self.states

    def finished(self) -> bool:
        return self.states == frozenset(((),))
