"""EBNF grammars for constrained decoding: parsing, the pushdown recogniser, token masks through the constraint interface."""
import random
import re

import pytest

from cuteafd_b200.serving.constraints import constraint_from_request, unpack_bits
from cuteafd_b200.serving.grammar import Grammar, GrammarError, GrammarPrefix

SQL = r'''
# a toy SELECT statement
root   ::= "SELECT " column (", " column)* " FROM " ident ( " WHERE " cond )? ";"
column ::= ident | "*"
cond   ::= ident " " op " " value
op     ::= "=" | "<" | ">" | "<=" | ">="
value  ::= [0-9]+ | "'" [^'\n]* "'"
ident  ::= [a-zA-Z_] [a-zA-Z0-9_]*
'''

EXPR = r'''
root ::= expr
expr ::= term (("+" | "-") term)*
term ::= factor (("*" | "/") factor)*
factor ::= [0-9]+ | "(" expr ")"
'''


def accepts(g, text):
    p = GrammarPrefix(g)
    return p.feed_text(text) and p.complete


def viable(g, text):
    return GrammarPrefix(g).feed_text(text)


def test_sentences_prefixes_and_rejections():
    g = Grammar(SQL)
    assert accepts(g, "SELECT a, b_2, * FROM t;")
    assert accepts(g, "SELECT x FROM t WHERE x >= 10;") and accepts(g, "SELECT x FROM t WHERE name = 'o k';")
    assert viable(g, "SELECT a, b") and not accepts(g, "SELECT a, b")
    assert not viable(g, "SELECT 1") and not viable(g, "SELECT a FROM t WHERE x => 1")
    assert not viable(g, "select")
    p = GrammarPrefix(g)
    assert p.feed_text("SELECT a FROM t;") and p.complete and p.finished()          # nothing may follow the semicolon
    q = GrammarPrefix(g)
    assert q.feed_text("SELECT a FROM t") and not q.complete and not q.finished()
    # nesting is exact: a pushdown language no regular expression describes
    e = Grammar(EXPR)
    assert accepts(e, "((1+2)*(3-4))/5") and viable(e, "((1+2") and not accepts(e, "((1+2)") and not viable(e, "(1+2))")


def test_repetition_bounds_escapes_and_any_char():
    g = Grammar(r'root ::= "id-" [0-9]{2,4} ("\t" | "\x41" | "é") .{1} "\"" ')
    assert accepts(g, 'id-12\tz"') and accepts(g, 'id-1234Aq"') and accepts(g, 'id-123é!"')
    assert not viable(g, "id-1\t") and not viable(g, "id-12345") and viable(g, "id-12")
    h = Grammar('root ::= ("ab")+ "c"? ')
    assert accepts(h, "abab") and accepts(h, "abc") and not viable(h, "aa") and not accepts(h, "")
    assert accepts(Grammar('root ::= "x"{3}'), "xxx") and not viable(Grammar('root ::= "x"{3}'), "xxxx")
    assert accepts(Grammar('root ::= "x"{2,}'), "xxxxx") and not accepts(Grammar('root ::= "x"{2,}'), "x")


def test_grammar_errors():
    for bad in ('root ::= a', 'r ::= "x"', 'root ::= "x', 'root ::= [a-', 'root ::= ("x"', 'root ::= "a" root2\nroot ::= "b"', 'root ::= root "a" | "b"',
                'root ::= [z-a]', 'root = "x"', 'root ::= "x"{3,2}'):
        with pytest.raises(GrammarError):
            Grammar(bad)


class ByteTok:
    """One token per byte value, plus a few multi-character tokens and the end-of-sequence token."""
    extra = ["SELECT ", " FROM ", ", ", "ab", "  "]

    def decode(self, ids):
        return "".join(self.piece(i) for i in ids)

    def piece(self, i):
        return chr(i) if i < 256 else (self.extra[i - 256] if i - 256 < len(self.extra) else "")

    def convert_ids_to_tokens(self, ids):
        return [self.piece(i) for i in ids]


def test_token_masks_drive_generation_to_a_sentence():
    tok = ByteTok()
    V, eos = 256 + len(ByteTok.extra) + 1, 256 + len(ByteTok.extra)
    rng = random.Random(3)
    done = 0
    for trial in range(6):
        c = constraint_from_request({"guided_grammar": SQL}, tok, V, 0, eos)
        assert c is not None
        toks = []
        for _ in range(200):
            allowed = [i for i, a in enumerate(unpack_bits(c.mask(toks), V)) if a]
            assert allowed
            closing = [a for a in allowed if a == eos or tok.piece(a) in (";", " FROM ", "t")]
            toks.append(rng.choice(closing) if closing and rng.random() < 0.5 else rng.choice(allowed))
            if toks[-1] == eos:
                break
        if toks[-1] == eos:
            text = tok.decode(toks[:-1])
            assert re.fullmatch(r"SELECT .* FROM [a-zA-Z_][a-zA-Z0-9_]*( WHERE .*)?;", text), text
            assert GrammarPrefix(Grammar(SQL)).feed_text(text)
            done += 1
    assert done >= 1
    # response_format form, and a multi-character token that the grammar allows only as a whole
    c = constraint_from_request({"response_format": {"type": "grammar", "grammar": 'root ::= "SELECT " "ab"'}}, tok, V, 0, eos)
    first = [i for i, a in enumerate(unpack_bits(c.mask([]), V)) if a]
    assert set(first) == {ord("S"), 256}
    after = [i for i, a in enumerate(unpack_bits(c.mask([256]), V)) if a]
    assert set(after) == {ord("a"), 259}
    assert [i for i, a in enumerate(unpack_bits(c.mask([256, 259]), V)) if a] == [eos]


def test_integer_bounds_of_a_json_schema():
    from cuteafd_b200.serving.constraints import SchemaSet, _int_prefix_ok
    assert _int_prefix_ok("1", 10, 99) and _int_prefix_ok("9", 10, 99) and not _int_prefix_ok("100", 10, 99) and not _int_prefix_ok("0", 10, 99)
    assert _int_prefix_ok("-", -5, 5) and _int_prefix_ok("-5", -5, 5) and not _int_prefix_ok("-6", -5, 5) and not _int_prefix_ok("-", 1, 5)
    assert _int_prefix_ok("12", 1000, None) and not _int_prefix_ok("12", None, 11) and _int_prefix_ok("-12", None, -100)
    schema = {"type": "object", "properties": {"age": {"type": "integer", "minimum": 18, "maximum": 120}, "delta": {"type": "integer", "exclusiveMinimum": -3, "exclusiveMaximum": 3}},
              "required": ["age"], "additionalProperties": False}

    def ok(text, whole=True):
        st = SchemaSet(schema)
        return st.feed_text(text) and (st.complete or not whole)
    assert ok('{"age": 18}') and ok('{"age":120, "delta": -2}') and ok('{"age": 42,"delta":0}')
    assert not ok('{"age": 17}') and not ok('{"age": 121}') and not ok('{"age": 1}') and not ok('{"age": 30, "delta": 3}') and not ok('{"age": 30, "delta": -3}')
    assert ok('{"age": 1', whole=False) and ok('{"age": 12', whole=False) and not ok('{"age": 13', whole=False) and not ok('{"age": 0', whole=False)
    assert not ok('{"age": -', whole=False) and ok('{"age": 20, "delta": -', whole=False)
    top = SchemaSet({"type": "integer", "minimum": 5, "maximum": 50})
    assert top.feed_text("4") and not top.complete
    top = SchemaSet({"type": "integer", "minimum": 5, "maximum": 50})
    assert top.feed_text("42") and top.complete and not SchemaSet({"type": "integer", "minimum": 5, "maximum": 50}).feed_text("51")


def test_schema_array_sizes_string_lengths_and_number_ranges():
    from cuteafd_b200.serving.constraints import SchemaSet

    def ok(schema, text, whole=True):
        s = SchemaSet(schema)
        r = s.feed_text(text)
        c = s.complete() if callable(s.complete) else s.complete
        return r and (c if whole else True)

    sch = {"type": "object", "additionalProperties": False, "required": ["tags", "score"], "properties": {
        "tags": {"type": "array", "items": {"type": "string", "minLength": 2, "maxLength": 4}, "minItems": 1, "maxItems": 3},
        "score": {"type": "number", "minimum": 0.5, "exclusiveMaximum": 10}}}
    assert ok(sch, '{"tags":["ab","abcd"],"score":9.99}')
    assert not ok(sch, '{"tags":[]', whole=False)                          # fewer than minItems: the bracket cannot close
    assert not ok(sch, '{"tags":["a"]', whole=False)                       # shorter than minLength: the quote cannot close
    assert not ok(sch, '{"tags":["abcde', whole=False)                     # the fifth character is refused
    assert not ok(sch, '{"tags":["ab","cd","ef",', whole=False)            # no comma after maxItems items
    assert ok(sch, '{"tags":["a\\u00e9"],"score":2}')                      # an escape is one code point
    assert not ok(sch, '{"tags":["\\n\\n\\n\\n\\n', whole=False)
    assert ok(sch, '{"tags":["ab"],"score":0.5}') and not ok(sch, '{"tags":["ab"],"score":10}') and ok(sch, '{"tags":["ab"],"score":9.999}')
    assert not ok(sch, '{"tags":["ab"],"score":0.4', whole=False)          # refused at the digit that rules the value out
    assert not ok(sch, '{"tags":["ab"],"score":12', whole=False) and not ok(sch, '{"tags":["ab"],"score":1e', whole=False)
    assert not ok(sch, '{"tags":["ab"],"score":-', whole=False)
    neg = {"type": "number", "minimum": -2.5, "maximum": -0.25}
    assert ok(neg, "-0.25") and ok(neg, "-2.5") and ok(neg, "-1") and not ok(neg, "-0.2") and not ok(neg, "-3", whole=False) and not ok(neg, "1", whole=False)
    assert not ok(neg, "-2.6", whole=False) and ok(neg, "-0.30")
    empty = {"type": "array", "maxItems": 0}
    assert ok(empty, "[]") and not ok(empty, "[1", whole=False)
    nested = {"type": "array", "items": {"type": "array", "items": {"type": "integer"}, "minItems": 2, "maxItems": 2}, "minItems": 1}
    assert ok(nested, "[[1,2],[3,4]]") and not ok(nested, "[[1]", whole=False) and not ok(nested, "[[1,2,", whole=False)
