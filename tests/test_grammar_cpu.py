"""Grammar engine: JSON-schema / regex matching and token masks vs brute force."""
import json

import numpy as np
import pytest

from ds41rt_b200.runtime.grammar import (Grammar, GrammarError, Matcher, TokenConstraint, Vocab, mask_allows)

SCHEMA8 = {
    "type": "object",
    "properties": {
        "name": {"type": "string"},
        "age": {"type": "integer"},
        "tier": {"enum": ["free", "pro", "enterprise"]},
        "active": {"type": "boolean"},
        "score": {"type": "number"},
        "tags": {"type": "array", "items": {"type": "string"}, "maxItems": 3},
        "address": {"type": "object",
                    "properties": {"city": {"type": "string"}, "zip": {"type": "string", "pattern": "[0-9]{5}"}},
                    "required": ["city", "zip"]},
        "note": {"type": ["string", "null"]},
    },
    "required": ["name", "age", "tier", "active", "address"],
}


def _ok(g, text):
    return Matcher(g).accept_bytes(text.encode()) 


def _complete(g, text):
    m = Matcher(g)
    return m.accept_bytes(text.encode()) and m.can_finish


def test_schema_accepts_valid_documents_and_rejects_invalid():
    g = Grammar.json_schema(SCHEMA8)
    good = {"name": "Ada", "age": 36, "tier": "pro", "active": True, "score": -1.5e3, "tags": ["a", "b"],
            "address": {"city": "Paris", "zip": "75001"}, "note": None}
    assert _complete(g, json.dumps(good))
    assert _complete(g, json.dumps(good, indent=2))
    minimal = {"name": "x", "age": 0, "tier": "free", "active": False, "address": {"city": "", "zip": "00000"}}
    assert _complete(g, json.dumps(minimal))
    assert not _complete(g, json.dumps({k: v for k, v in minimal.items() if k != "age"}))     # required missing
    bad = dict(minimal, tier="gold")
    assert not _complete(g, json.dumps(bad))
    bad = dict(minimal, age=1.5)
    assert not _complete(g, json.dumps(bad))
    bad = dict(minimal, address={"city": "x", "zip": "123"})
    assert not _complete(g, json.dumps(bad))
    bad = dict(good, tags=["a", "b", "c", "d"])
    assert not _complete(g, json.dumps(bad))
    assert not _complete(g, json.dumps(good)[:-1])            # prefix is accepted but cannot finish
    assert _ok(g, json.dumps(good)[:-1])
    assert not _ok(g, '{"age"')                                # declared order: name comes first
    assert not _ok(g, "{" + " " * 17)                          # whitespace bounded to 16


def test_refs_anyof_and_free_form():
    schema = {"$defs": {"node": {"type": "object", "properties": {"v": {"type": "integer"},
                                                                    "next": {"anyOf": [{"$ref": "#/$defs/node"},
                                                                                       {"type": "null"}]}},
                                 "required": ["v", "next"]}},
              "$ref": "#/$defs/node"}
    g = Grammar.json_schema(schema)
    assert _complete(g, '{"v":1,"next":{"v":2,"next":null}}')
    assert not _complete(g, '{"v":1,"next":{"v":2}}')
    any_obj = Grammar.json_object()
    assert _complete(any_obj, '{"a":[1,2,{"b":"c\\n"}],"d":{}}')
    assert not _complete(any_obj, '[1]')
    with pytest.raises(GrammarError):
        Grammar.json_schema({"type": "frobnicate"})
    with pytest.raises(GrammarError):
        Grammar("{not json")


def test_regex_and_until():
    g = Grammar.regex(r"(foo|ba+r)-[0-9]{2,3}\.[a-c]?x")
    assert _complete(g, "foo-12.x") and _complete(g, "baaar-123.bx")
    assert not _complete(g, "foo-1.x") and not _complete(g, "bar-1234.x") and not _complete(g, "foo-12.dx")
    u = Grammar({"seq": [{"until": "</end>"}, {"lit": "!"}]})
    assert _complete(u, "free <text </en </end>!")
    assert not _complete(u, "abc</end>?")
    m = Matcher(u)
    assert m.accept_bytes(b"abc</end>") and not m.can_finish and m.accept_bytes(b"!") and m.terminated


def _toy_vocab():
    pieces = ['{', '}', '"', ':', ',', ' ', '\n', '{"', '":', '",', 'name', 'age', 'tier', 'active', 'address', 'city',
              'zip', 'true', 'false', 'null', 'free', 'pro', 'enterprise', 'A', 'da', '0', '1', '23', '75001', '-',
              '.', 'e', '[', ']', '"}', '"name"', 'x' * 3, 'tru', 'e,', '": "', '{"name": "']
    toks = [b""] + [p.encode() for p in pieces]          # id 0 = EOS (no bytes)
    return Vocab(toks), toks


def test_token_mask_equals_brute_force_and_fork_is_independent():
    vocab, toks = _toy_vocab()
    g = Grammar.json_schema(SCHEMA8)
    m = Matcher(g)
    rng = np.random.default_rng(0)
    steps = 0
    while steps < 60 and not m.terminated:
        mask = m.fill_mask(vocab, stop_token=0)
        brute = [i for i in range(1, vocab.size) if m.fork().accept_bytes(toks[i])]
        got = [i for i in range(1, vocab.size) if mask_allows(mask, i)]
        assert got == brute
        assert mask_allows(mask, 0) == m.can_finish
        if not brute:
            break
        f = m.fork()
        pick = int(rng.choice(brute))
        assert m.accept_token(vocab, pick)
        assert f.fill_mask(vocab, 0).tolist() == mask.tolist()        # the fork did not move
        steps += 1
    assert steps > 10


def test_token_constraint_thinking_and_proposals():
    vocab, toks = _toy_vocab()
    think_end = vocab.size - 1
    ids = {t: i for i, t in enumerate(toks)}
    g = Grammar.json_schema({"type": "object", "properties": {"name": {"type": "string"}}, "required": ["name"]})
    c = TokenConstraint(vocab, g, eos=0, think_end=think_end, thinking=True)
    m = c.mask()
    assert not mask_allows(m, 0) and mask_allows(m, 5) and mask_allows(m, think_end)
    assert c.accept(ids[b"pro"]) and c.accept(think_end) and not c.in_thinking
    m = c.mask()
    assert mask_allows(m, ids[b'{']) and mask_allows(m, ids[b'{"']) and not mask_allows(m, ids[b'pro'])
    seq = [ids[b'{"'], ids[b'name'], ids[b'":'], ids[b'"'], ids[b'A'], ids[b'"}']]
    assert c.truncate_proposal(seq + [ids[b'pro']]) == seq            # trimmed at the first rejected token only
    assert c.accept(seq[0])                                            # the anchor is committed first
    masks = c.row_masks(seq[:3])
    assert len(masks) == 3 and mask_allows(masks[0], ids[b'name']) and mask_allows(masks[2], ids[b'"'])
    for t in seq[1:]:
        assert c.accept(t)
    assert mask_allows(c.mask(), 0) and c.accept(0) and c.finished


def test_triggered_tool_grammar_leaves_text_free_until_the_tag():
    """tool_choice "auto": plain text of any kind completes; once the opening tag of a calls block is written, only a
    well-formed block for a declared tool completes; masks along the way equal brute force (and repeat from the cache)."""
    from ds41rt_b200.serving import chat as C
    from ds41rt_b200.serving.http import tool_call_grammar
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}},
        "required": ["city"]}}}]
    g = Grammar(tool_call_grammar(tools, "auto", parallel=False, triggered=True))
    assert _complete(g, "") and _complete(g, "It is sunny. <not a tag> 1 < 2")
    assert _complete(g, "partial tag " + C.CALLS_OPEN[:-1])            # a prefix of the tag is still just text
    call = (f'{C.CALLS_OPEN}\n{C.DSML_OPEN} invoke name="get_weather">\n'
            f'{C.DSML_OPEN} parameter name="city" string="true">Paris{C.DSML_CLOSE} parameter>\n'
            f'{C.DSML_OPEN} parameter name="days" string="false">3{C.DSML_CLOSE} parameter>\n'
            f'{C.DSML_CLOSE} invoke>\n{C.CALLS_CLOSE}')
    assert _complete(g, "Let me check. " + call)
    m = Matcher(g)
    assert m.accept_bytes(("text " + C.CALLS_OPEN).encode()) and not m.can_finish          # the block must now be finished
    assert not _ok(g, "x " + C.CALLS_OPEN + "\n" + f'{C.DSML_OPEN} invoke name="unknown_tool">')
    assert not _complete(g, call + " trailing text")
    # token masks: a vocabulary with text pieces, tag pieces and a token that spans the tag boundary
    pieces = ["It", " is", " sunny", ".", C.CALLS_OPEN, C.CALLS_OPEN[:3], C.CALLS_OPEN[3:], "\n", "x" + C.CALLS_OPEN + "y",
              f'{C.DSML_OPEN} invoke name="get_weather">\n', f'{C.DSML_OPEN} invoke name="nope">\n', "Paris", " parameter>\n"]
    toks = [b""] + [p.encode() for p in pieces]
    vocab = Vocab(toks)
    m = Matcher(g)
    for text in ("It", " is", C.CALLS_OPEN[:3], C.CALLS_OPEN[3:], "\n"):
        for _ in range(2):                                            # second fill comes from the state cache
            mask = m.fill_mask(vocab, stop_token=0)
            brute = [i for i in range(1, vocab.size) if m.fork().accept_bytes(toks[i])]
            assert [i for i in range(1, vocab.size) if mask_allows(mask, i)] == brute
            assert mask_allows(mask, 0) == m.can_finish
        assert m.accept_bytes(text.encode())
    mask = m.fill_mask(vocab, stop_token=0)
    allowed = [pieces[i - 1] for i in range(1, vocab.size) if mask_allows(mask, i)]
    # inside the block only the declared tool's invoke line can follow (or a piece that is a prefix of it)
    assert f'{C.DSML_OPEN} invoke name="get_weather">\n' in allowed and not mask_allows(mask, 0)
    assert all(f'{C.DSML_OPEN} invoke name="get_weather">\n'.startswith(p) for p in allowed)


def _random_schema(rng, depth=0):
    """A schema from the supported subset and a generator of valid instances for it."""
    kinds = ["string", "integer", "number", "boolean", "null", "enum", "nullable"]
    if depth < 3:
        kinds += ["object", "object", "array", "anyOf"]
    kind = kinds[rng.integers(len(kinds))]
    if kind == "string":
        alphabet = ["a", "Z", " ", "é", "✓", '"', "\\", "\n", "\t", "/", "0", "😀"]
        return {"type": "string"}, lambda: "".join(alphabet[i] for i in rng.integers(len(alphabet), size=rng.integers(0, 6)))
    if kind == "integer":
        return {"type": "integer"}, lambda: int(rng.integers(-10 ** 6, 10 ** 6)) if rng.random() < 0.8 else 0
    if kind == "number":
        return {"type": "number"}, lambda: [0.5, -1.25e-7, 3.0e12, 7, -0.0, 1e-05][rng.integers(6)]
    if kind == "boolean":
        return {"type": "boolean"}, lambda: bool(rng.integers(2))
    if kind == "null":
        return {"type": "null"}, lambda: None
    if kind == "enum":
        values = [["red", "green", "blue"], [1, 2, 3], ["a b", "a"], [True, None, "x"]][rng.integers(4)]
        return {"enum": values}, lambda: values[rng.integers(len(values))]
    if kind == "nullable":
        return {"type": ["integer", "null"]}, lambda: None if rng.random() < 0.5 else int(rng.integers(100))
    if kind == "array":
        item, gen = _random_schema(rng, depth + 1)
        cap = int(rng.integers(1, 4))
        return {"type": "array", "items": item, "maxItems": cap}, lambda: [gen() for _ in range(rng.integers(0, cap + 1))]
    if kind == "anyOf":
        (a, ga), (b, gb) = _random_schema(rng, depth + 1), _random_schema(rng, depth + 1)
        return {"anyOf": [a, b]}, lambda: ga() if rng.random() < 0.5 else gb()
    names = [f"k{i}" for i in range(rng.integers(1, 5))]
    parts = {n: _random_schema(rng, depth + 1) for n in names}
    required = [n for n in names if rng.random() < 0.6]
    schema = {"type": "object", "properties": {n: parts[n][0] for n in names}, "required": required}

    def gen():
        return {n: parts[n][1]() for n in names if n in required or rng.random() < 0.5}      # declared order
    return schema, gen


def test_random_schemas_accept_their_instances_byte_by_byte_and_refuse_broken_ones():
    """Property test over the supported schema subset: every generated instance is accepted with every one of its byte
    prefixes on the way, compact or indented, ASCII-escaped or raw UTF-8; a truncated document cannot finish; a document
    without one of its required properties, or with a value of another type in place of a leaf, is refused."""
    rng = np.random.default_rng(11)
    docs = broken = 0
    for _ in range(60):
        schema, gen = _random_schema(rng, 0)
        if schema.get("type") != "object":
            schema, gen = {"type": "object", "properties": {"v": schema}, "required": ["v"]}, (lambda g=gen: {"v": g()})
        g = Grammar.json_schema(schema)
        for _ in range(4):
            value = gen()
            for text in (json.dumps(value), json.dumps(value, ensure_ascii=False), json.dumps(value, indent=1)):
                data = text.encode()
                m = Matcher(g)
                for i in range(len(data)):
                    assert m.accept_bytes(data[i:i + 1]), (schema, text, i)
                    if i < len(data) - 1:
                        assert not m.can_finish or text[: i + 1].rstrip() != text[: i + 1], (schema, text, i)
                assert m.can_finish, (schema, text)
                docs += 1
            for name in schema["required"]:
                cut = {k: v for k, v in value.items() if k != name}
                assert not _complete(g, json.dumps(cut)), (schema, cut)
                broken += 1
            for name, sub in schema["properties"].items():
                if name in value and sub.get("type") in ("integer", "boolean", "null", "string"):
                    wrong = {"integer": "7", "boolean": 1, "null": 0, "string": 5}[sub["type"]]
                    assert not _complete(g, json.dumps(dict(value, **{name: wrong}))), (schema, name)
                    broken += 1
    assert docs >= 700 and broken > 100
