"""Chat template rendering, streamed-output parsing and DSML tool calls.

Prompt format (reference: rust/crates/ds41rt-api/src/encoding.rs:6-45,95-140, native_v41/tools.rs:29-62,196-208):
    <BOS>[system text]<｜User｜>user text<｜Assistant｜><think>reasoning</think>answer<EOS><｜User｜>...
A request with thinking enabled ends the prompt with `<｜Assistant｜><think>`; otherwise with
`<｜Assistant｜></think>` so the model starts directly with the answer.  `Reasoning Effort: N` may precede the system text.
Tool calls are DSML blocks:
    <｜DSML｜ calls>
    <｜DSML｜ invoke name="fn">
    <｜DSML｜ parameter name="k" string="true|false">value</｜DSML｜ parameter>
    </｜DSML｜ invoke>
    </｜DSML｜ calls>
String parameters are raw text (must not contain `</｜DSML｜`), all others JSON.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

BOS_TEXT = "<｜begin▁of▁sentence｜>"
EOS_TEXT = "<｜end▁of▁sentence｜>"
USER, ASSISTANT = "<｜User｜>", "<｜Assistant｜>"
THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
DSML_OPEN, DSML_CLOSE = "<｜DSML｜", "</｜DSML｜"
CALLS_OPEN = f"{DSML_OPEN} calls>"
CALLS_CLOSE = f"{DSML_CLOSE} calls>"
EFFORT_LEVELS = {"none": None, "low": 1, "high": 3, "max": 4}


class ChatError(ValueError):
    pass


def _text_of(content) -> Tuple[str, List[str]]:
    """OpenAI content (string or parts) -> (text with image placeholders, image urls)."""
    if content is None:
        return "", []
    if isinstance(content, str):
        return content, []
    if not isinstance(content, list):
        raise ChatError("message content must be a string or a list of parts")
    text, images = [], []
    for part in content:
        if not isinstance(part, dict):
            raise ChatError("content part must be an object")
        if part.get("type") == "text":
            text.append(str(part.get("text", "")))
        elif part.get("type") == "image_url":
            url = part.get("image_url", {})
            url = url.get("url") if isinstance(url, dict) else url
            if not isinstance(url, str):
                raise ChatError("image_url part needs a url")
            images.append(url)
            text.append("<image>")
        else:
            raise ChatError(f"unsupported content part type {part.get('type')!r}")
    return "".join(text), images


def render_tool_call(name: str, arguments: dict) -> str:
    lines = [CALLS_OPEN, f'{DSML_OPEN} invoke name="{name}">']
    for k, v in arguments.items():
        if isinstance(v, str):
            lines.append(f'{DSML_OPEN} parameter name="{k}" string="true">{v}{DSML_CLOSE} parameter>')
        else:
            lines.append(f'{DSML_OPEN} parameter name="{k}" string="false">{json.dumps(v)}{DSML_CLOSE} parameter>')
    lines += [f"{DSML_CLOSE} invoke>", CALLS_CLOSE]
    return "\n".join(lines)


def render_tools_preamble(tools: List[dict]) -> str:
    if not tools:
        return ""
    out = ["## Tools", "You may call the following functions by emitting a DSML calls block.", ""]
    for t in tools:
        fn = t.get("function", t)
        out.append(json.dumps({"name": fn.get("name"), "description": fn.get("description", ""),
                               "parameters": fn.get("parameters", {})}, ensure_ascii=False))
    return "\n".join(out) + "\n"


def render_conversation(messages: List[dict], tools: Optional[List[dict]] = None, thinking: bool = True,
                        reasoning_effort: Optional[str] = None) -> Tuple[str, List[str]]:
    """-> (prompt text including BOS, image sources in order of appearance)."""
    if not isinstance(messages, list) or not messages:
        raise ChatError("messages must be a non-empty list")
    system, images = [], []
    body = []
    for m in messages:
        if not isinstance(m, dict) or "role" not in m:
            raise ChatError("every message needs a role")
        role = m["role"]
        text, imgs = _text_of(m.get("content"))
        images += imgs
        if role == "system" or role == "developer":
            system.append(text)
        elif role == "user":
            body.append(USER + text)
        elif role == "assistant":
            piece = ASSISTANT
            if m.get("reasoning_content"):
                piece += THINK_OPEN + str(m["reasoning_content"]) + THINK_CLOSE
            else:
                piece += THINK_CLOSE
            piece += text
            for call in m.get("tool_calls") or []:
                fn = call.get("function", {})
                args = fn.get("arguments", "{}")
                args = json.loads(args) if isinstance(args, str) else args
                piece += "\n" + render_tool_call(fn.get("name", ""), args)
            body.append(piece + EOS_TEXT)
        elif role == "tool":
            body.append(USER + f"<tool_result id=\"{m.get('tool_call_id', '')}\">" + text + "</tool_result>")
        else:
            raise ChatError(f"unknown role {role!r}")
    if messages[-1]["role"] == "assistant":
        raise ChatError("the last message must not be from the assistant")
    head = BOS_TEXT
    level = EFFORT_LEVELS.get(reasoning_effort or "", "missing") if reasoning_effort else None
    if level == "missing":
        raise ChatError("reasoning_effort must be one of none, low, high, max")
    if level is not None:
        head += f"Reasoning Effort: {level}\n"
    head += render_tools_preamble(tools or []) + "\n".join(s for s in system if s)
    tail = ASSISTANT + (THINK_OPEN if thinking else THINK_CLOSE)
    return head + "".join(body) + tail, images


# ---------------------------------------------------------------------------------------------- tool calls
_INVOKE = re.compile(re.escape(DSML_OPEN) + r' invoke name="([^"]*)">\n?(.*?)' + re.escape(DSML_CLOSE) + r" invoke>", re.S)
_PARAM = re.compile(re.escape(DSML_OPEN) + r' parameter name="([^"]*)" string="(true|false)">(.*?)' +
                    re.escape(DSML_CLOSE) + r" parameter>", re.S)


def loads_strict(text: str):
    """json.loads that refuses an object with the same property twice (compared after unescaping, so "a" and "\\u0061"
    collide) instead of keeping the last value - the reader the reference uses for completed arguments and answers
    (docs/release-v1-tool-serving.md of the reference, "rejects duplicate properties, including escaped aliases")."""
    def pairs(items):
        out = {}
        for k, v in items:
            if k in out:
                raise ValueError(f"duplicate property {k!r}")
            out[k] = v
        return out
    return json.loads(text, object_pairs_hook=pairs)


def parse_tool_calls(block: str) -> List[dict]:
    """DSML calls block -> OpenAI tool_calls entries.  Raises ChatError on malformed blocks."""
    if CALLS_OPEN not in block or CALLS_CLOSE not in block:
        raise ChatError("unterminated DSML calls block")
    inner = block[block.index(CALLS_OPEN) + len(CALLS_OPEN): block.rindex(CALLS_CLOSE)]
    calls = []
    for name, body in _INVOKE.findall(inner):
        args = {}
        for key, is_str, val in _PARAM.findall(body):
            if key in args:
                raise ChatError(f"parameter {key!r} of {name!r} is given twice")
            if is_str == "true":
                args[key] = val
            else:
                try:
                    args[key] = loads_strict(val)
                except ValueError as e:                   # JSONDecodeError is a ValueError; so is a duplicate property
                    raise ChatError(f"parameter {key!r} of {name!r} is not valid JSON: {e}")
        calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                      "function": {"name": name, "arguments": json.dumps(args, ensure_ascii=False)}})
    if not calls:
        raise ChatError("DSML calls block contains no invoke")
    return calls


def validate_tool_calls(calls: List[dict], tools: List[dict]) -> Optional[str]:
    """Post-hoc validation against the declared tool schemas (names, required arguments, JSON-schema types).
    Returns an error string or None."""
    from ..runtime.grammar import Grammar, GrammarError, Matcher
    by_name = {(t.get("function", t)).get("name"): t.get("function", t) for t in tools}
    for c in calls:
        fn = c["function"]
        if fn["name"] not in by_name:
            return f"call to undeclared tool {fn['name']!r}"
        schema = by_name[fn["name"]].get("parameters")
        if schema:
            try:
                m = Matcher(Grammar.json_schema(schema))
            except GrammarError:
                continue
            doc = json.loads(fn["arguments"])
            props = list((schema.get("properties") or {}).keys())
            ordered = {k: doc[k] for k in props if k in doc}
            ordered.update({k: v for k, v in doc.items() if k not in ordered})
            if not (m.accept_bytes(json.dumps(ordered).encode()) and m.can_finish):
                return f"arguments of {fn['name']!r} do not satisfy the declared schema"
    return None


def validate_json_output(text: str, schema: Optional[dict]) -> Optional[str]:
    from ..runtime.grammar import Grammar, Matcher
    try:
        loads_strict(text)
    except ValueError as e:
        return f"output is not valid JSON: {e}"
    if schema is not None:
        m = Matcher(Grammar.json_schema(schema))
        if not (m.accept_bytes(text.encode()) and m.can_finish):
            return "output does not satisfy the response schema"
    return None


# ---------------------------------------------------------------------------------------------- stream parser
@dataclass
class Delta:
    reasoning: str = ""
    content: str = ""
    tool_calls: List[dict] = field(default_factory=list)


class StreamParser:
    """Splits generated text into reasoning, content and tool calls as it streams.

    Text up to `</think>` is reasoning (when the request started inside a thinking block); a DSML calls block is
    withheld until it is complete and then parsed; text that could be the start of a marker is held back."""

    def __init__(self, thinking: bool):
        self.in_reasoning = thinking
        self.buf = ""
        self.in_calls = False
        self.tool_calls: List[dict] = []

    @staticmethod
    def _held(text: str, markers) -> int:
        """Length of the longest suffix of text that is a proper prefix of a marker."""
        best = 0
        for mk in markers:
            for n in range(min(len(mk) - 1, len(text)), 0, -1):
                if text.endswith(mk[:n]):
                    best = max(best, n)
                    break
        return best

    def push(self, text: str, final: bool = False) -> Delta:
        self.buf += text
        d = Delta()
        while True:
            if self.in_reasoning:
                i = self.buf.find(THINK_CLOSE)
                if i >= 0:
                    d.reasoning += self.buf[:i]
                    self.buf = self.buf[i + len(THINK_CLOSE):]
                    self.in_reasoning = False
                    continue
                hold = 0 if final else self._held(self.buf, [THINK_CLOSE])
                d.reasoning += self.buf[: len(self.buf) - hold]
                self.buf = self.buf[len(self.buf) - hold:]
                return d
            if self.in_calls:
                i = self.buf.find(CALLS_CLOSE)
                if i >= 0:
                    block = self.buf[: i + len(CALLS_CLOSE)]
                    self.buf = self.buf[i + len(CALLS_CLOSE):]
                    calls = parse_tool_calls(block)
                    self.tool_calls += calls
                    d.tool_calls += calls
                    self.in_calls = False
                    continue
                if final:
                    raise ChatError("generation ended inside a DSML calls block")
                return d
            i = self.buf.find(CALLS_OPEN)
            if i >= 0:
                d.content += self.buf[:i]
                self.buf = self.buf[i:]
                self.in_calls = True
                continue
            hold = 0 if final else self._held(self.buf, [CALLS_OPEN])
            d.content += self.buf[: len(self.buf) - hold]
            self.buf = self.buf[len(self.buf) - hold:]
            return d
