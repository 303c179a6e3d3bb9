"""OpenAI-compatible request parsing and limits for POST /v1/chat/completions.

Field handling follows the reference router (rust/crates/ds41rt-api/src/native_v41.rs:162-437, limits.rs:4-58):
temperature defaults to 0 (greedy); top_k 0 or -1 disables top-k; seed is a signed 64-bit integer; the model name
must match the served model; `response_format` is text | json_object | json_schema{strict} | regex; `thinking.type`
enabled/disabled (default enabled, effort "high"); `tool_choice` auto | none | required | {function:{name}}; `tool_decoding_assistance` (false: automatic selection over
non-strict tools decodes without the tool grammar).
Errors are {"error": {"message", "type": "native_v41_error"}} with a bounded message.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

MODEL_ID = "deepseek-ai/DeepSeek-V4.1-Flash"
MAX_CONTEXT = 1048576
MAX_OUTPUT = 393216
MAX_IMAGES = 16
ERROR_TYPE = "native_v41_error"


class ApiError(Exception):
    def __init__(self, status: int, message: str, retry_after: Optional[int] = None):
        super().__init__(message)
        self.status, self.message, self.retry_after = status, message[:512], retry_after

    def body(self) -> dict:
        return {"error": {"message": self.message, "type": ERROR_TYPE}}


@dataclass
class Sampling:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-5 or self.top_k == 1


@dataclass
class ChatRequest:
    messages: List[dict]
    stream: bool = False
    include_usage: bool = False
    max_tokens: Optional[int] = None
    sampling: Sampling = field(default_factory=Sampling)
    tools: List[dict] = field(default_factory=list)
    tool_choice: Any = "auto"
    parallel_tool_calls: bool = True
    tool_decoding_assistance: bool = True        # false: automatic selection over non-strict tools decodes unconstrained
    response_format: Dict[str, Any] = field(default_factory=lambda: {"type": "text"})
    thinking: bool = True
    reasoning_effort: Optional[str] = "high"
    stop: List[str] = field(default_factory=list)


def _num(body, key, default, lo=None, hi=None, integer=False):
    v = body.get(key, default)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (integer and not float(v).is_integer()):
        raise ApiError(400, f"'{key}' must be {'an integer' if integer else 'a number'}")
    if (lo is not None and v < lo) or (hi is not None and v > hi):
        raise ApiError(400, f"'{key}' is out of range")
    return int(v) if integer else float(v)


def parse_chat_request(body: Any, model_id: str = MODEL_ID, max_output: int = MAX_OUTPUT) -> ChatRequest:
    if not isinstance(body, dict):
        raise ApiError(400, "request body must be a JSON object")
    if body.get("model") != model_id:
        raise ApiError(400, f"model must be '{model_id}'")
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise ApiError(400, "'messages' must be a non-empty array")
    n_images = sum(1 for m in msgs if isinstance(m, dict) and isinstance(m.get("content"), list)
                   for p in m["content"] if isinstance(p, dict) and p.get("type") == "image_url")
    if n_images > MAX_IMAGES:
        raise ApiError(400, f"at most {MAX_IMAGES} images per request")
    req = ChatRequest(messages=msgs)
    req.stream = bool(body.get("stream", False))
    so = body.get("stream_options") or {}
    if not isinstance(so, dict):
        raise ApiError(400, "'stream_options' must be an object")
    req.include_usage = bool(so.get("include_usage", False))
    mt = body.get("max_tokens", body.get("max_completion_tokens"))
    if mt is not None:
        mt = _num({"max_tokens": mt}, "max_tokens", None, 1, None, integer=True)
        req.max_tokens = min(mt, max_output)
    s = Sampling()
    s.temperature = _num(body, "temperature", 0.0, 0.0, 2.0)
    s.top_p = _num(body, "top_p", 1.0, 0.0, 1.0)
    if s.top_p <= 0.0:
        raise ApiError(400, "'top_p' must be greater than 0")
    k = _num(body, "top_k", 0, -1, None, integer=True)
    s.top_k = 0 if k in (0, -1) else k
    s.min_p = _num(body, "min_p", 0.0, 0.0, 1.0)
    seed = _num(body, "seed", 0, -(2 ** 63), 2 ** 63 - 1, integer=True)
    s.seed = seed & (2 ** 64 - 1)
    req.sampling = s
    tools = body.get("tools") or []
    if not isinstance(tools, list):
        raise ApiError(400, "'tools' must be an array")
    for t in tools:
        fn = t.get("function") if isinstance(t, dict) else None
        if not isinstance(fn, dict) or not isinstance(fn.get("name"), str) or not fn["name"]:
            raise ApiError(400, "every tool needs function.name")
        if "parameters" in fn and not isinstance(fn["parameters"], dict):
            raise ApiError(400, f"tool '{fn['name']}' parameters must be a JSON schema object")
    req.tools = tools
    tc = body.get("tool_choice", "auto" if tools else "none")
    if isinstance(tc, str):
        if tc not in ("auto", "none", "required"):
            raise ApiError(400, "'tool_choice' must be auto, none, required or a named function")
    elif isinstance(tc, dict):
        name = (tc.get("function") or {}).get("name")
        if name not in [t["function"]["name"] for t in tools]:
            raise ApiError(400, "'tool_choice' names an undeclared function")
    else:
        raise ApiError(400, "'tool_choice' is malformed")
    if tc in ("required",) and not tools:
        raise ApiError(400, "'tool_choice' required needs tools")
    req.tool_choice = tc
    req.parallel_tool_calls = bool(body.get("parallel_tool_calls", True))
    assistance = body.get("tool_decoding_assistance")
    if assistance is not None and not isinstance(assistance, bool):
        raise ApiError(400, "'tool_decoding_assistance' must be boolean")
    req.tool_decoding_assistance = True if assistance is None else assistance
    rf = body.get("response_format") or {"type": "text"}
    if not isinstance(rf, dict) or rf.get("type") not in ("text", "json_object", "json_schema", "regex"):
        raise ApiError(400, "'response_format.type' must be text, json_object, json_schema or regex")
    if rf["type"] == "json_schema":
        js = rf.get("json_schema")
        if not isinstance(js, dict) or not isinstance(js.get("schema"), dict):
            raise ApiError(400, "'response_format.json_schema.schema' must be an object")
        from ..runtime.grammar import Grammar, GrammarError
        try:
            Grammar.json_schema(js["schema"])
        except GrammarError as e:
            raise ApiError(400, f"unsupported response schema: {e}")
    if rf["type"] == "regex":
        from ..runtime.grammar import Grammar, GrammarError
        if not isinstance(rf.get("regex"), str):
            raise ApiError(400, "'response_format.regex' must be a string")
        try:
            Grammar.regex(rf["regex"])
        except GrammarError as e:
            raise ApiError(400, f"unsupported regular expression: {e}")
    req.response_format = rf
    th = body.get("thinking")
    if th is not None:
        if not isinstance(th, dict) or th.get("type") not in ("enabled", "disabled"):
            raise ApiError(400, "'thinking.type' must be enabled or disabled")
        req.thinking = th["type"] == "enabled"
    eff = body.get("reasoning_effort", "high" if req.thinking else None)
    if eff is not None and eff not in ("none", "low", "high", "max"):
        raise ApiError(400, "'reasoning_effort' must be none, low, high or max")
    if eff == "none":
        req.thinking = False
    req.reasoning_effort = eff
    stop = body.get("stop") or []
    if isinstance(stop, str):
        stop = [stop]
    if not isinstance(stop, list) or any(not isinstance(x, str) for x in stop) or len(stop) > 8:
        raise ApiError(400, "'stop' must be a string or up to 8 strings")
    req.stop = [x for x in stop if x]
    return req


class StopStrings:
    """Streaming stop-string detector: text that could be the start of a stop string is held back."""

    def __init__(self, stops: List[str]):
        self.stops, self.buf, self.hit = stops, "", False

    def push(self, text: str, final: bool = False) -> str:
        if self.hit:
            return ""
        self.buf += text
        best = None
        for s in self.stops:
            i = self.buf.find(s)
            if i >= 0 and (best is None or i < best):
                best = i
        if best is not None:
            self.hit = True
            out, self.buf = self.buf[:best], ""
            return out
        hold = 0
        if not final:
            for s in self.stops:
                for n in range(min(len(s) - 1, len(self.buf)), 0, -1):
                    if self.buf.endswith(s[:n]):
                        hold = max(hold, n)
                        break
        out = self.buf[: len(self.buf) - hold]
        self.buf = self.buf[len(self.buf) - hold:]
        return out
