"""Protocol battery against a running server: one pass over everything a client relies on, with a verdict per check.

    python -m ds41rt_b200.utils.api_smoke --url http://127.0.0.1:8000 [--max-tokens 48] [--only chat,stream] [--json]

Checks (each prints one line; exit status 1 when a required check fails):

    health       GET /health answers 200
    models       GET /v1/models lists a model with its context and output limits
    stats        GET /v1/stats is a JSON document with the admission and totals sections
    chat         a greedy completion: choices[0].message, a finish reason, usage that adds up
    stream       the same request as server-sent events: content deltas, a finish reason, a usage chunk, [DONE];
                 the concatenated text equals the non-streamed answer (greedy decoding is deterministic)
    length       max_tokens = 1 ends with finish_reason "length" and one completion token
    stop         a stop string taken from the greedy answer cuts the answer before it and finishes with "stop"
    seed         two sampled requests with one seed give one text
    json_object  response_format json_object: the answer parses as a JSON object (or was cut by the token limit)
    json_schema  response_format json_schema: the answer parses and carries the required properties with their types
    tools        a forced tool call: finish_reason "tool_calls", the named function, arguments that parse and validate
    bad_request  malformed bodies are 400 with an {"error": {"message", "type"}} document, never a 500
    prefix       the same long prompt twice: the second answer is the same; cache hit tokens are reported when the
                 server exposes them (informational: a server without prompt snapshots still passes)

Generation checks accept a `length` finish where the model simply talked longer than --max-tokens; what they insist on is
protocol shape and the constraints the server promises to enforce.  Everything goes over plain HTTP from this process;
no GPU, no package internals.  Counterpart of the reference's API smokes and native API qualifier
(scripts/api-smoke.sh, scripts/api-constrained-smoke.sh, scripts/api-prefill-smoke.sh,
scripts/qualify-ds41-native-api.py).
"""
from __future__ import annotations

import argparse
import http.client
import json
import sys
import time
from typing import Callable, Dict, List, Optional, Tuple
from urllib.parse import urlparse

WEATHER = {"type": "function", "function": {"name": "get_weather", "description": "Weather for a city", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}, "required": ["city"]}}}
TRIP = {"type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"},
                                         "metric": {"type": "boolean"}}, "required": ["city", "days"]}
TYPES = {"string": str, "integer": int, "boolean": bool, "number": (int, float), "object": dict, "array": list}


class Failed(Exception):
    pass


def need(cond, why: str):
    if not cond:
        raise Failed(why)


class Client:
    def __init__(self, url: str, timeout: float = 600.0):
        u = urlparse(url if "//" in url else "http://" + url)
        self.host, self.port, self.timeout = u.hostname or "127.0.0.1", u.port or 80, timeout
        self.model = None

    def call(self, method: str, path: str, body=None) -> Tuple[int, Dict[str, str], str]:
        c = http.client.HTTPConnection(self.host, self.port, timeout=self.timeout)
        data = body if isinstance(body, (bytes, type(None))) else json.dumps(body).encode()
        c.request(method, path, body=data, headers={"Content-Type": "application/json"} if data is not None else {})
        r = c.getresponse()
        raw = r.read().decode("utf-8", "replace")
        c.close()
        return r.status, dict(r.getheaders()), raw

    def body(self, content="Name three colours.", **kw) -> dict:
        b = {"messages": [{"role": "user", "content": content}], "temperature": 0, "thinking": {"type": "disabled"}}
        if self.model:
            b["model"] = self.model
        b.update(kw)
        return b

    def chat(self, **kw) -> dict:
        st, _, raw = self.call("POST", "/v1/chat/completions", self.body(**kw))
        need(st == 200, f"status {st}: {raw[:160]}")
        doc = json.loads(raw)
        need(doc.get("choices") and "message" in doc["choices"][0], "no choices[0].message")
        return doc

    def stream(self, **kw) -> Tuple[str, Optional[str], Optional[dict], List[dict]]:
        """-> (text, finish reason, usage, chunks)"""
        st, hdr, raw = self.call("POST", "/v1/chat/completions",
                                 self.body(stream=True, stream_options={"include_usage": True}, **kw))
        need(st == 200, f"status {st}: {raw[:160]}")
        need(hdr.get("Content-Type", "").startswith("text/event-stream"), f"content type {hdr.get('Content-Type')}")
        events = [l[6:] for l in raw.split("\n") if l.startswith("data: ")]
        need(events and events[-1].strip() == "[DONE]", "stream does not end with [DONE]")
        chunks = [json.loads(e) for e in events[:-1]]
        need(not any("error" in c for c in chunks), "error event in the stream")
        text, finish, usage = [], None, None
        for c in chunks:
            usage = c.get("usage") or usage
            for ch in c.get("choices") or []:
                text.append((ch.get("delta") or {}).get("content") or "")
                finish = ch.get("finish_reason") or finish
        return "".join(text), finish, usage, chunks


def _text(doc: dict) -> str:
    return doc["choices"][0]["message"].get("content") or ""


def _finish(doc: dict) -> str:
    return doc["choices"][0].get("finish_reason")


def _check_schema(value, schema, where="answer"):
    need(isinstance(value, dict), f"{where} is not an object")
    for k in schema.get("required", []):
        need(k in value, f"{where} lacks required property {k!r}")
    for k, v in value.items():
        want = schema.get("properties", {}).get(k, {}).get("type")
        if want in TYPES:
            ok = isinstance(v, TYPES[want]) and not (want in ("integer", "number") and isinstance(v, bool))
            need(ok, f"{where}.{k} is not {want}")


# ---------------------------------------------------------------------------------------------- the checks
def check_health(c: Client, a) -> str:
    st, _, raw = c.call("GET", "/health")
    need(st == 200, f"status {st}")
    return raw.strip()[:60]


def check_models(c: Client, a) -> str:
    st, _, raw = c.call("GET", "/v1/models")
    need(st == 200, f"status {st}")
    data = json.loads(raw).get("data") or []
    need(data and data[0].get("id"), "no model listed")
    c.model = data[0]["id"]
    m = data[0]
    need(int(m.get("max_context_tokens", 0)) > 0, "model entry has no max_context_tokens")
    return f"{m['id']} context {m['max_context_tokens']} output {m.get('max_output_tokens')}"


def check_stats(c: Client, a) -> str:
    st, _, raw = c.call("GET", "/v1/stats")
    need(st == 200, f"status {st}")
    doc = json.loads(raw)
    need("admission" in doc, "no admission section")
    return ", ".join(sorted(doc))[:100]


def check_chat(c: Client, a) -> str:
    doc = c.chat(max_tokens=a.max_tokens)
    u = doc.get("usage") or {}
    need(_finish(doc) in ("stop", "length"), f"finish_reason {_finish(doc)!r}")
    need(u.get("prompt_tokens", 0) > 0 and u.get("completion_tokens", 0) > 0, "usage without token counts")
    need(u.get("total_tokens") == u["prompt_tokens"] + u["completion_tokens"], "usage does not add up")
    need(u["completion_tokens"] <= a.max_tokens, "more completion tokens than max_tokens")
    need(doc.get("object") == "chat.completion" and doc.get("id"), "object / id missing")
    a.greedy_text = _text(doc)
    return f"{u['completion_tokens']} tokens, finish {_finish(doc)}"


def check_stream(c: Client, a) -> str:
    text, finish, usage, chunks = c.stream(max_tokens=a.max_tokens)
    need(finish in ("stop", "length"), f"finish_reason {finish!r}")
    need(usage and usage.get("completion_tokens", 0) > 0, "no usage chunk")
    need(all(ch.get("object") == "chat.completion.chunk" for ch in chunks), "chunk object type")
    if getattr(a, "greedy_text", None) is not None:
        need(text == a.greedy_text, "streamed text differs from the non-streamed greedy answer")
    return f"{len(chunks)} chunks, {usage['completion_tokens']} tokens"


def check_length(c: Client, a) -> str:
    doc = c.chat(max_tokens=1)
    need(_finish(doc) == "length", f"finish_reason {_finish(doc)!r}")
    need(doc["usage"]["completion_tokens"] == 1, f"{doc['usage']['completion_tokens']} completion tokens")
    return "1 token"


def check_stop(c: Client, a) -> str:
    base = getattr(a, "greedy_text", None) or _text(c.chat(max_tokens=a.max_tokens))
    body = base.strip()
    if len(body) < 8:
        return "skipped: the greedy answer is too short to cut"
    mid = len(body) // 2
    stop = body[mid: mid + 4]
    doc = c.chat(max_tokens=a.max_tokens, stop=[stop])
    got = _text(doc)
    need(stop not in got, "the stop string is part of the answer")
    need(_finish(doc) == "stop", f"finish_reason {_finish(doc)!r}")
    need(base.startswith(got), "the cut answer is not a prefix of the uncut one")
    return f"cut at {len(got)} of {len(base)} characters"


def check_seed(c: Client, a) -> str:
    kw = dict(max_tokens=min(a.max_tokens, 24), temperature=0.9, top_p=0.95, seed=1234)
    one, two = _text(c.chat(**kw)), _text(c.chat(**kw))
    need(one == two, "one seed, two texts")
    return f"{len(one)} characters twice"


def check_json_object(c: Client, a) -> str:
    doc = c.chat(content="Reply with a JSON object describing a cat.", max_tokens=a.max_tokens,
                 response_format={"type": "json_object"})
    if _finish(doc) == "length":
        return "cut by the token limit (shape not checked)"
    need(isinstance(json.loads(_text(doc)), dict), "not a JSON object")
    return "object"


def check_json_schema(c: Client, a) -> str:
    doc = c.chat(content="Plan a trip: city, days, metric.", max_tokens=a.max_tokens,
                 response_format={"type": "json_schema", "json_schema": {"name": "trip", "strict": True, "schema": TRIP}})
    if _finish(doc) == "length":
        return "cut by the token limit (shape not checked)"
    _check_schema(json.loads(_text(doc)), TRIP)
    return _text(doc)[:60]


def check_tools(c: Client, a) -> str:
    doc = c.chat(content="What is the weather in Paris for three days?", max_tokens=max(a.max_tokens, 64),
                 tools=[WEATHER], tool_choice={"type": "function", "function": {"name": "get_weather"}})
    if _finish(doc) == "length":
        return "cut by the token limit (shape not checked)"
    need(_finish(doc) == "tool_calls", f"finish_reason {_finish(doc)!r}")
    calls = doc["choices"][0]["message"].get("tool_calls") or []
    need(calls and calls[0].get("type") == "function" and calls[0].get("id"), "no tool call")
    fn = calls[0]["function"]
    need(fn.get("name") == "get_weather", f"function {fn.get('name')!r}")
    _check_schema(json.loads(fn["arguments"]), WEATHER["function"]["parameters"], "arguments")
    return fn["arguments"][:60]


def check_bad_request(c: Client, a) -> str:
    cases = [("not json", b"{nope"), ("no messages", {"model": c.model}), ("bad temperature", c.body(temperature="hot")),
             ("negative max_tokens", c.body(max_tokens=-3)), ("unknown role", {"messages": [{"role": "wizard", "content": "x"}]})]
    for name, body in cases:
        st, _, raw = c.call("POST", "/v1/chat/completions", body)
        need(st == 400, f"{name}: status {st}")
        err = json.loads(raw).get("error") or {}
        need(err.get("message") and err.get("type"), f"{name}: error document lacks message / type")
    st, _, _ = c.call("GET", "/v1/no-such-route")
    need(st == 404, f"unknown route: status {st}")
    return f"{len(cases)} malformed bodies refused"


def check_prefix(c: Client, a) -> str:
    prompt = "Summarise: " + " ".join(f"item {i} is {i * i}." for i in range(a.prefix_items))
    one = c.chat(content=prompt, max_tokens=min(a.max_tokens, 16))
    t0 = time.perf_counter()
    two = c.chat(content=prompt, max_tokens=min(a.max_tokens, 16))
    dt = time.perf_counter() - t0
    need(_text(one) == _text(two), "one prompt, two greedy answers")
    u = two.get("usage") or {}
    hit = (u.get("prompt_tokens_details") or {}).get("cached_tokens", u.get("prompt_cache_hit_tokens"))
    return f"second answer in {dt:.2f} s, cache hit tokens: {hit if hit is not None else 'not reported'}"


CHECKS: List[Tuple[str, Callable]] = [
    ("health", check_health), ("models", check_models), ("stats", check_stats), ("chat", check_chat),
    ("stream", check_stream), ("length", check_length), ("stop", check_stop), ("seed", check_seed),
    ("json_object", check_json_object), ("json_schema", check_json_schema), ("tools", check_tools),
    ("bad_request", check_bad_request), ("prefix", check_prefix)]


def run(url: str, max_tokens: int = 48, only: Optional[List[str]] = None, prefix_items: int = 60, timeout: float = 600.0,
        emit=None) -> dict:
    c = Client(url, timeout)
    a = argparse.Namespace(max_tokens=max_tokens, prefix_items=prefix_items, greedy_text=None)
    results = []
    for name, fn in CHECKS:
        if only and name not in only and name != "models":
            continue
        t0 = time.perf_counter()
        try:
            note, ok = fn(c, a), True
        except Failed as e:
            note, ok = str(e), False
        except (OSError, ValueError, KeyError, IndexError, TypeError) as e:
            note, ok = f"{type(e).__name__}: {e}", False
        row = {"check": name, "ok": ok, "seconds": round(time.perf_counter() - t0, 3), "note": note}
        results.append(row)
        if emit:
            emit(row)
    return {"url": url, "ok": all(r["ok"] for r in results), "passed": sum(r["ok"] for r in results),
            "failed": [r["check"] for r in results if not r["ok"]], "checks": results}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--max-tokens", type=int, default=48)
    ap.add_argument("--only", default="", help="comma-separated check names (models always runs: it learns the model id)")
    ap.add_argument("--prefix-items", type=int, default=60, help="length of the repeated prompt of the prefix check")
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--json", action="store_true", help="print one JSON document instead of a line per check")
    args = ap.parse_args(argv)
    only = [x for x in args.only.split(",") if x] or None
    show = None if args.json else (lambda r: print(f"{'ok  ' if r['ok'] else 'FAIL'} {r['check']:<12} {r['seconds']:>7.2f} s  "
                                                   f"{r['note']}", flush=True))
    out = run(args.url, args.max_tokens, only, args.prefix_items, args.timeout, show)
    if args.json:
        print(json.dumps(out))
    else:
        print(f"{out['passed']} of {len(out['checks'])} checks passed" + (f"; failed: {', '.join(out['failed'])}"
                                                                           if out["failed"] else ""))
    return 0 if out["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
