"""HTTP API against a fake backend (no GPU): protocol errors, streaming, reasoning split, tools, schema validation,
admission 429, worker failures."""
import http.client
import json
import threading
import time

import pytest

from ds41rt_b200.serving import chat as C
from ds41rt_b200.serving.engine import FakeBackend
from ds41rt_b200.serving.http import ApiServer
from ds41rt_b200.serving.protocol import MODEL_ID, StopStrings
from ds41rt_b200.serving.tokenizer import ByteTokenizer, StreamingDecoder

TK = ByteTokenizer()


def serve(text=None, **kw):
    script = TK.encode(text) if text is not None else []
    backend = FakeBackend(script=script, tokenizer=TK, **{k: v for k, v in kw.items() if k in
                                                          ("delay", "fail_after", "drop_finish", "chunk")})
    srv = ApiServer(backend, TK, queue_depth=kw.get("queue_depth", 4), waiters=kw.get("waiters", 0),
                    first_event_timeout=kw.get("timeout", 5.0)).start()
    return srv, backend


def call(srv, body=None, path="/v1/chat/completions", method="POST"):
    c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=10)
    data = json.dumps(body).encode() if body is not None else None
    c.request(method, path, body=data, headers={"Content-Type": "application/json"} if data else {})
    r = c.getresponse()
    raw = r.read().decode()
    c.close()
    return r.status, dict(r.getheaders()), raw


def req(**kw):
    b = {"model": MODEL_ID, "messages": [{"role": "user", "content": "hi"}]}
    b.update(kw)
    return b


def sse(raw):
    return [l[6:] for l in raw.split("\n") if l.startswith("data: ")]


def test_health_models_stats_and_console():
    srv, be = serve("x")
    try:
        assert call(srv, path="/health", method="GET")[0] == 200
        st, _, raw = call(srv, path="/v1/models", method="GET")
        m = json.loads(raw)["data"][0]
        assert m["id"] == MODEL_ID and m["max_context_tokens"] == 1048576 and m["max_output_tokens"] == 393216
        assert "admission" in json.loads(call(srv, path="/v1/stats", method="GET")[2])
        assert call(srv, path="/v1/console/snapshot", method="GET")[0] == 200
        assert "console" in call(srv, path="/", method="GET")[2]
        be.healthy = False
        assert call(srv, path="/health", method="GET")[0] == 503
        assert call(srv, req())[0] == 503
    finally:
        srv.stop()


@pytest.mark.parametrize("patch,needle", [
    ({"model": "other"}, "model must be"), ({"messages": []}, "non-empty"), ({"temperature": "hot"}, "temperature"),
    ({"top_p": 0}, "top_p"), ({"top_k": 1.5}, "top_k"), ({"response_format": {"type": "xml"}}, "response_format"),
    ({"tool_choice": "required"}, "tools"), ({"thinking": {"type": "maybe"}}, "thinking"),
    ({"response_format": {"type": "json_schema", "json_schema": {"schema": {"type": "frob"}}}}, "unsupported"),
    ({"messages": [{"role": "wizard", "content": "x"}]}, "role"), ({"stop": [1]}, "stop"),
    ({"tool_decoding_assistance": "no"}, "tool_decoding_assistance"),
])
def test_bad_requests_are_400_with_error_shape(patch, needle):
    srv, _ = serve("x")
    try:
        st, _, raw = call(srv, req(**patch))
        err = json.loads(raw)["error"]
        assert st == 400 and err["type"] == "native_v41_error" and needle in err["message"]
    finally:
        srv.stop()


def test_completion_splits_reasoning_and_reports_usage():
    srv, be = serve("thinking hard</think>The answer is 4.")
    try:
        st, _, raw = call(srv, req())
        doc = json.loads(raw)
        msg = doc["choices"][0]["message"]
        assert st == 200 and msg["content"] == "The answer is 4." and msg["reasoning_content"] == "thinking hard"
        assert doc["choices"][0]["finish_reason"] == "stop" and doc["usage"]["completion_tokens"] > 0
        assert doc["usage"]["total_tokens"] == doc["usage"]["prompt_tokens"] + doc["usage"]["completion_tokens"]
        prompt = TK.decode(be.submitted[0].prompt_ids)
        assert prompt.endswith(C.ASSISTANT + C.THINK_OPEN) and C.USER + "hi" in prompt
        # thinking disabled: the prompt closes the thinking block itself
        call(srv, req(thinking={"type": "disabled"}))
        assert TK.decode(be.submitted[1].prompt_ids).endswith(C.ASSISTANT + C.THINK_CLOSE)
        assert be.submitted[0].sampling.greedy
    finally:
        srv.stop()


def test_streaming_sse_chunks_usage_and_utf8():
    srv, _ = serve("r</think>héllo wörld ✓", chunk=1)       # one byte per token: UTF-8 split across tokens
    try:
        st, hdr, raw = call(srv, req(stream=True, stream_options={"include_usage": True}))
        events = sse(raw)
        assert st == 200 and hdr["Content-Type"] == "text/event-stream" and events[-1] == "[DONE]"
        docs = [json.loads(e) for e in events[:-1]]
        text = "".join(d["choices"][0]["delta"].get("content", "") for d in docs if d["choices"])
        assert text == "héllo wörld ✓" and "�" not in text
        assert any(d["choices"] and d["choices"][0]["finish_reason"] == "stop" for d in docs)
        assert docs[-1]["choices"] == [] and docs[-1]["usage"]["completion_tokens"] > 0
    finally:
        srv.stop()


def test_length_finish_and_stop_strings():
    srv, _ = serve("</think>one two three four")
    try:
        doc = json.loads(call(srv, req(max_tokens=12))[2])
        assert doc["choices"][0]["finish_reason"] == "length"
        doc = json.loads(call(srv, req(stop=["three"]))[2])
        assert doc["choices"][0]["message"]["content"] == "one two " and doc["choices"][0]["finish_reason"] == "stop"
    finally:
        srv.stop()
    s = StopStrings(["END"])
    assert s.push("abcE") == "abc" and s.push("Nx") == "ENx" and s.push("..EN") == ".." and s.push("D!") == "" and s.hit


def test_tool_calls_are_parsed_validated_and_streamed():
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}},
        "required": ["city"]}}}]
    block = C.render_tool_call("get_weather", {"city": "Paris", "days": 3})
    srv, be = serve("</think>Let me check.\n" + block)
    try:
        doc = json.loads(call(srv, req(tools=tools))[2])
        ch = doc["choices"][0]
        args = json.loads(ch["message"]["tool_calls"][0]["function"]["arguments"])
        assert ch["finish_reason"] == "tool_calls" and args == {"city": "Paris", "days": 3}
        assert ch["message"]["content"] == "Let me check.\n"
        assert "get_weather" in TK.decode(be.submitted[0].prompt_ids)
        events = sse(call(srv, req(tools=tools, stream=True))[2])
        assert any("tool_calls" in e for e in events) and events[-1] == "[DONE]"
    finally:
        srv.stop()
    bad = C.render_tool_call("get_weather", {"city": "Paris", "days": "three"})
    srv, _ = serve("</think>" + bad)
    try:
        st, _, raw = call(srv, req(tools=tools))
        assert st == 500 and "schema" in json.loads(raw)["error"]["message"]
        st, _, raw = call(srv, req(tools=tools, tool_choice="none"))
        assert st == 200
    finally:
        srv.stop()
    srv, _ = serve("</think>no call here")
    try:
        st, _, raw = call(srv, req(tools=tools, tool_choice="required"))
        assert st == 500                                      # the grammar rejects it / validation catches it
    finally:
        srv.stop()
    # decoding assistance: automatic selection carries the triggered grammar unless the client switches it off; a tool
    # declared strict keeps it; the completed block is validated either way
    srv, be = serve("</think>Let me check.\n" + block)
    try:
        assert call(srv, req(tools=tools))[0] == 200 and be.submitted[-1].constraint is not None
        st, _, raw = call(srv, req(tools=tools, tool_decoding_assistance=False))
        assert st == 200 and be.submitted[-1].constraint is None
        assert json.loads(raw)["choices"][0]["finish_reason"] == "tool_calls"
        strict = [dict(tools[0], function=dict(tools[0]["function"], strict=True))]
        assert call(srv, req(tools=strict, tool_decoding_assistance=False))[0] == 200
        assert be.submitted[-1].constraint is not None
        assert call(srv, req(tools=tools, tool_choice="required", tool_decoding_assistance=False))[0] == 200
        assert be.submitted[-1].constraint is not None
    finally:
        srv.stop()


def test_json_schema_outputs_are_revalidated():
    schema = {"type": "object", "properties": {"n": {"type": "integer"}}, "required": ["n"]}
    rf = {"type": "json_schema", "json_schema": {"name": "x", "strict": True, "schema": schema}}
    srv, be = serve('</think>{"n": 7}')
    try:
        doc = json.loads(call(srv, req(response_format=rf))[2])
        assert json.loads(doc["choices"][0]["message"]["content"]) == {"n": 7}
        assert be.submitted[0].constraint is not None
    finally:
        srv.stop()
    srv, _ = serve('</think>{"n": "seven"}')
    try:
        assert call(srv, req(response_format=rf))[0] == 500
    finally:
        srv.stop()
    # the same property twice - also through an escaped alias - is an error, not "last value wins"
    for text in ('{"n": 1, "n": 2}', '{"n": 1, "\\u006e": 2}'):
        srv, _ = serve("</think>" + text)
        try:
            st, _, raw = call(srv, req(response_format={"type": "json_object"}))
            assert st == 500 and "duplicate" in json.loads(raw)["error"]["message"], text
        finally:
            srv.stop()
    assert C.loads_strict('{"a": {"b": 1}, "c": [{"b": 2}, {"b": 3}]}') == {"a": {"b": 1}, "c": [{"b": 2}, {"b": 3}]}
    twice = C.CALLS_OPEN + "\n" + f'{C.DSML_OPEN} invoke name="f">\n' + \
        f'{C.DSML_OPEN} parameter name="x" string="true">1{C.DSML_CLOSE} parameter>\n' * 2 + \
        f"{C.DSML_CLOSE} invoke>\n" + C.CALLS_CLOSE
    with pytest.raises(C.ChatError, match="twice"):
        C.parse_tool_calls(twice)
    nested = twice.replace('string="true">1', 'string="false">{"k": 1, "k": 2}', 1).replace(
        f'{C.DSML_OPEN} parameter name="x" string="true">1{C.DSML_CLOSE} parameter>\n', "", 1)
    with pytest.raises(C.ChatError, match="duplicate"):
        C.parse_tool_calls(nested)


def test_bounded_admission_answers_429_with_retry_after():
    srv, _ = serve("</think>" + "x" * 30, delay=0.2, queue_depth=1, waiters=0)
    try:
        results = []
        t = threading.Thread(target=lambda: results.append(call(srv, req())))
        t.start()
        time.sleep(0.15)
        st, hdr, raw = call(srv, req())
        assert st == 429 and hdr.get("Retry-After") == "1"
        t.join()
        assert results[0][0] == 200
        assert json.loads(call(srv, path="/v1/stats", method="GET")[2])["http"]["rejected_429"] == 1
    finally:
        srv.stop()


def test_backend_failure_and_missing_finish_are_errors():
    srv, _ = serve("</think>" + "y" * 40, fail_after=6)
    try:
        st, _, raw = call(srv, req())
        assert st == 500 and "scripted" in json.loads(raw)["error"]["message"]
        events = sse(call(srv, req(stream=True))[2])
        assert "error" in events[-1] and "[DONE]" not in events
    finally:
        srv.stop()
    srv, _ = serve("</think>abc", drop_finish=True, timeout=0.5)
    try:
        st, _, raw = call(srv, req())
        assert st == 500 and "finish" in json.loads(raw)["error"]["message"]
    finally:
        srv.stop()


def test_streaming_decoder_holds_incomplete_utf8():
    d = StreamingDecoder(TK)
    ids = TK.encode("a✓b")
    out = [d.push([t]) for t in ids]
    assert "".join(out) == "a✓b" and out[1] == "" and out[2] == ""


def test_console_websocket_feed_pushes_snapshots():
    """GET /v1/console with an upgrade request: RFC 6455 handshake, JSON text frames, ping answered, close echoed."""
    import base64
    import hashlib
    import os
    import socket
    from ds41rt_b200.serving.http import WS_GUID, ws_read_frame
    srv, be = serve("x")
    try:
        s = socket.create_connection(("127.0.0.1", srv.port), timeout=10)
        key = base64.b64encode(os.urandom(16)).decode()
        s.sendall((f"GET /v1/console HTTP/1.1\r\nHost: x\r\nUpgrade: websocket\r\nConnection: Upgrade\r\n"
                   f"Sec-WebSocket-Key: {key}\r\nSec-WebSocket-Version: 13\r\n\r\n").encode())
        head = b""
        while b"\r\n\r\n" not in head:
            head += s.recv(1)
        want = base64.b64encode(hashlib.sha1((key + WS_GUID).encode()).digest()).decode()
        assert head.startswith(b"HTTP/1.1 101") and f"Sec-WebSocket-Accept: {want}".encode() in head
        op, data = ws_read_frame(s)                              # server frames are unmasked: same parser
        assert op == 1 and "admission" in json.loads(data)

        def send(opcode, payload):
            mask = os.urandom(4)
            s.sendall(bytes([0x80 | opcode, 0x80 | len(payload)]) + mask +
                      bytes(b ^ mask[i & 3] for i, b in enumerate(payload)))
        send(0x9, b"hello")
        seen = []
        while 0xA not in [o for o, _ in seen]:
            seen.append(ws_read_frame(s))
        assert (0xA, b"hello") in seen
        op, data = ws_read_frame(s)                              # the next periodic snapshot
        assert op == 1 and json.loads(data)["http"]["requests"] >= 0
        send(0x8, (1000).to_bytes(2, "big"))
        while True:
            f = ws_read_frame(s)
            if f is None or f[0] == 0x8:
                break
        assert f is not None and f[0] == 0x8
        s.close()
        # a client that does not ask for the upgrade still gets the event stream
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=10)
        c.request("GET", "/v1/console")
        r = c.getresponse()
        assert r.status == 200 and r.getheader("Content-Type") == "text/event-stream"
        assert r.fp.readline().startswith(b"data: ")
        c.close()
    finally:
        srv.stop()


def test_campaign_tool_drives_mixed_traffic_through_the_server():
    """The concurrency campaign tool against the fake backend: every request kind completes, follow-up turns extend an
    earlier conversation, schema answers are checked, tokens and first-token times are reported."""
    from ds41rt_b200.utils.http_campaign import run_campaign
    srv, be = serve('{"city": "Paris", "days": 3, "metric": true}', queue_depth=16, waiters=16)
    try:
        out = run_campaign("127.0.0.1", srv.port, clients=4, requests=12, max_tokens=64)
    finally:
        srv.stop()
    assert out["completed"] == 12 and out["failed"] == 0 and out["rejected_429"] == 0
    assert sum(out["by_kind"].values()) == 12 and out["by_kind"]["sampled"] >= 2 and out["by_kind"]["followup"] >= 1
    assert out["schema_answers_valid_or_valid_prefix"] == "3/3"
    assert out["completion_tokens"] > 0 and out["tok_per_s"] > 0 and out["ttft_s"]["median"] is not None
    follow = [g for g in be.submitted if "Now shorter" in TK.decode(g.prompt_ids) and "Request" in TK.decode(g.prompt_ids)]
    assert follow, "a follow-up turn carries the earlier exchange in its prompt"


def test_api_smoke_battery_passes_on_a_conforming_server_and_names_what_fails():
    """The operator's protocol battery over scripted servers: every check passes where the server's answer fits it, a
    check whose promise the answer breaks is reported by name and fails the run."""
    from ds41rt_b200.utils import api_smoke as S
    general = ["health", "stats", "chat", "stream", "length", "stop", "seed", "bad_request", "prefix"]
    srv, _ = serve("one two three four five six seven", queue_depth=8, waiters=4)
    try:
        url = f"http://127.0.0.1:{srv.port}"
        out = S.run(url, max_tokens=48, only=general)
        assert out["ok"] and out["passed"] == len(general) + 1, out          # + models, which always runs
        notes = {r["check"]: r["note"] for r in out["checks"]}
        assert "cut at 16 of 33" in notes["stop"] and notes["length"] == "1 token" and "5 malformed" in notes["bad_request"]
        # the whole battery against this server: the plain text breaks the JSON and tool promises, and only those
        out = S.run(url, max_tokens=48)
        assert not out["ok"] and out["failed"] == ["json_object", "json_schema", "tools"]
        assert S.main(["--url", url, "--only", "chat,stream", "--json"]) == 0
        assert S.main(["--url", url, "--only", "tools"]) == 1
    finally:
        srv.stop()
    srv, _ = serve('{"city": "Paris", "days": 3, "metric": true}', queue_depth=8, waiters=4)
    try:
        out = S.run(f"http://127.0.0.1:{srv.port}", only=["json_object", "json_schema"])
        assert out["ok"] and out["passed"] == 3
    finally:
        srv.stop()
    srv, _ = serve('{"city": "Paris", "days": "three"}', queue_depth=8, waiters=4)      # wrong type: the server refuses
    try:
        out = S.run(f"http://127.0.0.1:{srv.port}", only=["json_schema"])
        assert out["failed"] == ["json_schema"] and "status 500" in out["checks"][-1]["note"]
    finally:
        srv.stop()
    srv, _ = serve("Let me check.\n" + C.render_tool_call("get_weather", {"city": "Paris", "days": 3}),
                   queue_depth=8, waiters=4)
    try:
        out = S.run(f"http://127.0.0.1:{srv.port}", only=["tools"], max_tokens=400)
        assert out["ok"] and '"city": "Paris"' in out["checks"][-1]["note"]
    finally:
        srv.stop()
    assert S.run("http://127.0.0.1:9", only=["health"], timeout=2.0)["failed"] == ["health", "models"]   # nobody listens
