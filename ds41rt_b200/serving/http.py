"""OpenAI-compatible HTTP front end.

Routes (reference: rust/crates/ds41rt-api/src/native_v41.rs:90-126,202-437):
  GET  /health                 200 {"status":"ok"} or 503 when the worker died
  GET  /v1/models              the served model with max_context_tokens / max_output_tokens
  GET  /v1/stats               backend counters, HTTP queue counters
  POST /v1/chat/completions    JSON or SSE ("data: {...}\\n\\n" ... "data: [DONE]")
  GET  /  and /v1/console/snapshot   a small live console page and its JSON feed; /v1/console pushes the same
                                     snapshots once a second over a WebSocket (RFC 6455 text frames; reference:
                                     native_v41.rs:94-106, v41_native_serve/console.rs:71-260), or as server-sent events
                                     to a client that does not ask for the upgrade
Errors: {"error":{"message","type":"native_v41_error"}}; 400 bad request, 429 + Retry-After: 1 when the bounded
admission queue is full, 500, 503.  A stream that ends without a Finish event is reported as an error, never as a
successful completion.
"""
from __future__ import annotations

import json
import queue
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Optional

from ..runtime import core as K
from ..runtime.grammar import Grammar, TokenConstraint, Vocab
from . import chat as C
from .engine import Backend, GenRequest
from .protocol import MAX_CONTEXT, MAX_OUTPUT, MODEL_ID, ApiError, StopStrings, parse_chat_request
from .tokenizer import StreamingDecoder

CONSOLE_HTML = """<!doctype html><meta charset=utf-8><title>ds41rt-b200 console</title>
<style>body{font:14px monospace;background:#111;color:#ddd;margin:2em}pre{background:#1b1b1b;padding:1em}</style>
<h3>ds41rt-b200 live console</h3><pre id=o>connecting...</pre>
<script>const o=document.getElementById('o');const show=d=>{o.textContent=JSON.stringify(JSON.parse(d),null,2)};
let w;try{w=new WebSocket((location.protocol=='https:'?'wss://':'ws://')+location.host+'/v1/console');
w.onmessage=e=>show(e.data);w.onerror=()=>{const s=new EventSource('/v1/console');s.onmessage=e=>show(e.data)}}
catch(e){const s=new EventSource('/v1/console');s.onmessage=e=>show(e.data)}</script>"""

WS_GUID = "258EAFA5-E914-47DA-95CA-C5AB0DC85B11"


def ws_frame(payload: bytes, opcode: int = 1) -> bytes:
    """One unmasked server-to-client frame (FIN set)."""
    n = len(payload)
    head = bytes([0x80 | opcode])
    if n < 126:
        head += bytes([n])
    elif n < 65536:
        head += bytes([126]) + n.to_bytes(2, "big")
    else:
        head += bytes([127]) + n.to_bytes(8, "big")
    return head + payload


def ws_read_frame(sock):
    """One client-to-server frame -> (opcode, payload), or None when the peer closed the connection."""
    def need(k):
        buf = b""
        while len(buf) < k:
            part = sock.recv(k - len(buf))
            if not part:
                return None
            buf += part
        return buf
    h = need(2)
    if h is None:
        return None
    n = h[1] & 0x7F
    if n == 126:
        ext = need(2)
        n = int.from_bytes(ext, "big") if ext else 0
    elif n == 127:
        ext = need(8)
        n = int.from_bytes(ext, "big") if ext else 0
    if n > 1 << 20:
        return None
    mask = need(4) if h[1] & 0x80 else b"\0\0\0\0"
    data = need(n) if n else b""
    if mask is None or data is None:
        return None
    return h[0] & 0x0F, bytes(b ^ mask[i & 3] for i, b in enumerate(data))


class ApiServer:
    def __init__(self, backend: Backend, tokenizer, host: str = "127.0.0.1", port: int = 0, model_id: str = MODEL_ID,
                 max_context: int = MAX_CONTEXT, max_output: int = MAX_OUTPUT, queue_depth: int = 16, waiters: int = 16,
                 default_max_tokens: int = 4096, first_event_timeout: float = 600.0, vision_cfg=None):
        self.backend, self.tk, self.model_id = backend, tokenizer, model_id
        self.max_context, self.max_output, self.default_max_tokens = max_context, max_output, default_max_tokens
        self.first_event_timeout = first_event_timeout
        self.vision_cfg = vision_cfg             # config.VisionConfig when the backend has a vision tower
        self.admission = K.Admission(queue_depth, waiters)
        self.vocab: Optional[Vocab] = None
        self.counters = {"requests": 0, "rejected_429": 0, "bad_request": 0, "errors": 0, "streams": 0}
        self.started = time.time()
        server = self

        class Handler(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def do_GET(self):
                server.handle_get(self)

            def do_POST(self):
                server.handle_post(self)

        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.httpd.daemon_threads = True
        self.port = self.httpd.server_address[1]
        self.thread = threading.Thread(target=self.httpd.serve_forever, name="ds41-http", daemon=True)

    def start(self):
        self.thread.start()
        return self

    def stop(self):
        self.httpd.shutdown()
        self.httpd.server_close()

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _send_json(h, status: int, obj, headers=None):
        data = json.dumps(obj).encode()
        h.send_response(status)
        h.send_header("Content-Type", "application/json")
        h.send_header("Content-Length", str(len(data)))
        for k, v in (headers or {}).items():
            h.send_header(k, v)
        h.end_headers()
        h.wfile.write(data)

    def _fail(self, h, err: ApiError):
        key = "rejected_429" if err.status == 429 else "bad_request" if err.status == 400 else "errors"
        self.counters[key] += 1
        self._send_json(h, err.status, err.body(), {"Retry-After": str(err.retry_after)} if err.retry_after else None)

    def snapshot(self) -> dict:
        return {"uptime_s": round(time.time() - self.started, 1), "healthy": self.backend.healthy,
                "http": dict(self.counters), "admission": self.admission.stats(), "backend": self.backend.stats()}

    def _vocab(self) -> Vocab:
        if self.vocab is None:
            self.vocab = Vocab(self.tk.token_bytes())
        return self.vocab

    # ------------------------------------------------------------------ GET
    def handle_get(self, h):
        path = h.path.split("?")[0]
        if path == "/health":
            ok = self.backend.healthy
            return self._send_json(h, 200 if ok else 503, {"status": "ok" if ok else "worker unavailable"})
        if path == "/v1/models":
            return self._send_json(h, 200, {"object": "list", "data": [{
                "id": self.model_id, "object": "model", "owned_by": "ds41rt-b200",
                "max_context_tokens": self.max_context, "max_output_tokens": self.max_output}]})
        if path == "/v1/stats":
            return self._send_json(h, 200, self.snapshot())
        if path == "/v1/console/snapshot":
            return self._send_json(h, 200, self.snapshot())
        if path == "/v1/console" and "websocket" in (h.headers.get("Upgrade") or "").lower():
            return self._console_socket(h)
        if path == "/v1/console":
            h.send_response(200)
            h.send_header("Content-Type", "text/event-stream")
            h.send_header("Cache-Control", "no-cache")
            h.end_headers()
            try:
                for _ in range(3600):
                    h.wfile.write(b"data: " + json.dumps(self.snapshot()).encode() + b"\n\n")
                    h.wfile.flush()
                    time.sleep(1.0)
            except (BrokenPipeError, ConnectionResetError):
                pass
            return
        if path == "/":
            data = CONSOLE_HTML.encode()
            h.send_response(200)
            h.send_header("Content-Type", "text/html; charset=utf-8")
            h.send_header("Content-Length", str(len(data)))
            h.end_headers()
            h.wfile.write(data)
            return
        self._fail(h, ApiError(404, "no such route"))

    def _console_socket(self, h, period: float = 1.0, max_frames: int = 86400):
        """WebSocket feed of the console: handshake, then one JSON text frame per `period`; pings are answered, a
        close frame (or a vanished peer) ends the feed."""
        import base64
        import hashlib
        import select
        key = h.headers.get("Sec-WebSocket-Key")
        if not key:
            return self._fail(h, ApiError(400, "missing Sec-WebSocket-Key"))
        accept = base64.b64encode(hashlib.sha1((key + WS_GUID).encode()).digest()).decode()
        h.send_response(101, "Switching Protocols")
        h.send_header("Upgrade", "websocket")
        h.send_header("Connection", "Upgrade")
        h.send_header("Sec-WebSocket-Accept", accept)
        h.end_headers()
        h.wfile.flush()
        h.close_connection = True
        sock = h.connection
        try:
            for _ in range(max_frames):
                sock.sendall(ws_frame(json.dumps(self.snapshot()).encode()))
                deadline = time.time() + period
                while True:
                    left = deadline - time.time()
                    if left <= 0:
                        break
                    ready, _, _ = select.select([sock], [], [], left)
                    if not ready:
                        break
                    frame = ws_read_frame(sock)
                    if frame is None:
                        return
                    op, data = frame
                    if op == 0x8:                                  # close: echo and stop
                        sock.sendall(ws_frame(data[:2], 0x8))
                        return
                    if op == 0x9:                                  # ping -> pong
                        sock.sendall(ws_frame(data, 0xA))
        except (BrokenPipeError, ConnectionResetError, OSError):
            pass

    # ------------------------------------------------------------------ POST
    def handle_post(self, h):
        if h.path.split("?")[0] != "/v1/chat/completions":
            return self._fail(h, ApiError(404, "no such route"))
        self.counters["requests"] += 1
        try:
            n = int(h.headers.get("Content-Length", "0"))
            if n <= 0 or n > 64 * 1024 * 1024:
                raise ApiError(400, "request body is missing or too large")
            try:
                body = json.loads(h.rfile.read(n).decode("utf-8"))
            except Exception:
                raise ApiError(400, "request body is not valid JSON")
            req = parse_chat_request(body, self.model_id, self.max_output)
            if not self.backend.healthy:
                raise ApiError(503, "inference worker is unavailable")
            try:
                prompt, images = C.render_conversation(req.messages, req.tools if req.tool_choice != "none" else [],
                                                       req.thinking, req.reasoning_effort)
            except C.ChatError as e:
                raise ApiError(400, str(e))
            ids, image_refs = self._encode_with_images(prompt, images)
            if len(ids) >= self.max_context:
                raise ApiError(400, f"prompt of {len(ids)} tokens exceeds the context window")
            max_tokens = min(req.max_tokens or self.default_max_tokens, self.max_output, self.max_context - len(ids))
            constraint = self._constraint(req)
            slot = self.admission.reserve()
            if slot < 0:
                raise ApiError(429, "server is at capacity, retry shortly", retry_after=1)
            gen = GenRequest(prompt_ids=ids, max_tokens=max_tokens, sampling=req.sampling, constraint=constraint,
                             images=image_refs)
            try:
                try:
                    self.backend.submit(gen)
                except queue.Full:
                    raise ApiError(429, "server is at capacity, retry shortly", retry_after=1)
                except RuntimeError as e:
                    raise ApiError(503, str(e))
                try:
                    first = gen.events.get(timeout=self.first_event_timeout)
                except queue.Empty:
                    gen.cancelled.set()
                    raise ApiError(503, "inference worker did not respond")
                if first.kind == "error":
                    raise ApiError(first.status, first.message)
                usage = dict(first.usage)
                if req.stream:
                    self._stream(h, req, gen, usage)
                else:
                    self._complete(h, req, gen, usage)
            finally:
                self.admission.release()
        except ApiError as e:
            try:
                self._fail(h, e)
            except (BrokenPipeError, ConnectionResetError):
                pass

    def _encode_with_images(self, prompt: str, images):
        """Token ids of the rendered prompt; every "<image>" mark becomes the span of its image (start, one placeholder
        per merged patch row group with a newline after each grid row, end).  Images are decoded and resized here, on
        the HTTP thread; the vision tower runs on the worker."""
        if not images:
            return self.tk.encode(prompt), []
        from . import images as IM
        if self.vision_cfg is None or not getattr(self.backend, "supports_images", False):
            raise ApiError(400, "this model does not accept images")
        special = getattr(self.tk, "special", {})
        try:
            tok, start, end, newline = (special[n] for n in ("<image>", "<image_start>", "<image_end>", "<image_newline>"))
        except KeyError:
            raise ApiError(400, "the tokenizer has no image tokens")
        pieces = prompt.split("<image>")
        if len(pieces) != len(images) + 1:
            raise ApiError(400, "image marks and image parts do not match")
        ids, refs = self.tk.encode(pieces[0]), []
        for url, text in zip(images, pieces[1:]):
            try:
                prepared = IM.prepare_image(IM.decode_data_url(url), self.vision_cfg)
            except IM.ImageError as e:
                raise ApiError(400, str(e))
            span = IM.image_span(prepared, self.vision_cfg, tok, start, end, newline)
            refs.append((prepared, [len(ids) + i for i, t in enumerate(span) if t == tok]))
            ids += span
            ids += self.tk.encode(text)
        return ids, refs

    def _constraint(self, req) -> Optional[TokenConstraint]:
        rf = req.response_format
        grammar = None
        if rf["type"] == "json_object":
            grammar = Grammar.json_object()
        elif rf["type"] == "json_schema":
            grammar = Grammar.json_schema(rf["json_schema"]["schema"])
        elif rf["type"] == "regex":
            grammar = Grammar.regex(rf["regex"])
        elif req.tools and (req.tool_choice == "required" or isinstance(req.tool_choice, dict)):
            grammar = Grammar(tool_call_grammar(req.tools, req.tool_choice, req.parallel_tool_calls))
        elif req.tools and req.tool_choice == "auto":
            # A client may switch the decoding assistance off for automatic selection; tools declared strict keep their
            # grammar (reference: rust/crates/ds41rt-api/src/constrained.rs:40-45).  The calls block is still parsed and
            # validated when the answer completes.
            strict = any(t.get("function", {}).get("strict") for t in req.tools)
            if req.tool_decoding_assistance or strict:
                grammar = Grammar(tool_call_grammar(req.tools, "auto", req.parallel_tool_calls, triggered=True))
        if grammar is None:
            return None
        return TokenConstraint(self._vocab(), grammar, eos=self.tk.eos, think_end=self.tk.think_end,
                               thinking=req.thinking)

    # ------------------------------------------------------------------ response assembly
    def _drain(self, gen: GenRequest):
        """Yield token lists until Finish; raises ApiError on backend errors or a missing Finish."""
        while True:
            try:
                ev = gen.events.get(timeout=self.first_event_timeout)
            except queue.Empty:
                gen.cancelled.set()
                raise ApiError(500, "generation ended without a finish event")
            if ev.kind == "tokens":
                yield ev.tokens, None
            elif ev.kind == "finish":
                yield [], ev
                return
            elif ev.kind == "error":
                raise ApiError(ev.status, ev.message)

    def _finalise(self, req, parser, text_content: str, reason: str):
        """Post-hoc validation of structured outputs; returns (finish_reason, error or None)."""
        finish = "tool_calls" if parser.tool_calls else ("length" if reason == "length" else "stop")
        if reason == "length":
            return finish, None
        rf = req.response_format
        if rf["type"] in ("json_object", "json_schema"):
            err = C.validate_json_output(text_content, rf.get("json_schema", {}).get("schema") if rf["type"] == "json_schema" else None)
            if err:
                return finish, err
        if parser.tool_calls and req.tools and req.tool_choice != "none":
            err = C.validate_tool_calls(parser.tool_calls, req.tools)
            if err:
                return finish, err
        if req.tool_choice == "required" and not parser.tool_calls:
            return finish, "a tool call was required but none was produced"
        return finish, None

    def _complete(self, h, req, gen, usage):
        dec, parser, stops = StreamingDecoder(self.tk), C.StreamParser(req.thinking), StopStrings(req.stop)
        reasoning, content, fin = "", "", None
        for toks, ev in self._drain(gen):
            text = dec.push(toks) if toks else ""
            if ev is not None:
                text += dec.flush()
                fin = ev
            d = parser.push(text, final=ev is not None)
            reasoning += d.reasoning
            content += stops.push(d.content, final=ev is not None)
            if stops.hit and ev is None:
                gen.cancelled.set()
        usage.update(fin.usage)
        reason = "stop" if stops.hit else fin.reason
        finish, err = self._finalise(req, parser, content, reason)
        if err:
            raise ApiError(500, err)
        msg = {"role": "assistant", "content": content}
        if reasoning:
            msg["reasoning_content"] = reasoning
        if parser.tool_calls:
            msg["tool_calls"] = parser.tool_calls
        usage["total_tokens"] = usage.get("prompt_tokens", 0) + usage.get("completion_tokens", 0)
        self._send_json(h, 200, {"id": "chatcmpl-" + uuid.uuid4().hex[:24], "object": "chat.completion",
                                 "created": int(time.time()), "model": self.model_id,
                                 "system_fingerprint": self.backend.fingerprint,
                                 "choices": [{"index": 0, "message": msg, "finish_reason": finish}], "usage": usage})

    def _stream(self, h, req, gen, usage):
        self.counters["streams"] += 1
        cid, created = "chatcmpl-" + uuid.uuid4().hex[:24], int(time.time())
        h.send_response(200)
        h.send_header("Content-Type", "text/event-stream")
        h.send_header("Cache-Control", "no-cache")
        h.send_header("Connection", "close")
        h.end_headers()

        def send(obj):
            h.wfile.write(b"data: " + (obj if isinstance(obj, bytes) else json.dumps(obj).encode()) + b"\n\n")
            h.wfile.flush()

        def chunk(delta, finish=None, extra=None):
            o = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": self.model_id,
                 "system_fingerprint": self.backend.fingerprint,
                 "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
            if extra:
                o.update(extra)
            return o

        dec, parser, stops = StreamingDecoder(self.tk), C.StreamParser(req.thinking), StopStrings(req.stop)
        content_all = ""
        try:
            send(chunk({"role": "assistant"}))
            fin = None
            try:
                for toks, ev in self._drain(gen):
                    text = dec.push(toks) if toks else ""
                    if ev is not None:
                        text += dec.flush()
                        fin = ev
                    d = parser.push(text, final=ev is not None)
                    if d.reasoning:
                        send(chunk({"reasoning_content": d.reasoning}))
                    out = stops.push(d.content, final=ev is not None)
                    if out:
                        content_all += out
                        send(chunk({"content": out}))
                    for i, call in enumerate(d.tool_calls):
                        send(chunk({"tool_calls": [dict(call, index=i)]}))
                    if stops.hit and ev is None:
                        gen.cancelled.set()
                reason = "stop" if stops.hit else fin.reason
                finish, err = self._finalise(req, parser, content_all, reason)
                if err:
                    raise ApiError(500, err)
            except (ApiError, C.ChatError) as e:
                self.counters["errors"] += 1
                msg = e.message if isinstance(e, ApiError) else str(e)
                send({"error": {"message": msg[:512], "type": "native_v41_error"}})
                return
            usage.update(fin.usage)
            usage["total_tokens"] = usage.get("prompt_tokens", 0) + usage.get("completion_tokens", 0)
            send(chunk({}, finish))
            if req.include_usage:
                o = chunk({}, None, {"usage": usage})
                o["choices"] = []
                send(o)
            send(b"[DONE]")
        except (BrokenPipeError, ConnectionResetError):
            gen.cancelled.set()              # client went away: stop generating


def tool_call_grammar(tools, tool_choice, parallel: bool, triggered: bool = False) -> dict:
    """Grammar description of a DSML calls block for the declared tools (string parameters raw, others JSON).
    `triggered` (tool_choice "auto"): the answer is plain text, or text up to the tag that opens a calls block and
    then a block that must be well formed - the model is free until it writes the tag
    (reference: rust/crates/ds41rt-api/src/native_v41/constraints.rs:35, the triggered-tag structural grammar)."""
    names = [t["function"]["name"] for t in tools]
    if isinstance(tool_choice, dict):
        names = [tool_choice["function"]["name"]]
    invokes = []
    for t in tools:
        fn = t["function"]
        if fn["name"] not in names:
            continue
        props = (fn.get("parameters") or {}).get("properties") or {}
        required = set((fn.get("parameters") or {}).get("required") or [])
        params = []
        for key, sch in props.items():
            is_str = sch.get("type") == "string" and "enum" not in sch
            if is_str:
                value = {"until": C.DSML_CLOSE}
                node = {"seq": [{"lit": f'{C.DSML_OPEN} parameter name="{key}" string="true">'}, value,
                                {"lit": " parameter>\n"}]}
            else:
                node = {"seq": [{"lit": f'{C.DSML_OPEN} parameter name="{key}" string="false">'}, {"schema": sch},
                                {"lit": f"{C.DSML_CLOSE} parameter>\n"}]}
            params.append(node if key in required else {"repeat": [node, 0, 1]})
        invokes.append({"seq": [{"lit": f'{C.DSML_OPEN} invoke name="{fn["name"]}">\n'}] + params +
                               [{"lit": f"{C.DSML_CLOSE} invoke>\n"}]})
    one = {"alt": invokes}
    body = {"repeat": [one, 1, -1 if parallel else 1]}
    if triggered:
        return {"alt": [{"text_without": C.CALLS_OPEN},
                        {"seq": [{"until": C.CALLS_OPEN}, {"lit": "\n"}, body, {"lit": C.CALLS_CLOSE}]}]}
    return {"seq": [{"lit": C.CALLS_OPEN + "\n"}, body, {"lit": C.CALLS_CLOSE}]}
