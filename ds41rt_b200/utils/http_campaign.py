"""Concurrency campaign through the HTTP API: N clients, mixed traffic, one JSON line of results.

    python -m ds41rt_b200.utils.http_campaign --model flash --layers 10 --clients 16 --requests 48
    python -m ds41rt_b200.utils.http_campaign --url http://127.0.0.1:8000 --clients 16        # against a running server

Without --url the tool builds the engine (random-init weights of the named architecture, byte-level tokenizer), starts
`serving.http.ApiServer` over `NativeBackend` in this process and talks to it over a real socket, so every request goes
through admission, chat templating, tokenisation, the scheduler (prompt chunks interleaved with decode rounds, graph
replays, speculative rounds for up to four active requests), sampling and SSE framing.  Traffic mix per client, round robin:
greedy streaming, seeded sampling (temperature / top-p), a JSON-schema-constrained answer, and a follow-up turn that
extends an earlier prompt (prefix reuse).  Reported: completed requests, aggregate completion tokens per second over
the wall clock of the campaign, time to first streamed token (median / p95), and the server's own counters.

Counterpart of the reference's API concurrency campaigns (scripts/bench-ds41-api-concurrency.py in the reference tree).
"""
from __future__ import annotations

import argparse
import http.client
import json
import statistics
import threading
import time
from urllib.parse import urlparse

MODEL_ID = "deepseek-ai/DeepSeek-V4.1-Flash"

SCHEMA = {"type": "object",
          "properties": {"city": {"type": "string"}, "days": {"type": "integer"}, "metric": {"type": "boolean"}},
          "required": ["city", "days", "metric"]}


def _request_body(kind: str, i: int, max_tokens: int, history):
    text = f"Request {i}: list three facts about the number {17 * i + 3}. " * 4
    msgs = [{"role": "user", "content": text}]
    body = {"model": MODEL_ID, "messages": msgs, "max_tokens": max_tokens, "stream": True,
            "stream_options": {"include_usage": True}, "thinking": {"type": "disabled"}}
    if kind == "sampled":
        body.update(temperature=0.8, top_p=0.9, seed=1000 + i)
    elif kind == "schema":
        body.update(temperature=0.0, response_format={"type": "json_schema", "json_schema": {"name": "trip",
                                                                                              "schema": SCHEMA}})
    elif kind == "followup" and history:
        prev_msgs, prev_answer = history[-1]
        body["messages"] = prev_msgs + [{"role": "assistant", "content": prev_answer},
                                        {"role": "user", "content": "Now shorter, please."}]
        body["temperature"] = 0.0
    else:
        body["temperature"] = 0.0
    return body


def _stream(host: str, port: int, body: dict, timeout: float):
    """POST one streaming chat completion -> (status, text, completion tokens, seconds to first token, seconds total)."""
    t0 = time.perf_counter()
    c = http.client.HTTPConnection(host, port, timeout=timeout)
    c.request("POST", "/v1/chat/completions", body=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    r = c.getresponse()
    if r.status != 200:
        raw = r.read().decode("utf-8", "replace")
        c.close()
        return r.status, raw[:200], 0, None, time.perf_counter() - t0
    first, text, tokens = None, [], 0
    for line in r:
        if not line.startswith(b"data: "):
            continue
        data = line[6:].strip()
        if data == b"[DONE]":
            break
        ev = json.loads(data)
        if "error" in ev:
            c.close()
            return 500, str(ev["error"])[:200], tokens, first, time.perf_counter() - t0
        if ev.get("usage"):
            tokens = ev["usage"].get("completion_tokens", tokens)
        for ch in ev.get("choices", []):
            delta = ch.get("delta") or {}
            piece = delta.get("content") or delta.get("reasoning_content") or ""
            if piece:
                if first is None:
                    first = time.perf_counter() - t0
                text.append(piece)
    c.close()
    return 200, "".join(text), tokens, first, time.perf_counter() - t0


def run_campaign(host: str, port: int, clients: int, requests: int, max_tokens: int, timeout: float = 600.0) -> dict:
    kinds = ["greedy", "sampled", "schema", "followup"]
    lock = threading.Lock()
    results, next_i = [], [0]

    def client(cid: int):
        history = []
        while True:
            with lock:
                i = next_i[0]
                if i >= requests:
                    return
                next_i[0] += 1
            kind = kinds[i % len(kinds)]
            if kind == "followup" and not history:
                kind = "greedy"
            body = _request_body(kind, i, max_tokens, history)
            status, text, tokens, first, total = _stream(host, port, body, timeout)
            if status == 200 and kind in ("greedy", "followup"):
                history.append((body["messages"], text))
            with lock:
                results.append({"kind": kind, "status": status, "tokens": tokens, "first_s": first, "total_s": total,
                                "valid_json": (_valid(text) if kind == "schema" and status == 200 else None)})

    t0 = time.perf_counter()
    threads = [threading.Thread(target=client, args=(c,)) for c in range(clients)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    ok = [r for r in results if r["status"] == 200]
    firsts = sorted(r["first_s"] for r in ok if r["first_s"] is not None)
    toks = sum(r["tokens"] for r in ok)
    by_kind = {k: sum(1 for r in ok if r["kind"] == k) for k in kinds}
    schema = [r["valid_json"] for r in ok if r["valid_json"] is not None]
    return {"clients": clients, "requests": requests, "completed": len(ok), "rejected_429": sum(r["status"] == 429 for r in results),
            "failed": sum(r["status"] not in (200, 429) for r in results), "by_kind": by_kind,
            "schema_answers_valid_or_valid_prefix": f"{sum(schema)}/{len(schema)}", "completion_tokens": toks, "wall_s": round(wall, 3),
            "tok_per_s": round(toks / wall, 1) if wall > 0 else 0.0,
            "ttft_s": {"median": round(statistics.median(firsts), 4) if firsts else None,
                       "p95": round(firsts[int(0.95 * (len(firsts) - 1))], 4) if firsts else None}}


def _valid(text: str) -> bool:
    """A complete answer must parse and carry the required fields; an answer cut off by max_tokens must still be a prefix
    the schema's grammar accepts (a random-init model rarely closes its strings)."""
    try:
        doc = json.loads(text)
        return isinstance(doc, dict) and set(SCHEMA["required"]) <= set(doc)
    except ValueError:
        from ..runtime.grammar import Grammar, Matcher
        return bool(text) and Matcher(Grammar.json_schema(SCHEMA)).accept_bytes(text.encode("utf-8"))


def _local_server(args):
    import torch
    from ..config import ModelConfig
    from ..models.ds41 import DS41Engine, EngineWeights
    from ..serving.engine import NativeBackend
    from ..serving.http import ApiServer
    from ..serving.tokenizer import ByteTokenizer
    dev = torch.device("cuda", 0)
    cfg = ModelConfig.flash(args.layers) if args.model == "flash" else getattr(ModelConfig, args.model)()
    weights = EngineWeights.random(cfg, 0, 1, dev, seed=0, expert_dtype=args.expert_dtype if args.model == "flash" else "bf16")
    slots = args.clients
    eng = DS41Engine(cfg, weights, max_rows=max(64, args.prefill_chunk), slots=slots, max_ctx=args.max_context,
                     kv_dtype=args.kv_dtype)
    drafter = None
    if cfg.dspark is not None and not args.no_drafter:
        from ..models.dspark import DSparkDrafter
        drafter = DSparkDrafter(cfg, eng, weights=None, seed=0,
                                expert_dtype=args.expert_dtype if args.model == "flash" else "bf16")
    tk = ByteTokenizer(vocab_size=cfg.vocab)
    backend = NativeBackend(eng, eos=tk.eos, concurrency=slots, queue_depth=4 * args.clients, drafter=drafter,
                            prefill_chunk=args.prefill_chunk)
    srv = ApiServer(backend, tk, queue_depth=4 * args.clients, waiters=4 * args.clients,
                    max_context=args.max_context).start()
    return srv, backend, cfg


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="", help="base URL of a running server (default: start one in this process)")
    ap.add_argument("--clients", type=int, default=16)
    ap.add_argument("--requests", type=int, default=48)
    ap.add_argument("--max-tokens", type=int, default=48)
    ap.add_argument("--model", default="flash", choices=["flash", "small", "tiny"])
    ap.add_argument("--layers", type=int, default=10)
    ap.add_argument("--expert-dtype", default="mxfp8")
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8", "fp4"])
    ap.add_argument("--max-context", type=int, default=4096)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--no-drafter", action="store_true")
    args = ap.parse_args(argv)
    srv = backend = None
    if args.url:
        u = urlparse(args.url)
        host, port = u.hostname, u.port or 80
        where = {"server": args.url}
    else:
        srv, backend, cfg = _local_server(args)
        host, port = "127.0.0.1", srv.port
        where = {"server": "in-process", "model": cfg.name, "layers": cfg.n_layers, "expert_dtype": args.expert_dtype,
                 "kv_dtype": args.kv_dtype}
    try:
        run_campaign(host, port, min(2, args.clients), 2, 8)                 # warm-up: graphs, grammar tables
        out = run_campaign(host, port, args.clients, args.requests, args.max_tokens)
        out.update(where)
        if backend is not None:
            st = backend.stats()
            t = st["totals"]
            out["server_totals"] = {k: t[k] for k in ("rounds", "graph_rounds", "spec_rounds", "prefill_passes",
                                                      "prompt_cache_hit_tokens", "gpu_sampled_rows",
                                                      "device_greedy_rows", "failed") if k in t}
        print(json.dumps(out))
    finally:
        if srv is not None:
            srv.stop()
        if backend is not None:
            backend.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
