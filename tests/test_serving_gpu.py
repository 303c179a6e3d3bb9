"""OpenAI API over the native engine on one GPU: greedy, seeded sampling on the GPU sampler, JSON-schema output."""
import http.client
import json

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def server():
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.serving.engine import NativeBackend
    from ds41rt_b200.serving.http import ApiServer
    from ds41rt_b200.serving.tokenizer import ByteTokenizer
    cfg = ModelConfig.tiny()
    tk = ByteTokenizer(vocab_size=cfg.vocab)
    dev = torch.device("cuda", 0)
    eng = DS41Engine(cfg, EngineWeights.random(cfg, 0, 1, dev, seed=0), max_rows=8, slots=4, max_ctx=1024)
    backend = NativeBackend(eng, eos=tk.eos, concurrency=4)
    srv = ApiServer(backend, tk, queue_depth=8, waiters=4, first_event_timeout=60.0).start()
    yield srv, backend
    srv.stop()
    backend.close()


def _call(srv, body):
    c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=120)
    c.request("POST", "/v1/chat/completions", body=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    r = c.getresponse()
    raw = r.read().decode()
    c.close()
    return r.status, raw


def _body(**kw):
    from ds41rt_b200.serving.protocol import MODEL_ID
    b = {"model": MODEL_ID, "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 24}
    b.update(kw)
    return b


def test_greedy_is_repeatable(server):
    srv, _ = server
    a = _call(srv, _body(temperature=0))
    b = _call(srv, _body(temperature=0))
    assert a[0] == 200 and b[0] == 200
    ja, jb = json.loads(a[1]), json.loads(b[1])
    assert ja["choices"][0]["message"] == jb["choices"][0]["message"]
    assert ja["usage"]["completion_tokens"] >= 1


def test_seeded_sampling_runs_on_the_gpu_sampler(server):
    srv, backend = server
    before = backend.totals["gpu_sampled_rows"]
    a = _call(srv, _body(temperature=0.9, top_p=0.9, top_k=50, seed=7))
    b = _call(srv, _body(temperature=0.9, top_p=0.9, top_k=50, seed=7))
    c = _call(srv, _body(temperature=0.9, top_p=0.9, top_k=50, seed=8))
    assert a[0] == 200 and b[0] == 200 and c[0] == 200
    assert json.loads(a[1])["choices"][0]["message"] == json.loads(b[1])["choices"][0]["message"]
    assert backend.totals["gpu_sampled_rows"] > before and backend.totals["cpu_sampled_rows"] == 0


def test_json_schema_output_validates(server):
    srv, _ = server
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}},
              "required": ["ok", "n"], "additionalProperties": False}
    st, raw = _call(srv, _body(temperature=0.8, seed=3, max_tokens=64, thinking={"type": "disabled"},
                               response_format={"type": "json_schema",
                                                "json_schema": {"name": "r", "strict": True, "schema": schema}}))
    assert st == 200, raw
    msg = json.loads(raw)["choices"][0]
    if msg["finish_reason"] == "stop":
        val = json.loads(msg["message"]["content"])
        assert isinstance(val["ok"], bool) and isinstance(val["n"], int)


def test_official_checkpoint_streams_into_the_engine(tmp_path):
    """export -> validated catalog -> lazy per-tensor streaming into a rank shard -> same logits as eager loading."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.loader import Catalog
    from ds41rt_b200.loader.official import export_official, load_engine_weights, load_official
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.weights import init_weights
    cfg = ModelConfig.tiny()
    d = str(tmp_path / "ckpt")
    export_official(cfg, init_weights(cfg, seed=5), d, shards=3)
    dev = torch.device("cuda", 0)
    streamed = load_engine_weights(d, cfg, 0, 1, dev, expert_dtype="bf16")
    eager = EngineWeights.from_fp32(cfg, load_official(Catalog(d, cfg, with_vision=False, with_engram=False)), 0, 1, dev)
    toks = list(range(5, 21))
    outs = []
    for w in (streamed, eager):
        eng = DS41Engine(cfg, w, max_rows=16, slots=1, max_ctx=256)
        eng.cache.ensure(0, 64)
        eng.set_rows(toks, list(range(len(toks))), [0] * len(toks))
        eng.forward_rows(len(toks), head=True)
        outs.append(eng.logits_rows(len(toks)).clone())
        eng.check_status()
    assert torch.equal(outs[0], outs[1])


def test_prefix_snapshots_reuse_prompt_and_turn(server):
    """A second request that extends an earlier prompt (or an earlier whole turn) restarts from the stored snapshot:
    usage reports the reused tokens and the continuation is what a cold run produces."""
    srv, backend = server
    from ds41rt_b200.serving.engine import GenRequest
    from ds41rt_b200.serving.protocol import Sampling
    g = torch.Generator().manual_seed(9)
    base = torch.randint(3, 2000, (70,), generator=g).tolist()
    ext = base + torch.randint(3, 2000, (25,), generator=g).tolist()

    def run(prompt, n=10):
        r = GenRequest(prompt_ids=prompt, max_tokens=n, sampling=Sampling(temperature=0.0))
        backend.submit(r)
        toks, usage = [], None
        while True:
            ev = r.events.get(timeout=120)
            if ev.kind == "ready":
                usage = ev.usage
            elif ev.kind == "tokens":
                toks += ev.tokens
            elif ev.kind == "finish":
                return toks, usage
            elif ev.kind == "error":
                raise RuntimeError(ev.message)

    backend.snapshots.clear()
    cold, u0 = run(ext)                                  # nothing stored yet
    assert u0["prompt_cache_hit_tokens"] == 0
    backend.snapshots.clear()
    first, _ = run(base)                                 # stores a prompt snapshot (70) and a turn snapshot (70 + 9)
    warm, u1 = run(ext)                                  # continues from the 70-token prompt snapshot
    assert u1["prompt_cache_hit_tokens"] == len(base)
    assert warm == cold
    again, u2 = run(base)                                # exact prompt hit: no prefill at all, first token from stored logits
    assert u2["prompt_cache_hit_tokens"] == len(base) and again == first
    turn = base + first[:-1] + [77, 78, 79]
    _, u3 = run(turn)                                    # previous turn + new tokens: continues from the turn snapshot
    assert u3["prompt_cache_hit_tokens"] == len(base) + len(first) - 1


def test_image_parts_reach_the_vision_tower():
    """A chat request with an image: decoded and gridded on the HTTP thread, encoded by the tower on the worker, its
    rows replace the placeholder embeddings; a different image changes the answer, a bad image is a 400."""
    import base64
    import io

    import numpy as np
    from PIL import Image

    from ds41rt_b200.config import ModelConfig, VisionConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.vision import VisionTower, init_vision_weights
    from ds41rt_b200.serving.engine import NativeBackend
    from ds41rt_b200.serving.http import ApiServer
    from ds41rt_b200.serving.tokenizer import ByteTokenizer
    cfg = ModelConfig.tiny()
    v = VisionConfig(layers=2, hidden=256, heads=4, intermediate=384, min_pixels=42 * 42 * 4, max_image_tokens=16)
    dev = torch.device("cuda", 0)
    tk = ByteTokenizer(vocab_size=cfg.vocab, extra_specials=["<image>", "<image_start>", "<image_end>", "<image_newline>"])
    eng = DS41Engine(cfg, EngineWeights.random(cfg, 0, 1, dev, seed=0), max_rows=16, slots=2, max_ctx=1024)
    tower = VisionTower(v, init_vision_weights(v, cfg.hidden, 2, seed=4, std=0.05), cfg.hidden, 2, dev, max_patches=144)
    backend = NativeBackend(eng, eos=tk.eos, concurrency=2, vision=tower)
    srv = ApiServer(backend, tk, queue_depth=4, waiters=2, first_event_timeout=60.0, vision_cfg=v).start()

    def data_url(seed):
        rng = np.random.default_rng(seed)
        buf = io.BytesIO()
        Image.fromarray(rng.integers(0, 256, size=(90, 120, 3), dtype=np.uint8)).save(buf, format="PNG")
        return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()

    def ask(url):
        body = _body(temperature=0, max_tokens=8, thinking={"type": "disabled"})
        body["messages"] = [{"role": "user", "content": [{"type": "text", "text": "what is this "},
                                                         {"type": "image_url", "image_url": {"url": url}}]}]
        return _call(srv, body)

    try:
        a, b, c = ask(data_url(1)), ask(data_url(1)), ask(data_url(2))
        assert a[0] == 200 and b[0] == 200 and c[0] == 200, (a, c)
        ma, mb, mc = (json.loads(x[1])["choices"][0]["message"]["content"] for x in (a, b, c))
        assert ma == mb
        assert json.loads(a[1])["usage"]["prompt_tokens"] > 20          # the span is part of the prompt
        bad = ask("data:image/png;base64," + base64.b64encode(b"nope").decode())
        assert bad[0] == 400
        print("image answers differ:", ma != mc)
    finally:
        srv.stop()
        backend.close()


def test_solo_request_is_served_by_speculative_rounds():
    """With a drafter, a lone greedy request runs draft + verify rounds and produces exactly the tokens plain decoding
    produces; when a second request joins mid-way both still receive exactly those tokens."""
    import threading
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.dspark import DSparkDrafter
    from ds41rt_b200.serving.engine import GenRequest, NativeBackend
    from ds41rt_b200.serving.protocol import Sampling
    cfg = ModelConfig.tiny()
    dev = torch.device("cuda", 0)
    w = EngineWeights.random(cfg, 0, 1, dev, seed=0)

    def backend(with_drafter):
        eng = DS41Engine(cfg, w, max_rows=8, slots=4, max_ctx=512)
        drafter = DSparkDrafter(cfg, eng, weights=None, seed=0) if with_drafter else None
        return NativeBackend(eng, eos=1, concurrency=4, drafter=drafter)

    def collect(r):
        toks = []
        while True:
            ev = r.events.get(timeout=120)
            if ev.kind == "tokens":
                toks += ev.tokens
            elif ev.kind == "finish":
                return toks
            elif ev.kind == "error":
                raise RuntimeError(ev.message)

    g = torch.Generator().manual_seed(21)
    p1 = torch.randint(3, 2000, (40,), generator=g).tolist()
    p2 = torch.randint(3, 2000, (33,), generator=g).tolist()
    req = lambda p, n: GenRequest(prompt_ids=p, max_tokens=n, sampling=Sampling(temperature=0.0))
    plain = backend(False)
    r = req(p1, 40); plain.submit(r); want1 = collect(r)
    r = req(p2, 12); plain.submit(r); want2 = collect(r)
    plain.close()
    spec = backend(True)
    r = req(p1, 40); spec.submit(r)
    assert collect(r) == want1
    assert spec.totals["spec_rounds"] > 0 and spec.totals["spec_tokens"] >= spec.totals["spec_rounds"]
    spec.snapshots.clear()
    a, b = req(p1, 40), req(p2, 12)
    spec.submit(a)
    threading.Timer(0.05, lambda: spec.submit(b)).start()
    assert collect(a) == want1 and collect(b) == want2
    assert spec.healthy, spec.error
    spec.close()


def test_speculative_rounds_serve_constrained_and_sampled_requests_losslessly():
    """A lone request decodes by draft + verify rounds also when it is grammar-constrained (verification rows selected
    under the masks of a matcher fork per draft row, proposals cut at the first rejected token) or stochastic (rows drawn
    with the request's own (seed, position) numbers; a draft counts while it equals the draw).  Both produce exactly the
    tokens of a backend without a drafter; decode rounds of that backend replay captured graphs and agree with eager
    launches; the verification policy reports its fit."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.dspark import DSparkDrafter
    from ds41rt_b200.runtime.grammar import Grammar, TokenConstraint, Vocab
    from ds41rt_b200.serving.engine import GenRequest, NativeBackend
    from ds41rt_b200.serving.protocol import Sampling
    from ds41rt_b200.serving.tokenizer import ByteTokenizer
    cfg = ModelConfig.tiny()
    dev = torch.device("cuda", 0)
    w = EngineWeights.random(cfg, 0, 1, dev, seed=0)
    tk = ByteTokenizer(vocab_size=cfg.vocab)
    vocab = Vocab(tk.token_bytes())
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "n": {"type": "integer"},
                                               "kind": {"enum": ["a", "b"]}}, "required": ["name", "n", "kind"]}

    def backend(with_drafter, graphs=True):
        eng = DS41Engine(cfg, w, max_rows=8, slots=4, max_ctx=512)
        drafter = DSparkDrafter(cfg, eng, weights=None, seed=0) if with_drafter else None
        return NativeBackend(eng, eos=tk.eos, concurrency=4, drafter=drafter, use_graphs=graphs)

    def collect(r):
        toks = []
        while True:
            ev = r.events.get(timeout=120)
            if ev.kind == "tokens":
                toks += ev.tokens
            elif ev.kind == "finish":
                return toks
            elif ev.kind == "error":
                raise RuntimeError(ev.message)

    g = torch.Generator().manual_seed(33)
    prompt = torch.randint(3, 250, (40,), generator=g).tolist()

    def requests():
        con = TokenConstraint(vocab, Grammar.json_schema(schema), eos=tk.eos)
        return [GenRequest(prompt_ids=prompt, max_tokens=48, sampling=Sampling(temperature=0.0), constraint=con),
                GenRequest(prompt_ids=prompt, max_tokens=32, sampling=Sampling(temperature=0.8, top_p=0.95, top_k=40,
                                                                               seed=5))]

    out = {}
    for name, be in (("plain", backend(False)), ("eager", backend(False, graphs=False)), ("spec", backend(True))):
        res = []
        for r in requests():
            be.snapshots.clear()
            be.submit(r)
            res.append(collect(r))
        out[name] = (res, dict(be.totals), be.stats())
        assert be.healthy, be.error
        be.close()
    assert out["plain"][0] == out["eager"][0] == out["spec"][0]
    assert out["plain"][1]["graph_rounds"] > 0 and out["eager"][1]["graph_rounds"] == 0
    tot = out["spec"][1]
    assert tot["spec_masked_rounds"] > 0 and tot["spec_rounds"] >= tot["spec_masked_rounds"]
    pol = out["spec"][2]["dspark_policy"]
    assert pol["rounds"] > 0 and len(pol["accepted_histogram"]) == 16
    text = tk.decode(out["spec"][0][0])
    assert text.lstrip().startswith("{")


def test_concurrent_requests_share_speculative_rounds_losslessly():
    """Several active requests - greedy, grammar-constrained and seeded-stochastic - decode by shared draft + verify
    rounds (one draft pass and one target pass for all of them) and each receives exactly the tokens that a backend
    without a drafter gives it when it runs alone."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.dspark import DSparkDrafter
    from ds41rt_b200.runtime.grammar import Grammar, TokenConstraint, Vocab
    from ds41rt_b200.serving.engine import GenRequest, NativeBackend
    from ds41rt_b200.serving.protocol import Sampling
    from ds41rt_b200.serving.tokenizer import ByteTokenizer
    cfg = ModelConfig.tiny()
    dev = torch.device("cuda", 0)
    w = EngineWeights.random(cfg, 0, 1, dev, seed=0)
    tk = ByteTokenizer(vocab_size=cfg.vocab)
    vocab = Vocab(tk.token_bytes())
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "n": {"type": "integer"}},
              "required": ["name", "n"]}

    def backend(with_drafter):
        eng = DS41Engine(cfg, w, max_rows=32, slots=4, max_ctx=512)
        drafter = DSparkDrafter(cfg, eng, weights=None, seed=0) if with_drafter else None
        return NativeBackend(eng, eos=tk.eos, concurrency=4, drafter=drafter)

    def collect(r):
        toks = []
        while True:
            ev = r.events.get(timeout=120)
            if ev.kind == "tokens":
                toks += ev.tokens
            elif ev.kind == "finish":
                return toks
            elif ev.kind == "error":
                raise RuntimeError(ev.message)

    g = torch.Generator().manual_seed(44)
    prompts = [torch.randint(3, 250, (n,), generator=g).tolist() for n in (40, 33, 47)]

    def requests():
        con = TokenConstraint(vocab, Grammar.json_schema(schema), eos=tk.eos)
        return [GenRequest(prompt_ids=prompts[0], max_tokens=60, sampling=Sampling(temperature=0.0)),
                GenRequest(prompt_ids=prompts[1], max_tokens=56, sampling=Sampling(temperature=0.0), constraint=con),
                GenRequest(prompt_ids=prompts[2], max_tokens=52, sampling=Sampling(temperature=0.7, top_p=0.9, seed=9))]

    plain = backend(False)
    want = []
    for r in requests():
        plain.submit(r)
        want.append(collect(r))
    plain.close()
    spec = backend(True)
    assert spec.spec_lanes >= 3
    reqs = requests()
    for r in reqs:
        spec.submit(r)
    got = [collect(r) for r in reqs]
    tot = dict(spec.totals)
    assert spec.healthy, spec.error
    spec.close()
    assert got == want
    assert tot["spec_lane_rounds"] > 0 and tot["spec_tokens"] >= tot["spec_rounds"]


def test_engram_pipeline_serves_requests(tmp_path):
    """A backend whose engine has an Engram layer: every pass hashes its tokens, gathers table rows on the I/O thread and
    applies the gated update.  The emitted tokens are what the fp32 oracle picks when it is given the same rows
    (teacher forced over the emitted sequence), and a request continued from a prompt snapshot emits the same tokens as
    a cold run (the slot's n-gram history is rebuilt from the reused tokens)."""
    import numpy as np
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.engram import (EngramLayer, dequant_rows_reference, engram_reference,
                                            init_engram_weights, random_table_rows)
    from ds41rt_b200.models.reference import ReferenceModel
    from ds41rt_b200.models.weights import init_weights
    from ds41rt_b200.runtime.core import EngramHistory
    from ds41rt_b200.runtime.engram import EngramPipeline
    from ds41rt_b200.runtime.engram_io import EngramTable
    from ds41rt_b200.serving.engine import GenRequest, NativeBackend
    from ds41rt_b200.serving.protocol import Sampling
    cfg = ModelConfig.tiny()
    w = init_weights(cfg, seed=11)
    dev = torch.device("cuda", 0)
    n_rows = 4096
    rec = random_table_rows(n_rows, seed=2)
    path = str(tmp_path / "engram.bin")
    rec.numpy().tofile(path)
    wkv, q_w, k_w = init_engram_weights(cfg.hidden, seed=4, std=0.002)
    bf = lambda t: t.bfloat16()
    eng = DS41Engine(cfg, EngineWeights.from_fp32(cfg, w, 0, 1, dev), max_rows=16, slots=2, max_ctx=512)
    eng.attach_engram(1, EngramLayer(bf(wkv).to(dev), bf(q_w).to(dev), bf(k_w).to(dev), cfg.hidden))
    pipe = EngramPipeline([1], [EngramTable(path, n_rows, 264)], pad_id=2, max_rows=16, fold=True)
    backend = NativeBackend(eng, eos=cfg.vocab - 1, concurrency=2, engram=pipe)

    def run(prompt, n=8):
        r = GenRequest(prompt_ids=prompt, max_tokens=n, sampling=Sampling(temperature=0.0))
        backend.submit(r)
        toks, usage = [], None
        while True:
            ev = r.events.get(timeout=120)
            if ev.kind == "ready":
                usage = ev.usage
            elif ev.kind == "tokens":
                toks += ev.tokens
            elif ev.kind == "finish":
                return toks, usage
            elif ev.kind == "error":
                raise RuntimeError(ev.message)

    try:
        g = torch.Generator().manual_seed(3)
        prompt = torch.randint(3, 2000, (40,), generator=g).tolist()
        cold, _ = run(prompt + [5, 6, 7])
        backend.snapshots.clear()
        got, _ = run(prompt)
        warm, usage = run(prompt + [5, 6, 7])
        assert usage["prompt_cache_hit_tokens"] == len(prompt) and warm == cold
        assert pipe.stats()["gather"][0]["requests"] > 0
    finally:
        backend.close()
    # teacher-forced oracle over prompt + emitted tokens with the same table rows
    full = prompt + got
    ids = (EngramHistory(2).prepare(full)[:, 0, :].reshape(-1) % np.uint64(n_rows)).astype(np.int64)
    deq = dequant_rows_reference(rec[torch.from_numpy(ids)], 256).bfloat16().view(len(full), 24 * 256)
    ref = ReferenceModel(cfg, w)
    ref.engram_hook = lambda l, s: engram_reference(s.bfloat16(), deq[: s.shape[0]], bf(wkv), bf(q_w), bf(k_w)) if l == 1 else s
    logits = ref.forward(torch.tensor(full))
    want = logits[len(prompt) - 1:-1].argmax(-1).tolist()
    agree = sum(int(a == b) for a, b in zip(want, got))
    assert agree >= len(got) - 2, (want, got)
    plain = ReferenceModel(cfg, w).forward(torch.tensor(full))[len(prompt) - 1:-1].argmax(-1).tolist()
    assert plain != want                                  # the memory layer changes what is generated


def test_engram_backend_speculates_losslessly(tmp_path):
    """An engine with an Engram layer and a drafter: the drafts come back to the host before the verification pass (the
    n-gram hashes of its rows need them), only the accepted rows advance the slot's history, and the request emits what
    the same engine emits without the drafter."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.dspark import DSparkDrafter
    from ds41rt_b200.models.engram import EngramLayer, init_engram_weights, random_table_rows
    from ds41rt_b200.runtime.engram import EngramPipeline
    from ds41rt_b200.runtime.engram_io import EngramTable
    from ds41rt_b200.serving.engine import GenRequest, NativeBackend
    from ds41rt_b200.serving.protocol import Sampling
    cfg = ModelConfig.tiny()
    dev = torch.device("cuda", 0)
    w = EngineWeights.random(cfg, 0, 1, dev, seed=0)
    n_rows = 4096
    path = str(tmp_path / "engram.bin")
    random_table_rows(n_rows, seed=2).numpy().tofile(path)
    wkv, q_w, k_w = init_engram_weights(cfg.hidden, seed=4, std=0.002)
    bf = lambda t: t.bfloat16().to(dev)

    def backend(with_drafter, rows=8):
        eng = DS41Engine(cfg, w, max_rows=rows, slots=2, max_ctx=512)
        eng.attach_engram(1, EngramLayer(bf(wkv), bf(q_w), bf(k_w), cfg.hidden, max_tokens=rows))
        pipe = EngramPipeline([1], [EngramTable(path, n_rows, 264)], pad_id=2, max_rows=rows, fold=True)
        drafter = DSparkDrafter(cfg, eng, weights=None, seed=0) if with_drafter else None
        return NativeBackend(eng, eos=1, concurrency=2, engram=pipe, drafter=drafter)

    def run(b, prompt, n):
        r = GenRequest(prompt_ids=prompt, max_tokens=n, sampling=Sampling(temperature=0.0))
        b.submit(r)
        toks = []
        while True:
            ev = r.events.get(timeout=120)
            if ev.kind == "tokens":
                toks += ev.tokens
            elif ev.kind == "finish":
                return toks
            elif ev.kind == "error":
                raise RuntimeError(ev.message)

    prompt = torch.randint(3, 2000, (40,), generator=torch.Generator().manual_seed(9)).tolist()
    plain = backend(False)
    try:
        want = run(plain, prompt, 24)
    finally:
        plain.close()
    spec = backend(True)
    try:
        got = run(spec, prompt, 24)
        assert got == want
        assert spec.totals["spec_rounds"] > 0 and spec.totals["spec_masked_rounds"] == spec.totals["spec_rounds"]
        assert spec.healthy, spec.error
    finally:
        spec.close()
    # two requests at once share draft + verify rounds; each slot's n-gram history advances by its accepted rows only
    prompt2 = torch.randint(3, 2000, (31,), generator=torch.Generator().manual_seed(10)).tolist()
    plain = backend(False, rows=16)
    try:
        want2 = run(plain, prompt2, 20)
    finally:
        plain.close()
    spec = backend(True, rows=16)
    try:
        ra = GenRequest(prompt_ids=prompt, max_tokens=24, sampling=Sampling(temperature=0.0))
        rb = GenRequest(prompt_ids=prompt2, max_tokens=20, sampling=Sampling(temperature=0.0))
        spec.submit(ra)
        spec.submit(rb)
        outs = []
        for r in (ra, rb):
            toks = []
            while True:
                ev = r.events.get(timeout=120)
                if ev.kind == "tokens":
                    toks += ev.tokens
                elif ev.kind == "finish":
                    break
                elif ev.kind == "error":
                    raise RuntimeError(ev.message)
            outs.append(toks)
        assert outs == [want, want2]
        assert spec.totals["spec_lane_rounds"] > 0 and spec.healthy, spec.error
    finally:
        spec.close()


def test_host_tier_restore_continues_like_a_cold_run():
    """Page pressure pushes a prompt snapshot out of the device pool into pinned host pages; a prompt that extends it
    is restored from them (H2D page copies, rings, carry) and generates exactly what a backend without any cache
    generates."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.serving.engine import GenRequest, NativeBackend
    from ds41rt_b200.serving.protocol import Sampling
    cfg = ModelConfig.tiny()
    dev = torch.device("cuda", 0)
    w = EngineWeights.random(cfg, 0, 1, dev, seed=0)

    def run(b, prompt, n):
        r = GenRequest(prompt_ids=prompt, max_tokens=n, sampling=Sampling(temperature=0.0))
        b.submit(r)
        toks, usage = [], None
        while True:
            ev = r.events.get(timeout=120)
            if ev.kind == "ready":
                usage = ev.usage
            elif ev.kind == "tokens":
                toks += ev.tokens
            elif ev.kind == "finish":
                return toks, usage
            elif ev.kind == "error":
                raise RuntimeError(ev.message)

    g = torch.Generator().manual_seed(4)
    first = torch.randint(3, 2000, (130,), generator=g).tolist()
    big = torch.randint(3, 2000, (440,), generator=g).tolist()
    tail = [11, 12, 13]
    cold = NativeBackend(DS41Engine(cfg, w, max_rows=16, slots=2, max_ctx=512), eos=1, concurrency=2)
    try:
        want, _ = run(cold, first + tail, 12)
    finally:
        cold.close()
    be = NativeBackend(DS41Engine(cfg, w, max_rows=16, slots=2, max_ctx=512, n_pages=9), eos=1, concurrency=2,
                       host_cache_bytes=64 << 20)
    try:
        run(be, first, 3)
        run(be, big, 60)                                   # 8 of the 9 pages: the first prompt's snapshot leaves the device
        assert be.totals["snapshots_demoted"] >= 1
        got, usage = run(be, first + tail, 12)
        assert be.totals["host_tier_hits"] == 1 and usage["prompt_cache_hit_tokens"] == len(first)
        assert got == want
    finally:
        be.close()


def test_partial_prefix_overlap_reuses_compressed_rows(server):
    """A prompt that shares only its first 100 tokens with a stored one: the compressed rows below
    skipped = 100 / 2 * 2 - window are taken from the snapshot, the tokens from there on are run again to rebuild the
    windows (their own compressed rows are kept up to the common prefix), and the request completes."""
    srv, backend = server
    from ds41rt_b200.serving.engine import GenRequest
    from ds41rt_b200.serving.protocol import Sampling
    g = torch.Generator().manual_seed(17)
    base = torch.randint(3, 2000, (100,), generator=g).tolist()
    a = base + torch.randint(3, 2000, (20,), generator=g).tolist()
    b = base + torch.randint(2001, 3000, (20,), generator=g).tolist()

    def run(prompt, n=6):
        r = GenRequest(prompt_ids=prompt, max_tokens=n, sampling=Sampling(temperature=0.0))
        backend.submit(r)
        toks, usage = [], None
        while True:
            ev = r.events.get(timeout=120)
            if ev.kind == "ready":
                usage = ev.usage
            elif ev.kind == "tokens":
                toks += ev.tokens
            elif ev.kind == "finish":
                return toks, usage
            elif ev.kind == "error":
                raise RuntimeError(ev.message)

    window = backend.e.cfg.window
    backend.snapshots.clear()
    cold, u0 = run(b)
    assert u0["prompt_cache_hit_tokens"] == 0
    backend.snapshots.clear()
    run(a)
    before = backend.totals["partial_prefix_hits"]
    warm, u1 = run(b)
    assert u1["prompt_cache_hit_tokens"] == 100 - window
    assert backend.totals["partial_prefix_hits"] == before + 1
    assert len(warm) == len(cold)
    # the rebuilt windows are complete for the newest tokens; the first generated token normally agrees
    print("agreement with the cold run:", sum(int(x == y) for x, y in zip(warm, cold)), "of", len(cold))
    again, u2 = run(b)                                   # now an exact hit on b's own prompt snapshot
    assert u2["prompt_cache_hit_tokens"] == len(b) and again == warm


def test_http_campaign_runs_mixed_traffic_through_the_real_server():
    """The campaign tool against an in-process server on the tiny model: greedy, sampled, schema-constrained and
    follow-up requests from four clients all complete, schema answers are valid (or valid prefixes when cut by
    max_tokens), and the follow-up turns hit the prefix banks."""
    import argparse
    from ds41rt_b200.utils import http_campaign as HC
    args = argparse.Namespace(model="tiny", layers=0, expert_dtype="bf16", kv_dtype="bf16", max_context=1024,
                              prefill_chunk=64, clients=4, no_drafter=False)
    srv, backend, cfg = HC._local_server(args)
    try:
        out = HC.run_campaign("127.0.0.1", srv.port, 4, 12, 24)
        assert out["completed"] == 12 and out["failed"] == 0 and out["rejected_429"] == 0
        assert out["by_kind"]["schema"] >= 2 and out["by_kind"]["sampled"] >= 2
        ok, total = map(int, out["schema_answers_valid_or_valid_prefix"].split("/"))
        assert ok == total
        assert out["completion_tokens"] > 0 and backend.healthy, backend.error
    finally:
        srv.stop()
        backend.close()


def test_prefill_matrix_reports_cold_and_retained_rows():
    """The matrix tool drives the backend like the HTTP layer does: a retained row restores the base from the prompt
    snapshot an earlier request left and computes only the rest; a cold row computes everything."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.serving.engine import NativeBackend
    from ds41rt_b200.utils.prefill_matrix import run_matrix
    cfg = ModelConfig.tiny()
    dev = torch.device("cuda", 0)
    eng = DS41Engine(cfg, EngineWeights.random(cfg, 0, 1, dev, seed=0), max_rows=32, slots=2, max_ctx=512)
    be = NativeBackend(eng, eos=-1, concurrency=1, prefill_chunk=32)
    try:
        rows = run_matrix(be, cfg.vocab, [0, 96], [16, 48])
        assert be.healthy, be.error
    finally:
        be.close()
    assert [(r["base"], r["suffix"], r["mode"]) for r in rows] == [
        (0, 16, "cold"), (0, 48, "cold"), (96, 16, "cold"), (96, 16, "retained"), (96, 48, "cold"), (96, 48, "retained")]
    for r in rows:
        assert r["seconds"] > 0 and r["tok_per_s"] > 0
        if r["mode"] == "cold":
            assert r["cache_hit_tokens"] == 0 and r["computed_tokens"] == r["base"] + r["suffix"]
        else:
            assert 0 < r["cache_hit_tokens"] <= r["base"] and r["computed_tokens"] < r["base"] + r["suffix"]
