"""End-to-end: tiny DS41 model on the GPU engine vs the CPU fp32 oracle (prefill + greedy decode)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(cfg_name="tiny", max_rows=8, max_ctx=512):
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.weights import init_weights
    from ds41rt_b200.models.reference import ReferenceModel
    from ds41rt_b200.models.ds41 import EngineWeights, DS41Engine
    cfg = getattr(ModelConfig, cfg_name)()
    w = init_weights(cfg, seed=0)
    # the engine stores matrices in bf16: give the oracle the same rounded values
    wr = {k: (v.bfloat16().float() if v.dim() == 2 and not k.endswith("_fn") else v) for k, v in w.items()}
    ref = ReferenceModel(cfg, wr)
    ew = EngineWeights.from_fp32(cfg, wr, 0, 1, torch.device("cuda"))
    eng = DS41Engine(cfg, ew, max_rows=max_rows, slots=2, max_ctx=max_ctx)
    return cfg, ref, eng


def _decisions_match(cfg, traces, debug, c0, n, positions):
    """Per row: did the engine take the same discrete decisions (routed experts, selected keys) as the oracle?"""
    ok = torch.ones(n, dtype=torch.bool)
    for rec in debug:
        l = rec["layer"]
        tr = traces[l]
        ids = rec["ids"].cpu()
        for r in range(n):
            t = c0 + r
            if sorted(ids[r].tolist()) != sorted(tr.experts[t].tolist()):
                ok[r] = False
            if tr.select is not None:
                want = tr.select[t].nonzero().flatten().tolist()
                got = rec["sel"][r, : int(rec["n_sel"][r])].cpu().tolist()
                if got != want:
                    ok[r] = False
    return ok


@pytest.mark.parametrize("chunk", [8, 64])
def test_prefill_logits_match_oracle(chunk):
    """Logits agree with the fp32 oracle wherever the discrete decisions (top-k experts, top-k keys) agree;
    bf16 activations may flip near-ties in those selections, which legitimately changes the result.
    chunk 64 exceeds the decode MoE row limit and the window ring slack: it runs the sorted expert path and the
    unfused hyper-connection kernels."""
    cfg, ref, eng = _setup(max_rows=chunk)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (128,), generator=g)
    with torch.no_grad():
        want, traces = ref.forward(prompt, return_trace=True)
    assert eng.cache.ensure(0, 200)
    got, same = [], []
    toks = prompt.tolist()
    for c0 in range(0, len(toks), chunk):
        part = toks[c0:c0 + chunk]
        eng.debug = []
        eng.set_rows(part, list(range(c0, c0 + len(part))), [0] * len(part))
        eng.forward_rows(len(part))
        got.append(eng.logits_rows(len(part)).cpu())
        same.append(_decisions_match(cfg, traces, eng.debug, c0, len(part), None))
    eng.debug = None
    torch.cuda.synchronize()
    eng.check_status()
    got, same = torch.cat(got, 0), torch.cat(same, 0)
    err = (got - want).abs().max(dim=1).values
    scale = float(want.abs().max())
    print("rows with identical decisions:", int(same.sum()), "of", len(same), "max err there:",
          float(err[same].max()), "max err elsewhere:", float(err[~same].max()) if (~same).any() else 0.0,
          "scale", scale)
    assert int(same.sum()) >= 0.6 * len(same)
    assert float(err[same].max()) < 0.05 * scale
    agree = (got.argmax(-1) == want.argmax(-1)).float().mean()
    assert float(agree) > 0.85


def test_greedy_decode_matches_oracle():
    cfg, ref, eng = _setup(max_rows=8)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (128,), generator=g)
    with torch.no_grad():
        want_tokens, want_logits = ref.generate_greedy(prompt, 32)
    nxt = eng.prefill(0, prompt.tolist())
    out = [nxt]
    pos = len(prompt)
    errs = []
    # teacher-force the oracle's tokens so every step's logits are comparable
    for i in range(31):
        eng.cache.ensure(0, pos + 2)
        eng.set_rows([int(want_tokens[i])], [pos], [0])
        eng.forward_rows(1)
        errs.append(float((eng.logits_rows(1).cpu()[0] - want_logits[i + 1]).abs().max()))
        out.append(int(eng.chosen[0].item()))
        pos += 1
    eng.check_status()
    scale = float(want_logits.abs().max())
    print("decode max logit err", max(errs), "scale", scale)
    errs_sorted = sorted(errs)
    assert errs_sorted[len(errs) // 2] < 0.03 * scale          # typical step is bf16-close
    assert errs_sorted[int(len(errs) * 0.75)] < 0.06 * scale   # outliers = flipped near-tie selections
    match = sum(int(a == int(b)) for a, b in zip(out, want_tokens.tolist()))
    assert match >= 26


def test_verify_rows_equal_single_steps():
    """A 5-row verification chunk must give the same tokens as five single-row steps (position-indexed caches)."""
    cfg, ref, eng = _setup(max_rows=8)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg.vocab, (77,), generator=g).tolist()
    nxt = eng.prefill(0, prompt)
    seq = [nxt]
    pos = len(prompt)
    for _ in range(5):
        eng.cache.ensure(0, pos + 2)
        eng.set_rows([seq[-1]], [pos], [0])
        eng.forward_rows(1)
        seq.append(int(eng.chosen[0].item()))
        pos += 1
    # replay the same 5 inputs as one chunk on slot 1 after an identical prefill
    nxt2 = eng.prefill(1, prompt)
    assert nxt2 == nxt
    eng.cache.ensure(1, len(prompt) + 8)
    eng.set_rows(seq[:5], list(range(len(prompt), len(prompt) + 5)), [1] * 5)
    eng.forward_rows(5)
    chunk = eng.chosen[:5].tolist()
    eng.check_status()
    assert chunk == seq[1:6]


@pytest.mark.parametrize("dtype,chunk", [("mxfp8", 8), ("mxfp8", 40), ("mxfp4", 8), ("mxfp4", 40), ("nvfp4", 8),
                                         ("nvfp4", 40)])
def test_block_scaled_experts_match_oracle(dtype, chunk):
    """Routed experts stored as FP8 E4M3 + 128x128 power-of-two block scales, run through the block-scaled
    tcgen05 path, vs the oracle evaluated on the dequantised weights (chunk 40: the sorted expert path)."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.weights import init_weights
    from ds41rt_b200.models.reference import ReferenceModel
    from ds41rt_b200.models.ds41 import EngineWeights, DS41Engine, dequantize_expert, dequantize_expert_fp4
    cfg = ModelConfig.tiny()
    w = init_weights(cfg, seed=0)
    wr = {k: (v.bfloat16().float() if v.dim() == 2 and not k.endswith("_fn") else v) for k, v in w.items()}
    ew = EngineWeights.from_fp32(cfg, wr, 0, 1, torch.device("cuda"), expert_dtype=dtype)
    if dtype == "mxfp4":
        dequantize_expert = dequantize_expert_fp4
    if dtype == "nvfp4":
        from ds41rt_b200.models.ds41 import dequantize_expert_nvfp4
    I = cfg.inter
    for l, lw in enumerate(ew.layers):
        for e in range(cfg.n_experts):
            if dtype == "nvfp4":
                w13 = dequantize_expert_nvfp4(lw.w13[e], lw.w13_sf[e], float(lw.w13_gs[e]))
                wr[f"layers.{l}.ffn.experts.{e}.w1.weight"] = w13[:I]
                wr[f"layers.{l}.ffn.experts.{e}.w3.weight"] = w13[I:]
                wr[f"layers.{l}.ffn.experts.{e}.w2.weight"] = dequantize_expert_nvfp4(lw.w2[e], lw.w2_sf[e],
                                                                                      float(lw.w2_gs[e]))
                continue
            w13 = dequantize_expert(lw.w13[e], lw.w13_sf[e])
            wr[f"layers.{l}.ffn.experts.{e}.w1.weight"] = w13[:I]
            wr[f"layers.{l}.ffn.experts.{e}.w3.weight"] = w13[I:]
            wr[f"layers.{l}.ffn.experts.{e}.w2.weight"] = dequantize_expert(lw.w2[e], lw.w2_sf[e])
    ref = ReferenceModel(cfg, wr)
    if dtype == "nvfp4":
        # W4A4: the oracle quantises the expert inputs the same way (fixed per-tensor scales, E4M3 scale per 16)
        from ds41rt_b200.models.ds41 import NVFP4_IN_SCALE_FC1, NVFP4_IN_SCALE_FC2
        from ds41rt_b200.ops import quant_ref as Q
        qdq = lambda gs: (lambda t: Q.dequant_nvfp4(*Q.quant_nvfp4(t.bfloat16().float(), gs)[:2], gs))
        ref.expert_act_qdq = (qdq(NVFP4_IN_SCALE_FC1), qdq(NVFP4_IN_SCALE_FC2))
    eng = DS41Engine(cfg, ew, max_rows=chunk, slots=1, max_ctx=256)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g)
    with torch.no_grad():
        want, traces = ref.forward(prompt, return_trace=True)
    eng.cache.ensure(0, 64)
    got, same = [], []
    toks = prompt.tolist()
    for c0 in range(0, len(toks), chunk):
        part = toks[c0:c0 + chunk]
        eng.debug = []
        eng.set_rows(part, list(range(c0, c0 + len(part))), [0] * len(part))
        eng.forward_rows(len(part))
        got.append(eng.logits_rows(len(part)).cpu())
        same.append(_decisions_match(cfg, traces, eng.debug, c0, len(part), None))
    eng.check_status()
    got, same = torch.cat(got, 0), torch.cat(same, 0)
    err = (got - want).abs().max(dim=1).values
    scale = float(want.abs().max())
    print("mx: same", int(same.sum()), "of", len(same), "max err", float(err[same].max()), "scale", scale)
    assert int(same.sum()) >= 0.6 * len(same)
    # fp8 activations (1x128 scales) add quantisation noise on top of bf16
    assert float(err[same].max()) < 0.08 * scale


def test_cuda_graph_decode_matches_eager():
    from ds41rt_b200.runtime.session import DecodeSession
    cfg, ref, eng = _setup(max_rows=8)
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, cfg.vocab, (50,), generator=g).tolist()
    sess = DecodeSession(eng, use_graphs=True)
    out_graph = sess.generate(prompt, 12, slot=0)
    sess2 = DecodeSession(eng, use_graphs=False)
    out_eager = sess2.generate(prompt, 12, slot=1)
    assert out_graph == out_eager
    # device feedback loop reproduces the host loop
    nxt = eng.prefill(0, prompt)
    eng.cache.ensure(0, len(prompt) + 16)
    eng.set_rows([nxt], [len(prompt)], [0])
    sess.run_device_loop(1, 5)
    torch.cuda.synchronize()
    assert int(eng.row_pos[0]) == len(prompt) + 5
    assert int(eng.in_tokens[0]) == out_graph[5]
    # NVTX ranges around every launch (DS41_NVTX=1) change nothing but the timeline a profiler sees
    eng.nvtx = True
    out_ranges = DecodeSession(eng, use_graphs=False).generate(prompt, 12, slot=1)
    eng.nvtx = False
    assert out_ranges == out_eager


def test_fp8_kv_cache_rows_and_logits():
    """FP8 cache rows are exactly the MX-FP8 (1x32, ceil-pow2 scale) image of the bf16 rows, and the model's logits
    move only by the quantisation noise."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.ops import quant_ref as Q
    cfg = ModelConfig.tiny()
    dev = torch.device("cuda")
    ew = EngineWeights.random(cfg, 0, 1, dev, seed=3)
    engines = {kv: DS41Engine(cfg, ew, max_rows=16, slots=1, max_ctx=256, kv_dtype=kv) for kv in ("bf16", "fp8")}
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(3, cfg.vocab, (48,), generator=g).tolist()
    logits = {}
    for kv, eng in engines.items():
        eng.cache.ensure(0, 128)
        for c0 in range(0, len(toks), 16):
            part = toks[c0:c0 + 16]
            eng.set_rows(part, list(range(c0, c0 + len(part))), [0] * len(part))
            eng.forward_rows(len(part))
        logits[kv] = eng.logits_rows(16).float().cpu()
        eng.check_status()
    D = cfg.head_dim
    # layer 0 sees identical inputs in both engines: its window rows must be the exact FP8 image
    ref_rows = engines["bf16"].cache.win[0][0]                      # [ring, D] bf16
    got = engines["fp8"].cache.win[0][0]                             # [ring, row_bytes] uint8
    q, e = Q.quant_mxfp8(ref_rows.float(), 32)
    live = [p % engines["bf16"].cache.ring for p in range(len(toks))]
    bad = (got[live, :D] != q.view(torch.uint8)[live]).sum().item()
    bad_e = (got[live, D:D + D // 32] != e.to(torch.uint8)[live]).sum().item()
    assert bad == 0 and bad_e == 0, (bad, bad_e, got[live[0], :8].tolist(), q.view(torch.uint8)[live[0], :8].tolist(),
                                     got[live[0], D:D + 4].tolist(), e[live[0], :4].tolist())
    src = next(iter(engines["bf16"].cache.comp))
    rows = len(toks) // cfg.source_layers[src]
    qc, ec = Q.quant_mxfp8(engines["bf16"].cache.comp[src].float(), 32)
    if src == 0:
        pages = engines["bf16"].cache.pages_of(0)
        pr = engines["bf16"].cache.page_rows[src]
        phys = [pages[i // pr] * pr + i % pr for i in range(rows)]
        assert torch.equal(engines["fp8"].cache.comp[src][phys, :D], qc.view(torch.uint8)[phys])
    scale = float(logits["bf16"].abs().max())
    # random weights amplify any perturbation and may flip a routed expert or a selected key in some row, so the
    # bound is on the typical row, not the worst one
    err = (logits["fp8"] - logits["bf16"]).abs().max(dim=1).values
    agree = float((logits["fp8"].argmax(-1) == logits["bf16"].argmax(-1)).float().mean())
    print("fp8 kv: median / max logit drift", float(err.median()), float(err.max()), "scale", scale, "agreement", agree)
    assert float(err.median()) < 0.1 * scale and agree >= 0.5


def test_candidate_blocks_restrict_later_index_layers():
    """Three index layers over one compressed source; the first is the candidate layer (top-2 blocks of 8 keys), so the
    two above it select their keys inside 16 candidates.  Rows whose discrete decisions agree with the oracle must have
    matching logits, and the restriction must actually bite (the oracle's selections differ from unrestricted ones)."""
    import dataclasses
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.reference import ReferenceModel
    from ds41rt_b200.models.weights import init_weights
    base = ModelConfig.tiny()
    cfg = dataclasses.replace(base, name="tiny-cand", n_layers=3, source_layers={0: 2}, compress_ratios=[2, 2, 2],
                              index_layers=(0, 1, 2), index_topk=8, candidate_layer=0, candidate_topk_blocks=2,
                              candidate_block=8,
                              dspark=dataclasses.replace(base.dspark, tap_layers=(0, 1)))
    cfg.validate()
    w = init_weights(cfg, seed=2)
    wr = {k: (v.bfloat16().float() if v.dim() == 2 and not k.endswith("_fn") else v) for k, v in w.items()}
    ref = ReferenceModel(cfg, wr)
    free = ReferenceModel(dataclasses.replace(cfg, candidate_layer=-1, candidate_topk_blocks=0), wr)
    eng = DS41Engine(cfg, EngineWeights.from_fp32(cfg, wr, 0, 1, torch.device("cuda")), max_rows=8, slots=1,
                     max_ctx=256)
    prompt = torch.randint(0, cfg.vocab, (96,), generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        want, traces = ref.forward(prompt, return_trace=True)
        _, free_traces = free.forward(prompt, return_trace=True)
    assert any(not torch.equal(a.select, b.select) for a, b in zip(traces[1:], free_traces[1:]))
    assert eng.cache.ensure(0, 128)
    got, same = [], []
    toks = prompt.tolist()
    for c0 in range(0, len(toks), 8):
        part = toks[c0:c0 + 8]
        eng.debug = []
        eng.set_rows(part, list(range(c0, c0 + len(part))), [0] * len(part))
        eng.forward_rows(len(part))
        got.append(eng.logits_rows(len(part)).cpu())
        same.append(_decisions_match(cfg, traces, eng.debug, c0, len(part), None))
    eng.debug = None
    torch.cuda.synchronize()
    eng.check_status()
    got, same = torch.cat(got, 0), torch.cat(same, 0)
    err = (got - want).abs().max(dim=1).values
    scale = float(want.abs().max())
    assert int(same.sum()) >= 0.5 * len(same), int(same.sum())
    assert float(err[same].max()) < 0.05 * scale, (float(err[same].max()), scale)


@pytest.mark.parametrize("deep", [False, True])
def test_ced_prefill_matches_full_prefill_and_oracle(deep):
    """Prompt passes with the decoder layers replayed for the tail only.  (a) A prompt that fits the replay span takes
    exactly the computations of the ordinary prefill: same logits bit for bit.  (b) A longer prompt follows the fp32
    oracle of the same scheme (complete compressed sources, decoder windows from the tail only)."""
    import dataclasses
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.reference import ReferenceModel
    from ds41rt_b200.models.weights import init_weights
    cfg = dataclasses.replace(ModelConfig.tiny(), ced_boundary=1, ced_replay=24)
    if deep:      # two decoder layers above the boundary, all three layers read the source of layer 0
        cfg = dataclasses.replace(cfg, name="tiny-ced3", n_layers=3, source_layers={0: 2}, compress_ratios=[2, 2, 2],
                                  index_layers=(0, 1, 2), index_topk=16,
                                  dspark=dataclasses.replace(cfg.dspark, tap_layers=(1, 2)))
        cfg.validate()
    assert cfg.ced_on
    w = init_weights(cfg, seed=0)
    wr = {k: (v.bfloat16().float() if v.dim() == 2 and not k.endswith("_fn") else v) for k, v in w.items()}
    ref = ReferenceModel(cfg, wr)
    dev = torch.device("cuda")
    eng = DS41Engine(cfg, EngineWeights.from_fp32(cfg, wr, 0, 1, dev), max_rows=8, slots=2, max_ctx=512)
    g = torch.Generator().manual_seed(5)
    short = torch.randint(0, cfg.vocab, (21,), generator=g).tolist()
    t_full = eng.prefill(0, short)
    l_full = eng.logits_rows(eng.last_head_row + 1)[eng.last_head_row].clone()
    t_ced = eng.prefill_ced(1, short)
    l_ced = eng.logits_rows(eng.last_head_row + 1)[eng.last_head_row].clone()
    eng.check_status("ced short")
    assert t_full == t_ced and torch.equal(l_full, l_ced)
    eng.cache.release(0)
    eng.cache.release(1)
    # (b) 100 tokens, replay 24: chunks of 8 cross the replay start (76) inside a chunk
    prompt = torch.randint(0, cfg.vocab, (100,), generator=g)
    with torch.no_grad():
        want = ref.forward_ced(prompt, 1, replay=24)[-4:]
        full = ref.forward(prompt)[-4:]
    eng.prefill_ced(0, prompt.tolist())
    got = eng.logits_rows(eng.last_head_row + 1).float().cpu()       # the last replay slice: positions 92..99
    eng.check_status("ced long")
    assert got.shape[0] == 8
    got = got[-4:]
    scale = float(want.abs().max())
    # single rows can flip a near-tied expert or key selection under bf16: judge the typical row
    err_ced = (got - want).abs().max(dim=1).values.median()
    err_full = (got - full).abs().max(dim=1).values.median()
    assert float((want - full).abs().max()) > 0.02 * scale          # the scheme differs from the full pass here
    assert float(err_ced) < 0.1 * scale and float(err_ced) < 0.5 * float(err_full), (err_ced, err_full, scale)
    # decoding continues from the replayed windows
    nxt = int(eng.chosen[eng.last_head_row].item())
    eng.set_rows([nxt], [100], [0])
    eng.forward_rows(1)
    torch.cuda.synchronize()
    eng.check_status("ced decode")


def test_long_chunks_leave_the_same_state_as_short_ones():
    """A 43-token prompt run in passes of 16 rows (two even rows of one pass share a pair-carry place) and in passes of
    8 rows: the ratio-2 pair carry and the following decode steps are bit-identical."""
    cfg, ref, eng = _setup(max_rows=16)
    prompt = torch.randint(3, cfg.vocab - 8, (43,), generator=torch.Generator().manual_seed(21)).tolist()
    outs = []
    for slot, chunk in ((0, 16), (1, 8)):
        tok = eng.prefill(slot, prompt, chunk=chunk)
        carry = {k: v[slot].clone() for k, v in eng.cache.pending.items()}
        steps = []
        assert eng.cache.ensure(slot, len(prompt) + 8)
        for i in range(4):
            eng.set_rows([tok], [len(prompt) + i], [slot])
            eng.forward_rows(1)
            steps.append(eng.logits[:1].clone())
            tok = int(eng.chosen[0].item())
        outs.append((carry, steps))
    eng.check_status()
    place = (42 >> 1) & 3
    for k in outs[0][0]:
        assert torch.equal(outs[0][0][k][place], outs[1][0][k][place]), k
    for a, b in zip(outs[0][1], outs[1][1]):
        assert torch.equal(a, b)


def test_fp4_compressed_rows_and_logits():
    """kv_dtype "fp4": window rings FP8, compressed rows FP4 (e2m1 + E4M3 scale per 16).  The compressed rows of the
    first source layer are the exact FP4 image of the bf16 engine's rows (same inputs there), and the logits move only
    by quantisation noise."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.ops import quant_ref as Q
    cfg = ModelConfig.tiny()
    dev = torch.device("cuda")
    ew = EngineWeights.random(cfg, 0, 1, dev, seed=3)
    engines = {kv: DS41Engine(cfg, ew, max_rows=16, slots=1, max_ctx=256, kv_dtype=kv) for kv in ("bf16", "fp4")}
    toks = torch.randint(3, cfg.vocab, (48,), generator=torch.Generator().manual_seed(11)).tolist()
    logits = {}
    for kv, eng in engines.items():
        eng.cache.ensure(0, 128)
        for c0 in range(0, len(toks), 16):
            part = toks[c0:c0 + 16]
            eng.set_rows(part, list(range(c0, c0 + len(part))), [0] * len(part))
            eng.forward_rows(len(part))
        logits[kv] = eng.logits_rows(16).float().cpu()
        eng.check_status()
    D = cfg.head_dim
    assert D // 2 + D // 16 <= engines["fp4"].cache.comp_row_bytes < engines["fp4"].cache.row_bytes
    src = 0                                                    # layer 0: identical inputs in both engines
    assert src in engines["bf16"].cache.comp
    n = len(toks) // cfg.source_layers[src]
    pr = engines["bf16"].cache.page_rows[src]
    rows = [engines["bf16"].cache.pages_of(0)[i // pr] * pr + i % pr for i in range(n)]
    ref = engines["bf16"].cache.comp[src][rows].float().cpu()
    rows4 = [engines["fp4"].cache.pages_of(0)[i // pr] * pr + i % pr for i in range(n)]
    got = engines["fp4"].cache.comp[src][rows4].cpu()
    packed, bs = Q.quant_kv_fp4_e4m3_16(ref)
    assert torch.equal(got[:, :D // 2], packed.view(torch.uint8).reshape(n, D // 2))
    assert torch.equal(got[:, D // 2:D // 2 + D // 16], bs.view(torch.uint8).reshape(n, D // 16))
    # the index keys of that layer are FP4 rows too (E2M1 pairs + one UE8M0 scale per 32 values): the exact image of the
    # bf16 engine's keys
    ID = cfg.index_dim
    c4 = engines["fp4"].cache
    assert c4.index_dtype == "fp4" and c4.idx_row_bytes >= ID // 2 + ID // 32 and engines["bf16"].cache.idx_row_bytes == 0
    ikeys = engines["bf16"].cache.idx[src][rows].float().cpu()
    p4, e4 = Q.quant_mxfp4(ikeys, 32)
    got_i = c4.idx[src][rows4].cpu()
    assert torch.equal(got_i[:, :ID // 2], p4.view(torch.uint8).reshape(n, ID // 2))
    assert torch.equal(got_i[:, ID // 2:ID // 2 + ID // 32], e4.to(torch.uint8).reshape(n, ID // 32))
    a, b = logits["bf16"], logits["fp4"]
    scale = float(a.abs().max())
    drift = (a - b).abs().max(dim=1).values
    assert float(drift.median()) < 0.15 * scale, (float(drift.median()), scale)
    assert float((a.argmax(-1) == b.argmax(-1)).float().mean()) >= 0.5


@pytest.mark.parametrize("cfg_name,n,ced,seed", [("tiny", 200, False, 11), ("small", 300, False, 11),
                                                 ("tiny", 330, True, 12)])
def test_row_sharded_long_pass_matches_replicated(cfg_name, n, ced, seed):
    """long_pass="sp" forced on one GPU (the one rank owns every row): own-row hyper-connections, q_a / kv projection in
    the gathered orientation, q_b / attention / wo over all heads with the unsharded weights, router and shared expert
    on the own rows.  A prompt that is no multiple of 128 rows runs padded.  Caches, last-row logits and the decode
    steps that follow must agree with the replicated long pass."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.weights import init_weights
    cfg = getattr(ModelConfig, cfg_name)()
    if ced and not cfg.ced_on:
        import dataclasses
        cfg = dataclasses.replace(cfg, ced_boundary=1, ced_replay=cfg.window)
    w = init_weights(cfg, seed=0)
    ew = EngineWeights.from_fp32(cfg, w, 0, 1, torch.device("cuda"))
    # The two layouts sum in different orders, so bf16 roundings of the streams differ by an ulp here and there; a prompt
    # whose LAST row sits on a router or index near-tie then takes another expert in one layout and every compared logit
    # moves (seen for about one prompt in six with either form of the mixes projection).  The seeds avoid such prompts.
    g = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, cfg.vocab, (n,), generator=g).tolist()
    out = {}
    for mode in ("replicated", "sp"):
        eng = DS41Engine(cfg, ew, max_rows=384, slots=1, max_ctx=512, long_pass=mode)
        run = eng.prefill_ced if ced else eng.prefill
        nxt = run(0, prompt)
        logits = eng.logits_rows(1)[0].float().cpu()
        win, comp = eng.cache.win.float().cpu(), {s: t.float().cpu() for s, t in eng.cache.comp.items()}
        toks = [nxt]
        for i in range(4):
            eng.set_rows([toks[-1]], [n + i], [0])
            eng.forward_rows(1)
            toks.append(int(eng.chosen[0].item()))
        torch.cuda.synchronize()
        eng.check_status(mode)
        out[mode] = (logits, toks, win, comp)
        assert (eng._sp is not None) == (mode == "sp")
    la, ta, wa, ca = out["replicated"]
    lb, tb, wb, cb = out["sp"]
    scale = float(la.abs().max())
    assert float((la - lb).abs().max()) < 0.03 * scale
    assert int(la.argmax()) == int(lb.argmax())
    # a row whose router or index selection sat on a near-tie may take the other branch under the different summation
    # order of the two layouts; all but a few rows of every cache must agree closely
    def close(a, b):
        bad = (a - b).abs().amax(-1) > 0.05 * max(1.0, float(a.abs().max()))
        return float(bad.float().mean()) < 0.03
    assert close(wa, wb)
    for s_ in ca:
        assert close(ca[s_], cb[s_])
    assert ta[:2] == tb[:2]


def test_flash_width_layers_match_oracle():
    """The release model's widths - hidden 5120, 64 heads x 512, 8 output groups, 384 experts top-6 stored as FP8 with
    block scales, a 32 x 128 indexer over ratio-2 compressed rows - on a 2-layer stack with a shortened expert width
    and vocabulary (so the fp32 oracle fits in host memory): 8-row passes against the oracle on the dequantised
    weights."""
    import dataclasses
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.weights import init_weights
    from ds41rt_b200.models.reference import ReferenceModel
    from ds41rt_b200.models.ds41 import EngineWeights, DS41Engine, dequantize_expert
    cfg = dataclasses.replace(ModelConfig.flash(2), name="flash-width-L2", vocab=8192, inter=128,
                              source_layers={1: 2}, compress_ratios=[0, 2], index_layers=(1,), candidate_layer=-1,
                              candidate_topk_blocks=0, dspark=None, engram=None, image_token=8191,
                              think_end_token=8190)
    cfg.validate()
    assert cfg.hidden == 5120 and cfg.n_experts == 384 and cfg.n_heads == 64 and cfg.head_dim == 512
    w = init_weights(cfg, seed=0)
    wr = {k: (v.bfloat16().float() if v.dim() == 2 and not k.endswith("_fn") else v) for k, v in w.items()}
    del w
    ew = EngineWeights.from_fp32(cfg, wr, 0, 1, torch.device("cuda"), expert_dtype="mxfp8")
    I = cfg.inter
    for l, lw in enumerate(ew.layers):
        for e in range(cfg.n_experts):
            w13 = dequantize_expert(lw.w13[e], lw.w13_sf[e])
            wr[f"layers.{l}.ffn.experts.{e}.w1.weight"] = w13[:I]
            wr[f"layers.{l}.ffn.experts.{e}.w3.weight"] = w13[I:]
            wr[f"layers.{l}.ffn.experts.{e}.w2.weight"] = dequantize_expert(lw.w2[e], lw.w2_sf[e])
    ref = ReferenceModel(cfg, wr)
    eng = DS41Engine(cfg, ew, max_rows=8, slots=1, max_ctx=256)
    prompt = torch.randint(0, cfg.vocab, (48,), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want, traces = ref.forward(prompt, return_trace=True)
    eng.cache.ensure(0, 64)
    got, same = [], []
    toks = prompt.tolist()
    for c0 in range(0, len(toks), 8):
        part = toks[c0:c0 + 8]
        eng.debug = []
        eng.set_rows(part, list(range(c0, c0 + len(part))), [0] * len(part))
        eng.forward_rows(len(part))
        got.append(eng.logits_rows(len(part)).cpu())
        same.append(_decisions_match(cfg, traces, eng.debug, c0, len(part), None))
    eng.check_status()
    got, same = torch.cat(got, 0), torch.cat(same, 0)
    err = (got - want).abs().max(dim=1).values
    scale = float(want.abs().max())
    print("flash width: same", int(same.sum()), "of", len(same), "max err", float(err[same].max()), "scale", scale)
    assert int(same.sum()) >= 0.6 * len(same)
    assert float(err[same].max()) < 0.08 * scale
