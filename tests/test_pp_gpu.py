"""Two-stage pipeline: both stages on one GPU (the handoff kernels read the other stage's buffer through a plain device
pointer, exactly as they read a peer's) against the undivided engine: bit-identical logits and tokens."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunk", [8, 24])
def test_two_stage_pipeline_matches_the_undivided_engine(chunk):
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    from ds41rt_b200.models.weights import init_weights
    from ds41rt_b200.parallel.pp import PipelineStage, buffer_bytes
    cfg = ModelConfig.tiny()
    w = init_weights(cfg, seed=4)
    dev = torch.device("cuda", 0)
    kw = dict(max_rows=chunk, slots=1, max_ctx=256)
    full = DS41Engine(cfg, EngineWeights.from_fp32(cfg, w, 0, 1, dev), **kw)
    B = 1
    lower = DS41Engine(cfg, EngineWeights.from_fp32(cfg, w, 0, 1, dev, layer_range=(0, B)), **kw)
    upper = DS41Engine(cfg, EngineWeights.from_fp32(cfg, w, 0, 1, dev, layer_range=(B, cfg.n_layers)), **kw)
    assert lower.w.nbytes() + upper.w.nbytes() < 1.6 * full.w.nbytes()      # embedding / head are held twice, layers once
    nb = buffer_bytes(chunk, cfg.hidden, cfg.hc_mult)
    buf0 = torch.zeros(nb, dtype=torch.uint8, device=dev)
    buf1 = torch.zeros(nb, dtype=torch.uint8, device=dev)
    s0 = PipelineStage(lower, 0, B, buf0, buf1.data_ptr())
    s1 = PipelineStage(upper, 1, B, buf1, buf0.data_ptr())
    prompt = torch.randint(3, cfg.vocab - 8, (52,), generator=torch.Generator().manual_seed(8)).tolist()
    for e in (full, lower, upper):
        assert e.cache.ensure(0, 80)
    # chunked prompt
    for c0 in range(0, len(prompt), chunk):
        part = prompt[c0:c0 + chunk]
        pos, last = list(range(c0, c0 + len(part))), c0 + chunk >= len(prompt)
        full.set_rows(part, pos, [0] * len(part))
        full.forward_rows(len(part), head=last)
        lower.set_rows(part, pos, [0] * len(part))
        s0.run_lower(len(part))
        upper.set_rows(part, pos, [0] * len(part))
        s1.run_upper(len(part), head=last)
    torch.cuda.synchronize()
    r = full.last_head_row
    assert upper.last_head_row == r
    assert torch.equal(full.logits[r], upper.logits[r])
    # greedy decode: the token travels back to the lower stage on the device
    tok = int(full.chosen[r].item())
    s1.give_tokens(1, row0=r)                   # the prompt's last row holds the next token
    for i in range(4):
        p = len(prompt) + i
        full.set_rows([tok], [p], [0])
        full.forward_rows(1)
        lower.set_rows(None, [p], [0])          # the token id arrives through the pipeline
        s0.take_tokens(1)
        s0.run_lower(1)
        upper.set_rows([0], [p], [0])
        s1.run_upper(1)
        torch.cuda.synchronize()
        assert torch.equal(full.logits[0], upper.logits[0]), i
        tok = int(full.chosen[0].item())
        assert int(upper.chosen[0].item()) == tok
        s1.give_tokens(1)
    for e in (full, lower, upper):
        e.check_status("pipeline test")
