"""Vision tower on the GPU kernels vs the PyTorch fp32 statement of the same network."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("grid,layers,tile", [((6, 9), 2, 1024), ((12, 15), 3, 64)])
def test_vision_tower_matches_reference(grid, layers, tile):
    from ds41rt_b200.config import VisionConfig
    from ds41rt_b200.models.vision import VisionTower, init_vision_weights, vision_reference
    from ds41rt_b200.ops import lib
    v = VisionConfig(layers=layers, hidden=256, heads=4, intermediate=384)
    hidden = 512
    w = init_vision_weights(v, hidden, layers, seed=1, std=0.05)
    wr = {k: t.bfloat16().float() for k, t in w.items()}
    gh, gw = grid
    g = torch.Generator().manual_seed(2)
    patches = torch.randn(gh * gw, 3 * v.patch * v.patch, generator=g).bfloat16().float()
    want = vision_reference(v, wr, patches, grid, layers)
    dev = torch.device("cuda")
    tower = VisionTower(v, w, hidden, layers, dev, max_patches=256, query_tile=tile)
    got = tower.encode(patches, grid).float().cpu()
    torch.cuda.synchronize()
    lib.raise_on_status(tower.status, "vision gemm")
    assert got.shape == want.shape == (gh * gw // 9, hidden)
    err = float((got - want).abs().max() / want.abs().max())
    assert err < 4e-2, err
    # rows land in every stream copy of the embedding buffer
    streams = torch.zeros(20, 4, hidden, dtype=torch.bfloat16, device=dev)
    ids = torch.tensor([3, 7, -1, 11][: got.shape[0]] + [-1] * max(0, got.shape[0] - 4), dtype=torch.int32, device=dev)
    tower.scatter(tower.out[: got.shape[0]], ids, streams)
    torch.cuda.synchronize()
    assert torch.equal(streams[3, 2].cpu(), tower.out[0].cpu()) and float(streams[4].abs().sum()) == 0.0


def test_image_rows_replace_placeholder_embeddings():
    """Placeholder rows of a pass get the tower's rows: the logits of those positions change, other rows do not when
    the image rows equal the placeholder's own embedding."""
    from ds41rt_b200.config import ModelConfig
    from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights
    cfg = ModelConfig.tiny()
    dev = torch.device("cuda")
    eng = DS41Engine(cfg, EngineWeights.random(cfg, 0, 1, dev, seed=0), max_rows=8, slots=1, max_ctx=128)
    eng.cache.ensure(0, 64)
    toks = [5, 9, 9, 9, 7, 8]
    def run(patch):
        eng.image_patch = patch
        eng.set_rows(toks, list(range(len(toks))), [0] * len(toks))
        eng.forward_rows(len(toks))
        eng.image_patch = None
        return eng.logits_rows(len(toks)).clone()
    base = run(None)
    same_rows = eng.w.embed[9].view(1, -1).repeat(3, 1).contiguous()
    ids = torch.tensor([1, 2, 3], dtype=torch.int32, device=dev)
    assert torch.equal(run((same_rows, ids)), base)
    other = (torch.randn(3, cfg.hidden, device=dev) * 0.02).bfloat16()
    changed = run((other, ids))
    assert not torch.equal(changed[1:4], base[1:4]) and torch.equal(changed[0], base[0])
    eng.check_status()
