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
