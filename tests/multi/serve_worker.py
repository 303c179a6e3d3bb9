"""Worker: the serving backend on rank 0 with the other ranks mirroring its engine calls (tensor/expert parallel)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from ds41rt_b200.config import ModelConfig  # noqa: E402
from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights  # noqa: E402
from ds41rt_b200.parallel.fabric import Fabric  # noqa: E402
from ds41rt_b200.serving.distributed import LeaderEngine, follower_loop, make_control_group  # noqa: E402
from ds41rt_b200.serving.engine import GenRequest, NativeBackend  # noqa: E402
from ds41rt_b200.serving.protocol import Sampling  # noqa: E402


def collect(req, timeout=120):
    toks, finish = [], None
    while finish is None:
        ev = req.events.get(timeout=timeout)
        if ev.kind == "tokens":
            toks += ev.tokens
        elif ev.kind == "finish":
            finish = ev.reason
        elif ev.kind == "error":
            raise RuntimeError(ev.message)
    return toks, finish


def main():
    fabric = Fabric.create()
    ctl = make_control_group(fabric)
    cfg = ModelConfig.tiny()
    ew = EngineWeights.random(cfg, fabric.rank, fabric.world, fabric.device, seed=0)
    eng = DS41Engine(cfg, ew, fabric, max_rows=8, slots=4, max_ctx=256)
    if fabric.rank != 0:
        n = follower_loop(eng, ctl)
        print(f"follower {fabric.rank}: {n} passes")
    else:
        lead = LeaderEngine(eng, ctl)
        backend = NativeBackend(lead, eos=1, concurrency=4)
        g = torch.Generator().manual_seed(3)
        prompt = torch.randint(3, cfg.vocab, (20,), generator=g).tolist()
        greedy = [GenRequest(prompt_ids=prompt, max_tokens=12, sampling=Sampling(temperature=0.0)) for _ in range(2)]
        sampled = [GenRequest(prompt_ids=prompt, max_tokens=12,
                              sampling=Sampling(temperature=0.9, top_p=0.9, top_k=40, seed=5)) for _ in range(2)]
        for r in greedy + sampled:           # all four run concurrently in one batch
            backend.submit(r)
        out = [collect(r) for r in greedy + sampled]
        backend.close()
        lead.stop_followers()
        assert backend.healthy, backend.error
        assert out[0] == out[1] and out[2] == out[3], out
        assert all(len(t) >= 1 and f in ("stop", "length") for t, f in out), out
        assert backend.totals["gpu_sampled_rows"] > 0
        print("SERVE_WORKER_OK", out[0][0][:6], out[2][0][:6])
    fabric.barrier()


if __name__ == "__main__":
    main()
