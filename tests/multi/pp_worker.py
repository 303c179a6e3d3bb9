"""Two-stage pipeline on 2 GPUs: rank 0 runs the lower layers, rank 1 the upper layers and the head; rank 1 also runs the
undivided engine and checks that the pipeline's logits and greedy tokens are bit-identical to it."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from ds41rt_b200.config import ModelConfig  # noqa: E402
from ds41rt_b200.models.ds41 import DS41Engine, EngineWeights  # noqa: E402
from ds41rt_b200.models.weights import init_weights  # noqa: E402
from ds41rt_b200.parallel.fabric import Fabric  # noqa: E402
from ds41rt_b200.parallel.pp import make_stage  # noqa: E402


def main():
    fabric = Fabric.create()
    assert fabric.world == 2
    cfg = ModelConfig.tiny()
    w = init_weights(cfg, seed=4)
    dev = fabric.device
    chunk, B = 16, 1
    st = make_stage(fabric, cfg, lambda rng: EngineWeights.from_fp32(cfg, w, 0, 1, dev, layer_range=rng), B, chunk,
                    slots=2, max_ctx=256)
    eng = st.e
    assert eng.cache.ensure(0, 96)
    full = None
    if fabric.rank == 1:
        full = DS41Engine(cfg, EngineWeights.from_fp32(cfg, w, 0, 1, dev), Fabric.single(dev), max_rows=chunk, slots=2,
                          max_ctx=256)
        assert full.cache.ensure(0, 96)
    prompt = torch.randint(3, cfg.vocab - 8, (52,), generator=torch.Generator().manual_seed(8)).tolist()
    for c0 in range(0, len(prompt), chunk):
        part = prompt[c0:c0 + chunk]
        pos, last = list(range(c0, c0 + len(part))), c0 + chunk >= len(prompt)
        eng.set_rows(part, pos, [0] * len(part))
        if fabric.rank == 0:
            st.run_lower(len(part))
        else:
            st.run_upper(len(part), head=last)
            full.set_rows(part, pos, [0] * len(part))
            full.forward_rows(len(part), head=last)
    n_steps = 6
    if fabric.rank == 1:
        torch.cuda.synchronize()
        r = full.last_head_row
        assert torch.equal(full.logits[r], eng.logits[r]), "prompt logits differ"
        st.give_tokens(1, row0=r)
        tok = int(full.chosen[r].item())
    for i in range(n_steps):
        p = len(prompt) + i
        if fabric.rank == 0:
            eng.set_rows(None, [p], [0])
            st.take_tokens(1)
            st.run_lower(1)
        else:
            eng.set_rows([0], [p], [0])
            st.run_upper(1)
            full.set_rows([tok], [p], [0])
            full.forward_rows(1)
            torch.cuda.synchronize()
            assert torch.equal(full.logits[0], eng.logits[0]), f"decode step {i} differs"
            tok = int(full.chosen[0].item())
            assert int(eng.chosen[0].item()) == tok
            st.give_tokens(1)
    if fabric.rank == 0:
        st.take_tokens(1)          # the token of the last step was published but not used: keep the counters level
    torch.cuda.synchronize()
    eng.check_status("pipeline stage")
    fabric.barrier()
    two_lanes(fabric, cfg, st, full, chunk)
    torch.cuda.synchronize()
    eng.check_status("two lanes")
    fabric.barrier()
    if fabric.rank == 1:
        print("PP_WORKER_OK", flush=True)


def two_lanes(fabric, cfg, st, full, chunk):
    """Two requests decode through the two stages in alternation: while the upper stage works on lane A's step the
    lower stage already runs lane B's (two handoff slots, tokens fed back on the device).  Every step of both lanes is
    compared with the undivided engine; the lanes' device time is printed next to one lane's."""
    import time
    eng, rank = st.e, fabric.rank
    g = torch.Generator().manual_seed(31)
    prompts = [torch.randint(3, cfg.vocab - 8, (20 + 9 * i,), generator=g).tolist() for i in range(2)]
    slots = [0, 1]
    for e in ([eng] if full is None else [eng, full]):
        for s in slots:
            e.cache.release(s)
            assert e.cache.ensure(s, 96)
    toks = [0, 0]
    for lane in range(2):
        pr = prompts[lane]
        for c0 in range(0, len(pr), chunk):
            part = pr[c0:c0 + chunk]
            pos, last = list(range(c0, c0 + len(part))), c0 + chunk >= len(pr)
            eng.set_rows(part, pos, [slots[lane]] * len(part))
            if rank == 0:
                st.run_lower(len(part))
            else:
                st.run_upper(len(part), head=last)
                full.set_rows(part, pos, [slots[lane]] * len(part))
                full.forward_rows(len(part), head=last)
        if rank == 1:
            torch.cuda.synchronize()
            r = full.last_head_row
            assert torch.equal(full.logits[r], eng.logits[r])
            toks[lane] = int(full.chosen[r].item())
            st.give_tokens(1, row0=r)
        else:
            # the lower stage keeps each lane's first token aside until that lane's first decode step
            st.take_tokens(1)
            toks[lane] = eng.in_tokens[0:1].clone()
    steps = 12
    t0 = time.perf_counter()
    for i in range(steps):
        for lane in range(2):
            p = len(prompts[lane]) + i
            if rank == 0:
                eng.set_rows(None, [p], [slots[lane]])
                if i == 0:
                    eng.in_tokens[0:1].copy_(toks[lane])
                else:
                    st.take_tokens(1)
                st.run_lower(1)
            else:
                eng.set_rows([0], [p], [slots[lane]])
                st.run_upper(1)
                st.give_tokens(1)
                full.set_rows([toks[lane]], [p], [slots[lane]])
                full.forward_rows(1)
                torch.cuda.synchronize()
                assert torch.equal(full.logits[0], eng.logits[0]), (lane, i)
                toks[lane] = int(full.chosen[0].item())
    if rank == 0:
        # the tokens of the last step were published but never taken: drain them so the counters end level
        for lane in range(2):
            st.take_tokens(1)
    torch.cuda.synchronize()
    if rank == 1:
        print(f"two lanes: {2 * steps} tokens in {1e3 * (time.perf_counter() - t0):.1f} ms wall (checked step by step)",
              flush=True)


if __name__ == "__main__":
    main()
