"""Engram host I/O: exact-size mapping, gather order, bounded slots, cancellation, prefetch advice."""
import numpy as np
import pytest

from ds41rt_b200.runtime.engram_io import EngramGather, EngramTable


@pytest.fixture()
def table(tmp_path):
    rng = np.random.default_rng(0)
    rows = rng.integers(0, 256, size=(5000, 264), dtype=np.uint8)
    path = tmp_path / "engram.bin"
    rows.tofile(path)
    t = EngramTable(str(path), 5000, 264)
    yield t, rows, path
    t.close()


def test_size_must_match(table, tmp_path):
    _, _, path = table
    with pytest.raises(OSError):
        EngramTable(str(path), 4999, 264)
    with pytest.raises(OSError):
        EngramTable(str(tmp_path / "missing.bin"), 10, 264)


def test_gather_returns_rows_in_request_order(table):
    t, rows, _ = table
    g = EngramGather(t, slots=2, max_rows=96)
    ids = [4999, 0, 17, 17, 2500] + list(range(100, 150))
    assert t.prefetch(ids) > 0
    tk = g.submit(ids)
    got = g.wait(tk)
    assert np.array_equal(got, rows[ids])
    assert g.release(tk)
    with pytest.raises(IndexError):
        g.submit([5000])
    with pytest.raises(IndexError):
        g.submit(list(range(97)))
    g.close()


def test_pool_is_bounded_and_cancel_frees_a_slot(table):
    t, rows, _ = table
    g = EngramGather(t, slots=2, max_rows=64)
    a = g.submit(list(range(64)))
    b = g.submit(list(range(64, 128)))
    assert a is not None and b is not None and g.submit([1]) is None        # every slot in use
    assert np.array_equal(g.wait(a), rows[:64])
    g.cancel(b)                                   # finished or not, the slot can be handed back afterwards
    while g.poll(b) is False:
        pass
    assert g.release(a) and g.release(b)
    c = g.submit([7, 8, 9])
    assert np.array_equal(g.wait(c), rows[[7, 8, 9]])
    st = g.stats()
    assert st["requests"] == 3 and st["refused"] == 1
    g.close()


# ------------------------------------------------------------------------------------------- request pipeline
def test_compressed_ids_merge_case_accents_and_whitespace():
    from ds41rt_b200.runtime.engram import compressed_token_ids
    vocab = ["[UNK]", " The", "THE", "thé", " ", "", "\t", "the  cat", "The\ncat"]
    ids = compressed_token_ids([v.encode() for v in vocab] + [b"\xff\xfe", b"\xff\xfe", b"\xe2\x82"])
    assert ids[1] == ids[2] == ids[3]
    assert ids[4] != ids[5] and ids[4] == ids[6]
    assert ids[7] == ids[8]
    assert ids[9] == ids[10] != ids[11]                 # byte fragments are keyed by their raw bytes
    assert ids[0] == 0 and int(ids.max()) == len(set(ids.tolist())) - 1


class _FakeEngine:
    def __init__(self, layers):
        self.engram = {l: None for l in layers}
        self.got = {}

    def set_engram_rows(self, layer, rows, mask):
        self.got[layer] = (np.array(rows), np.array(mask))


def test_pipeline_hashes_gathers_and_commits_only_accepted(table):
    from ds41rt_b200.runtime.core import EngramHistory
    from ds41rt_b200.runtime.engram import EngramPipeline
    t, rows, _ = table
    pipe = EngramPipeline([1], [t], pad_id=2, max_rows=16, fold=True)
    eng = _FakeEngine([1])
    toks = [11, 12, 13, 14, 15]
    p = pipe.begin(toks, [0] * 5)
    want_ids = EngramHistory(2).prepare(toks)[:, 0, :].reshape(-1) % np.uint64(5000)
    assert np.array_equal(p.ids[0], want_ids)
    pipe.apply(p, eng)
    got, mask = eng.got[1]
    assert np.array_equal(got, rows[want_ids.astype(np.int64)]) and mask.tolist() == [1] * 5
    pipe.commit(p, {0: 2})                              # a speculative pass of which two rows were accepted
    assert pipe.history(0).position == 2
    # the next pass hashes against [11, 12] only
    h = EngramHistory(2)
    h.commit([11, 12], 2)
    p2 = pipe.begin([13, 99], [0, 0])
    assert np.array_equal(p2.ids[0], h.prepare([13, 99])[:, 0, :].reshape(-1) % np.uint64(5000))
    pipe.cancel(p2)
    # two requests in one pass keep separate histories; image rows are masked and break the lookback
    p3 = pipe.begin([13, 7, 14], [0, 1, 0], is_image=[False, False, True])
    assert p3.text_mask.tolist() == [1, 1, 0] and p3.tokens[2] == -1
    pipe.apply(p3, eng)
    pipe.commit(p3)
    assert pipe.history(0).position == 4 and pipe.history(1).position == 1
    snap = pipe.fork(0)
    pipe.release(0)
    assert pipe.history(0).position == 0
    pipe.adopt(0, snap)
    assert pipe.history(0).position == 4
    assert pipe.stats()["gather"][0]["requests"] >= 3
    for g in pipe.gathers:
        g.close()


def test_row_delivery_bench_runs_every_route_and_eviction_is_scoped_to_the_file(table, capsys):
    t, rows, path = table
    warm = t.bench(tokens=8, mode="mmap", iters=2)
    assert warm["records_per_pass"] <= 8 * 24 and warm["mean_us"] > 0 and t.resident() > 0
    for mode in ("willneed", "pread", "pread-mt"):
        out = t.bench(tokens=8, mode=mode, iters=2, threads=3, cold=(mode == "pread"))
        assert out["mode"] == mode and out["min_us"] <= out["mean_us"] <= out["max_us"]
    t.evict()                                        # advice only: the file system may keep some pages
    assert 0.0 <= t.resident() <= 1.0
    g = EngramGather(t, slots=1, max_rows=8)         # the mapping still reads correctly afterwards
    ticket = g.submit([1, 4998])
    assert np.array_equal(g.wait(ticket), rows[[1, 4998]])
    g.release(ticket)
    g.close()
    with pytest.raises(OSError):
        t.bench(tokens=0)
    from ds41rt_b200.runtime.engram_io import main
    assert main([str(path), "--rows", "5000", "--tokens", "4", "--iters", "2", "--cache", "cold", "--mode", "pread"]) == 0
    assert '"cache": "cold"' in capsys.readouterr().out
