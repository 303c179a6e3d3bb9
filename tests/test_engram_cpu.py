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
