"""Packed candidate files: save a bound set, bind it back whole and as row shards, and check that the scores are
bit-identical to the set it was saved from (the file keeps the packed codes and scales, nothing is re-quantised)."""
import os

import numpy as np
import pytest

from helpers import make_rows, pack

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    from manta_b200 import native

    r = native.Runtime(0)
    yield r
    r.close()


@pytest.mark.parametrize("layout,cols", [("q8", 100), ("q8", 768), ("q4", 256), ("f16", 33)])
def test_save_load_round_trip(rt, tmp_path, layout, cols):
    from manta_b200 import native

    rng = np.random.default_rng(cols)
    rows = 5000
    data, scales, _ = pack(layout, make_rows(rng, rows, cols, normalised=(layout != "q4")))
    q = make_rows(rng, 3, cols)
    cands = rt.bind(layout, data, scales, row_base=1000)
    path = str(tmp_path / f"set_{layout}.mb2")
    rt.save_candidates(cands, path)
    info = native.packed_file_info(path)
    assert info["rows"] == rows and info["cols"] == cols and info["row_base"] == 1000
    per_row = {"q8": cols + 4, "q4": cols // 2 + cols // 16, "f16": 2 * cols}[layout]
    assert info["stored_bytes"] == rows * per_row  # packed bytes, not rows * cols * 4
    assert os.path.getsize(path) <= 256 + rows * per_row + 512
    want = rt.score(cands, "cosine", q)
    back = rt.load_candidates(path, verify=True)
    np.testing.assert_array_equal(rt.score(back, "cosine", q), want)
    ids, sc = rt.score_topk(cands, "dot", q, 7)
    ids2, sc2 = rt.score_topk(back, "dot", q, 7)
    np.testing.assert_array_equal(ids, ids2)
    np.testing.assert_array_equal(sc, sc2)
    assert ids.min() >= 1000
    # row shards: ids continue from the file's row base, scores equal the matching slice
    lo, hi = 1234, 4321
    shard = rt.load_candidates(path, lo, hi)
    np.testing.assert_array_equal(rt.score(shard, "cosine", q), want[:, lo:hi])
    sid, _ = rt.score_topk(shard, "dot", q, 5)
    assert sid.min() >= 1000 + lo and sid.max() < 1000 + hi
    for c in (cands, back, shard):
        c.unbind()


def test_load_errors(rt, tmp_path):
    from manta_b200 import native

    bad = tmp_path / "bad.mb2"
    bad.write_bytes(b"not a packed file" * 40)
    with pytest.raises(native.MantaError, match="not a packed candidate file"):
        rt.load_candidates(str(bad))
    with pytest.raises(native.MantaError, match="No such file"):
        rt.load_candidates(str(tmp_path / "missing.mb2"))
    rng = np.random.default_rng(0)
    data, scales, _ = pack("q8", make_rows(rng, 100, 64))
    cands = rt.bind("q8", data, scales)
    path = str(tmp_path / "ok.mb2")
    rt.save_candidates(cands, path)
    cands.unbind()
    with pytest.raises(native.MantaError, match="outside the file"):
        rt.load_candidates(path, 50, 101)
    raw = bytearray(open(path, "rb").read())
    raw[300] ^= 0xFF
    open(path, "wb").write(bytes(raw))
    with pytest.raises(native.MantaError, match="checksum mismatch"):
        rt.load_candidates(path, verify=True)
