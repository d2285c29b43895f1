import numpy as np
import pytest
import torch

from hibana_b200 import _native as nv
from hibana_b200.models.ple import PleTable, ngram_rows


@pytest.mark.skipif(not nv.LIB_PATH.exists(), reason="native library not built")
def test_row_gather_over_shards(tmp_path):
    rng = np.random.default_rng(0)
    row_bytes, per = 160, 1000
    shards, data = [], []
    for i in range(4):
        a = rng.integers(0, 256, size=(per, row_bytes), dtype=np.uint8)
        p = tmp_path / f"shard{i}.bin"
        a.tofile(p)
        shards.append(p)
        data.append(a)
    full = np.concatenate(data)
    t = PleTable(shards, row_bytes, per, threads=4)
    rows = rng.integers(0, 4 * per, size=(37, 5))
    got = t.gather(rows).numpy()
    assert got.shape == (37, 5, row_bytes) and np.array_equal(got, full[rows])
    with pytest.raises(IOError):
        t.gather(np.array([4 * per + 3]))
    t.close()
    res = PleTable(shards, row_bytes, per, resident_limit_bytes=1 << 30)
    assert np.array_equal(res.gather(rows).numpy(), full[rows])


def test_ngram_rows_are_causal_and_stable():
    ids = [5, 9, 9, 2, 7, 9, 9, 2]
    r = ngram_rows(ids, orders=(1, 2, 3), table_rows=1 << 20)
    assert r.shape == (8, 3)
    assert r[2, 0] == r[1, 0] == r[5, 0]           # unigram of token 9
    assert r[3, 1] == r[7, 1]                      # bigram (9, 2)
    assert r[3, 2] == r[7, 2]                      # trigram (9, 9, 2)
    assert np.array_equal(ngram_rows(ids[:5], (1, 2, 3), 1 << 20), r[:5])   # a prefix gives the same rows
