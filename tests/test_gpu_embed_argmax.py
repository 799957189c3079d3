"""Device-side embedding gather and per-row argmax (row N2) through the host mirror of the reference's tensor
interface, against numpy.  Integer / copy work: the gate is equality."""
import numpy as np
import pytest

from oracle import ref_attention as R

pytestmark = pytest.mark.gpu


def _tensor(a):
    from baranet_bdml_b200.tensor import TensorF
    t = TensorF(a.shape[0], a.shape[1], True)
    t.copy_from_numpy(np.ascontiguousarray(a, dtype=np.float32))
    return t


def ref_argmax(x):
    return R.argmax_rows(x)[:, 0]


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (5, 256), (4, 1001), (2, 32000), (300, 33)])
def test_argmax_matches_sequential_rule(lib, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    got = _tensor(x).argmax().to_numpy()
    assert got.shape == (rows, 1)
    assert np.array_equal(got[:, 0], np.argmax(x, axis=1).astype(np.uint32))


def test_argmax_ties_nan_and_views(lib):
    x = np.zeros((6, 50), dtype=np.float32)
    x[0, [7, 20, 33]] = 5.0                       # ties: the first one
    x[1, :] = -np.inf                             # nothing compares greater than element 0
    x[2, 10] = np.nan; x[2, 30] = 2.0             # a NaN in the middle never wins
    x[3, 0] = np.nan; x[3, 5] = 9.0               # a NaN at element 0 is never beaten
    x[4, 49] = 1.0                                # the last column
    x[5, :] = np.nan
    got = _tensor(x).argmax().to_numpy()[:, 0]
    assert np.array_equal(got, ref_argmax(x))
    assert list(got) == [7, 0, 30, 0, 49, 0]
    # transposed view (element strides): column argmax of the original
    rng = np.random.default_rng(1)
    y = rng.standard_normal((40, 12), dtype=np.float32)
    got_t = _tensor(y).transpose().argmax().to_numpy()[:, 0]
    assert np.array_equal(got_t, np.argmax(y, axis=0).astype(np.uint32))


@pytest.mark.parametrize("vocab,hidden,n", [(50, 8, 7), (1000, 2048, 64), (32000, 2048, 300), (17, 5, 40)])
def test_embedding_gather_is_the_host_gather(lib, vocab, hidden, n):
    rng = np.random.default_rng(vocab + n)
    table = rng.standard_normal((vocab, hidden), dtype=np.float32)
    ids = rng.integers(0, vocab, n).astype(np.uint32)
    ids[0], ids[-1] = 0, vocab - 1
    got = _tensor(table).gather_rows(ids).to_numpy()
    assert np.array_equal(got, R.embed(table, ids))   # what LLaMAModel.embed builds on the host
    # ids straight from a device argmax
    logits = rng.standard_normal((n, vocab), dtype=np.float32)
    nxt = _tensor(logits).argmax()
    assert np.array_equal(_tensor(table).gather_rows(nxt).to_numpy(), table[np.argmax(logits, axis=1)])


def test_embedding_gather_rejects_out_of_range(lib):
    table = np.ones((10, 4), dtype=np.float32)
    with pytest.raises(IndexError):
        _tensor(table).gather_rows(np.array([1, 10], dtype=np.uint32))


def test_argmax_full_vocab_batch(lib):
    """2048 rows x 32000 logits (a prefill's logits): the planted maximum of every row is found."""
    import torch
    from baranet_bdml_b200 import _lib
    rows, cols = 2048, 32000
    x = torch.randn((rows, cols), device="cuda")
    where = torch.randint(0, cols, (rows,), device="cuda")
    x[torch.arange(rows, device="cuda"), where] = 100.0
    out = torch.zeros((rows,), dtype=torch.int32, device="cuda")
    _lib.check(_lib.load().bn_argmax_rows_f32(x.data_ptr(), cols, 1, out.data_ptr(), rows, cols,
                                              torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(out.long(), where)
