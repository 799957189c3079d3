"""RMSNorm and residual-add + RMSNorm kernels against the bit-faithful C restatement of op_rmsnorm, through the C
ABI and through the host mirror of the reference's tensor / layer interface.  fp32 with the reference's own
arithmetic order: the gate is bit equality."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _tensor(a):
    from baranet_bdml_b200.tensor import TensorF
    t = TensorF(a.shape[0], a.shape[1], True)
    t.copy_from_numpy(np.ascontiguousarray(a, dtype=np.float32))
    return t


@pytest.mark.parametrize("rows,hidden", [(1, 1), (3, 255), (4, 256), (5, 257), (7, 300), (16, 2048), (2, 4096),
                                         (3, 5000), (1500, 64)])
def test_rmsnorm_bit_exact(lib, cref, rows, hidden):
    rng = np.random.default_rng(rows * 31 + hidden)
    x = (rng.standard_normal((rows, hidden), dtype=np.float32) * 2).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal((1, hidden))).astype(np.float32)
    got = _tensor(x).rmsnorm(_tensor(w), 1e-6).to_numpy()
    assert np.array_equal(got, cref.rmsnorm(x, w, 1e-6))


@pytest.mark.parametrize("rows,hidden", [(2, 64), (9, 2048), (3, 4100)])
def test_add_rmsnorm_is_add_then_norm(lib, cref, rows, hidden):
    rng = np.random.default_rng(rows + hidden)
    a = rng.standard_normal((rows, hidden), dtype=np.float32)
    b = rng.standard_normal((rows, hidden), dtype=np.float32)
    w = (1 + 0.1 * rng.standard_normal((1, hidden))).astype(np.float32)
    total, out = _tensor(a).add_rmsnorm(_tensor(b), _tensor(w), 1e-5)
    s_ref, y_ref = cref.add_rmsnorm(a, b, w, 1e-5)
    assert np.array_equal(total.to_numpy(), s_ref)
    assert np.array_equal(out.to_numpy(), y_ref)
    # and equal to the two separate operators
    assert np.array_equal(out.to_numpy(), _tensor(a + b).rmsnorm(_tensor(w), 1e-5).to_numpy())


def test_rmsnorm_on_strided_views(lib, cref):
    """Transposed and sliced views (element strides), as the reference's Tensor allows."""
    rng = np.random.default_rng(3)
    base = rng.standard_normal((40, 24), dtype=np.float32)
    w = (1 + 0.1 * rng.standard_normal((1, 40))).astype(np.float32)
    t = _tensor(base).transpose()                      # (24, 40) view with swapped strides
    got = t.rmsnorm(_tensor(w), 1e-6).to_numpy()
    assert np.array_equal(got, cref.rmsnorm(np.ascontiguousarray(base.T), w, 1e-6))
    sl = _tensor(base).slice(4, 20, 2, 22)             # rows 4..19, columns 2..21
    w2 = np.ones((1, 20), dtype=np.float32)
    assert np.array_equal(sl.rmsnorm(_tensor(w2), 1e-6).to_numpy(),
                          cref.rmsnorm(np.ascontiguousarray(base[4:20, 2:22]), w2, 1e-6))


def test_rmsnorm_layer_mirror_and_errors(lib, cref):
    from baranet_bdml_b200.layers import RMSNorm
    from baranet_bdml_b200.tensor import AGTensor, TensorF
    rng = np.random.default_rng(11)
    x = rng.standard_normal((4, 128), dtype=np.float32)
    r = rng.standard_normal((4, 128), dtype=np.float32)
    norm = RMSNorm(128, eps=1e-6)
    assert len(norm.parameters()) == 1 and norm.weight.shape == (1, 128)
    y = norm(AGTensor(x)).numpy()
    assert np.array_equal(y, cref.rmsnorm(x, np.ones((1, 128), np.float32), 1e-6))
    total, y2 = norm.add_norm(AGTensor(r), AGTensor(x))
    assert np.array_equal(total.numpy(), r + x)
    assert np.array_equal(y2.numpy(), cref.rmsnorm(r + x, np.ones((1, 128), np.float32), 1e-6))
    with pytest.raises(RuntimeError, match="weight shape must be"):
        _tensor(x).rmsnorm(_tensor(np.ones((1, 64), np.float32)))
    cpu = TensorF(4, 128, False)
    with pytest.raises(RuntimeError, match="only GPU implementation available"):
        cpu.rmsnorm(_tensor(np.ones((1, 128), np.float32)))


def test_rmsnorm_full_size_properties(lib):
    """TinyLLaMA prefill size (16384 rows x 2048): every row has unit RMS after the norm with unit weights, and the
    norm is invariant to a power-of-two rescale of its input (exact in fp32 away from eps)."""
    import torch
    from baranet_bdml_b200 import _lib
    rows, hidden = 16384, 2048
    x = torch.randn((rows, hidden), device="cuda")
    w = torch.ones((hidden,), device="cuda")
    y, y4 = torch.empty_like(x), torch.empty_like(x)
    L = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.bn_rmsnorm_f32(x.data_ptr(), hidden, 1, w.data_ptr(), 1, y.data_ptr(), hidden, 1, rows, hidden, 0.0, st))
    x4 = x * 4
    _lib.check(L.bn_rmsnorm_f32(x4.data_ptr(), hidden, 1, w.data_ptr(), 1, y4.data_ptr(), hidden, 1, rows, hidden, 0.0, st))
    torch.cuda.synchronize()
    rms = y.double().pow(2).mean(dim=1).sqrt()
    assert float((rms - 1).abs().max()) < 1e-6
    assert torch.equal(y, y4)


@pytest.mark.parametrize("rows,hidden", [(1, 8), (5, 2048), (3, 4096), (4, 4104), (700, 512)])
def test_bf16_add_rmsnorm(lib, rows, hidden):
    """bf16 residual stream: the sum is the bf16 rounding of a + b (bit-exact against torch), the norm is within one
    bf16 ulp of fp64 on that rounded sum, and the fused call equals add followed by the plain norm bit for bit."""
    import torch
    from baranet_bdml_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(rows + hidden)
    a = torch.randn((rows, hidden), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn((rows, hidden), generator=g, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn((hidden,), generator=g, device="cuda")).to(torch.bfloat16)
    total, y = ops.add_rmsnorm_bf16(a, b, w, 1e-6)
    want_sum = (a.float() + b.float()).to(torch.bfloat16)
    assert torch.equal(total, want_sum)
    s64 = want_sum.double()
    ref = s64 / torch.sqrt((s64 * s64).mean(dim=1, keepdim=True) + 1e-6) * w.double()
    assert float((y.double() - ref).abs().max()) <= float(ref.abs().max()) * 2.0 ** -8
    _, y_plain = ops.add_rmsnorm_bf16(want_sum, None, w, 1e-6)
    assert torch.equal(y, y_plain)
