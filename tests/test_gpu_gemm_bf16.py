"""bf16 tcgen05 GEMM (C = A @ Bt^T, fp32 accumulation) through the C ABI against an fp64 product of the same
bf16-rounded operands.  Gate: max|got - ref| <= 2^-8 * max|ref| (one bf16 ulp at the largest magnitude) + the
accumulation-order slack of fp32, far below it."""
import numpy as np
import pytest
import torch

from oracle import ref_attention as R

pytestmark = pytest.mark.gpu


def run_case(M, N, K, seed):
    from baranet_bdml_b200 import ops
    rng = np.random.default_rng(seed)
    a = R.round_bf16(rng.standard_normal((M, K), dtype=np.float32))
    bt = R.round_bf16((rng.standard_normal((N, K)) * 0.05).astype(np.float32))
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.gemm_bf16_nt(torch.from_numpy(a).cuda().to(torch.bfloat16), torch.from_numpy(bt).cuda().to(torch.bfloat16),
                           error_word=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = a.astype(np.float64) @ bt.astype(np.float64).T
    return got.float().cpu().numpy(), ref


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 2048), (256, 512, 128), (1, 8, 8), (100, 264, 72),
                                   (129, 257 // 8 * 8, 65 // 8 * 8), (300, 2048, 2048), (1000, 512, 2048),
                                   (4096, 256, 256)])
def test_gemm_matches_fp64_product(lib, M, N, K):
    got, ref = run_case(M, N, K, M + 3 * N + 7 * K)
    scale = max(np.abs(ref).max(), 1e-30)
    assert np.abs(got - ref).max() <= scale * 2.0 ** -8, (M, N, K, np.abs(got - ref).max() / scale)


def test_gemm_projection_shapes_of_the_layer(lib):
    """q_proj / k_proj of TinyLLaMA on 2048 tokens: (2048, 2048) @ (2048, 2048)^T and (2048, 2048) @ (256, 2048)^T;
    linearity in A: gemm(2a) == 2 gemm(a) exactly (a power-of-two scale commutes with every rounding)."""
    from baranet_bdml_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((2048, 2048), generator=g, device="cuda").to(torch.bfloat16)
    for n_out in (2048, 256):
        w = (torch.randn((n_out, 2048), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        y = ops.gemm_bf16_nt(x, w)
        y2 = ops.gemm_bf16_nt((x.float() * 2).to(torch.bfloat16), w)
        torch.cuda.synchronize()
        assert torch.equal(y2.float(), y.float() * 2)
        ref = x.double() @ w.double().T
        assert float((y.double() - ref).abs().max()) <= float(ref.abs().max()) * 2.0 ** -8


def test_gemm_rejects_bad_arguments(lib):
    from baranet_bdml_b200 import ops
    a = torch.zeros((16, 12), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiples of 8"):
        ops.gemm_bf16_nt(a, torch.zeros((8, 12), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError, match="inner dimensions mismatch"):
        ops.gemm_bf16_nt(torch.zeros((16, 16), dtype=torch.bfloat16, device="cuda"),
                         torch.zeros((8, 8), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError, match="only GPU implementation available"):
        ops.gemm_bf16_nt(torch.zeros((16, 16), dtype=torch.bfloat16), torch.zeros((8, 16), dtype=torch.bfloat16))
