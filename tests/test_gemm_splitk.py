"""Cluster split-K GEMM (DSMEM reduction) against fp32 matmul, forced split counts and the automatic choice."""
import pytest
import torch

from vllm_metax_b200 import _custom_ops as ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("splits", [2, 4])
@pytest.mark.parametrize("M,N,K", [(256, 4096, 4096), (200, 520, 1024), (129, 4096, 14336), (256, 264, 512), (65, 128, 64)])
def test_gemm_splitk_forced(M, N, K, splits, kernel_status_ok):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    want = a.float() @ w.float().t() + bias.float() + res.float()
    got = ops.gemm(a, w, bias, res, force_bn=1000 + splits)
    assert (got.float() - want).abs().max() / want.abs().max() < 1.5e-2


def test_gemm_splitk_auto_and_gated(kernel_status_ok):
    torch.manual_seed(1)
    a = torch.randn(256, 14336, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(4096, 14336, device="cuda", dtype=torch.bfloat16) * 0.02
    want = a.float() @ w.float().t()
    got = ops.gemm(a, w)                        # 64 tiles -> split-K path
    assert (got.float() - want).abs().max() / want.abs().max() < 1.5e-2
    # SiLU-gate epilogue over interleaved rows through the split-K kernel
    x = torch.randn(256, 1024, device="cuda", dtype=torch.float16)
    wg = torch.randn(2048, 1024, device="cuda", dtype=torch.float16) * 0.05
    y = x.float() @ wg.float().t()
    want2 = torch.nn.functional.silu(y[:, 0::2].half().float()) * y[:, 1::2].half().float()
    got2 = ops.gemm_silu_mul(x, wg)
    assert (got2.float() - want2).abs().max() / want2.abs().max() < 2e-2
