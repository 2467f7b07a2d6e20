"""Weight-only int4 (group-wise) GEMM (ops/csrc/gemm_w8.cu, QB = 4) against an fp32 PyTorch
matmul with the bf16 dequantised weight ((q - 8) * scale + zero, rounded after each step)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(T, F, K, g, seed=0):
    from easy_to_hard_b200.ops.gemm import Int4Weight
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(T, K, device="cuda", generator=gen) * 0.5).bfloat16()
    codes = torch.randint(0, 16, (F, K), device="cuda", generator=gen, dtype=torch.int32)
    scales = (torch.rand(F, K // g, device="cuda", generator=gen) * 0.02 + 0.001).bfloat16()
    zeros = (torch.randn(F, K // g, device="cuda", generator=gen) * 0.05).bfloat16()
    sz = torch.stack([scales, zeros], -1).transpose(0, 1).contiguous()     # [K/g, F, 2]
    w = Int4Weight.from_int(codes, sz, g)
    assert torch.equal(w.codes(), codes)
    return x, w


@pytest.mark.parametrize("T,F,K,g,splitk", [(64, 512, 512, 128, None), (1, 256, 4096, 128, None),
                                            (17, 384, 1024, 64, 1), (64, 256, 4096, 256, 4),
                                            (33, 200, 768, 128, 2), (100, 512, 1024, 128, None),
                                            (64, 256, 11008, 128, 4)])
def test_w4_linear(T, F, K, g, splitk):
    from easy_to_hard_b200.ops import _lib, gemm
    x, w = _case(T, F, K, g)
    want = x.float() @ w.dequant().float().T
    out32 = gemm.linear(x, w, out_dtype=torch.float32, splitk=splitk)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    err = (out32 - want).abs().max() / want.abs().max()
    assert float(err) < 1e-4, float(err)       # identical bf16 weights, fp32 accumulation
    out = gemm.linear(x, w, splitk=splitk)
    assert float((out.float() - want).abs().max() / want.abs().max()) < 1e-2


def test_w4_residual_and_swiglu():
    from easy_to_hard_b200.ops import _lib, gemm
    T, F, K = 64, 640, 1024
    x, w1 = _case(T, F, K, 128, 1)
    _, w3 = _case(T, F, K, 128, 2)
    res = torch.randn(T, F, device="cuda").bfloat16()
    got = gemm.linear_residual(x, w1, res)
    d1, d3 = (x.float() @ w1.dequant().float().T), (x.float() @ w3.dequant().float().T)
    want = res.float() + d1.bfloat16().float()
    assert float((got.float() - want).abs().max()) < 0.03 * float(want.abs().max())
    act = gemm.linear_swiglu(x, w1, w3)
    want = torch.nn.functional.silu(d1.bfloat16().float()).bfloat16().float() * d3.bfloat16().float()
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    assert float((act.float() - want).abs().max()) < 0.03 * float(want.abs().max()) + 1e-3


def test_w4_many_tokens_takes_the_dequantised_path():
    from easy_to_hard_b200.ops import gemm
    x, w = _case(700, 256, 512, 128)
    out = gemm.linear(x, w)
    want = x.float() @ w.dequant().float().T
    assert float((out.float() - want).abs().max() / want.abs().max()) < 1e-2
