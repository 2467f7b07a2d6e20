"""Weight-only int8 GEMM (ops/csrc/gemm_w8.cu) against an fp32 PyTorch computation of
(x @ w_int8^T) * scales and its fused epilogues."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(T, F, K, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(T, K, device="cuda", generator=g) * 0.5).bfloat16()
    w = torch.randint(-128, 128, (F, K), device="cuda", generator=g, dtype=torch.int8)
    s = (torch.rand(F, device="cuda", generator=g) * 0.01 + 0.001).float()
    return x, w, s


def _ref(x, w, s):
    return (x.float() @ w.float().T) * s[None, :]


@pytest.mark.parametrize("T,F,K,splitk", [(64, 512, 512, None), (1, 256, 4096, None),
                                          (17, 384, 1024, 1), (64, 256, 4096, 4),
                                          (33, 200, 768, 2), (100, 512, 1024, None), (64, 256, 11008, 4),
                                          (64, 128, 11008 // 64 * 64, 8)])
def test_w8_linear(T, F, K, splitk):
    from easy_to_hard_b200.ops import _lib, gemm
    x, w, s = _case(T, F, K)
    out = gemm.linear(x, w, scale=s, splitk=splitk)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    want = _ref(x, w, s)
    err = (out.float() - want).abs().max() / want.abs().max()
    assert float(err) < 1e-2, float(err)
    out32 = gemm.linear(x, w, scale=s, out_dtype=torch.float32, splitk=splitk)
    err = (out32 - want).abs().max() / want.abs().max()
    assert float(err) < 2e-5, float(err)        # exact integers, fp32 accumulation


@pytest.mark.parametrize("F,th,dual", [(1100, 80, False), (1408, 88, False), (1100, 80, True),
                                       (11008, None, True)])
def test_w8_lower_tiles(F, th, dual):
    """Tile heights below 128 rows (what the host picks so that a wide layer covers all SMs):
    same result as the fp32 reference, rows past the tile and past F never leak."""
    from easy_to_hard_b200.ops import _lib, gemm
    T, K = 64, 1024
    x, w1, s1 = _case(T, F, K, 5)
    if dual:
        _, w3, s3 = _case(T, F, K, 6)
        act = gemm.linear_swiglu(x, w1, w3, scale=torch.cat([s1, s3]), th=th)
        g, u = _ref(x, w1, s1).bfloat16().float(), _ref(x, w3, s3).bfloat16().float()
        want = torch.nn.functional.silu(g).bfloat16().float() * u
        assert float((act.float() - want).abs().max()) < 0.03 * float(want.abs().max()) + 1e-3
    else:
        out32 = gemm.linear(x, w1, scale=s1, out_dtype=torch.float32, th=th)
        want = _ref(x, w1, s1)
        assert float((out32 - want).abs().max() / want.abs().max()) < 2e-5
    torch.cuda.synchronize()
    assert _lib.read_status() == 0


def test_w8_residual_and_swiglu():
    from easy_to_hard_b200.ops import _lib, gemm
    T, F, K = 64, 640, 1024
    x, w1, s1 = _case(T, F, K, 1)
    _, w3, s3 = _case(T, F, K, 2)
    res = torch.randn(T, F, device="cuda").bfloat16()
    got = gemm.linear_residual(x, w1, res, scale=s1)
    want = res.float() + _ref(x, w1, s1).bfloat16().float()
    assert float((got.float() - want).abs().max()) < 0.05 * float(want.abs().max())
    act = gemm.linear_swiglu(x, w1, w3, scale=torch.cat([s1, s3]))
    g, u = _ref(x, w1, s1).bfloat16().float(), _ref(x, w3, s3).bfloat16().float()
    want = torch.nn.functional.silu(g).bfloat16().float() * u
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    assert float((act.float() - want).abs().max()) < 0.03 * float(want.abs().max()) + 1e-3


def test_w8_many_tokens_takes_the_expanded_path():
    from easy_to_hard_b200.ops import gemm
    x, w, s = _case(700, 256, 512)
    out = gemm.linear(x, w, scale=s)
    want = _ref(x, w, s)
    assert float((out.float() - want).abs().max() / want.abs().max()) < 1e-2
