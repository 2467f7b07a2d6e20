"""Work-split skinny GEMM (ops/csrc/gemm_streamk.cu) against an fp32 PyTorch computation of
x @ w^T and its fused epilogues, over CTA counts that make tiles whole, shared by two and
shared by many CTAs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(T, F, K, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(T, K, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(F, K, device="cuda", generator=g) * 0.05).bfloat16()
    return x, w


def _ref(x, w):
    return x.float() @ w.float().T


def _relerr(got, want):
    return float((got.float() - want).abs().max() / want.abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("T,F,K,ctas,kps", [
    (64, 12288, 4096, 0, 0),        # fused QKV shape of the 7B model: 96 tiles over 148 CTAs
    (64, 4096, 11008, 0, 0),        # 32 tiles, 172 k-blocks
    (33, 4096, 4096, 0, 1),
    (16, 32016, 4096, 0, 4),        # more tiles than CTAs, last tile ragged, 32-token tile
    (8, 768, 512, 0, 2),            # fewer units than SMs: every tile shared by 4 CTAs
    (64, 1024, 2048, 7, 2),         # odd CTA count
    (64, 1024, 2048, 8, 4),         # whole tiles only (no workspace traffic)
    (100, 1536, 1024, 37, 2),       # 128-token tile
    (1, 256, 4096, 0, 0),
])
def test_streamk_linear(T, F, K, ctas, kps):
    from easy_to_hard_b200.ops import _lib, gemm
    x, w = _case(T, F, K)
    want = _ref(x, w)
    out32 = gemm.linear(x, w, out_dtype=torch.float32, streamk=True, sk_ctas=ctas, kps=kps)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    assert _relerr(out32, want) < 2e-3
    out = gemm.linear(x, w, streamk=True, sk_ctas=ctas, kps=kps)
    assert _relerr(out, want) < 1e-2
    # the partial sums are added in slot order whichever CTA finishes a tile: bitwise repeatable
    for _ in range(3):
        again = gemm.linear(x, w, out_dtype=torch.float32, streamk=True, sk_ctas=ctas, kps=kps)
        assert torch.equal(again, out32)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0


@pytest.mark.parametrize("T,ctas", [(64, 0), (128, 0), (20, 53)])
def test_streamk_epilogues(T, ctas):
    from easy_to_hard_b200.ops import _lib, gemm
    F, K = 1408, 1024
    x, w1 = _case(T, F, K, 1)
    _, w3 = _case(T, F, K, 2)
    res = torch.randn(T, F, device="cuda").bfloat16()
    got = gemm.linear_residual(x, w1, res, streamk=True, sk_ctas=ctas)
    want = res.float() + _ref(x, w1).bfloat16().float()
    assert float((got.float() - want).abs().max()) < 0.03 * float(want.abs().max())
    act = gemm.linear_swiglu(x, w1, w3, streamk=True, sk_ctas=ctas)
    g, u = _ref(x, w1).bfloat16().float(), _ref(x, w3).bfloat16().float()
    want = torch.nn.functional.silu(g).bfloat16().float() * u
    assert float((act.float() - want).abs().max()) < 0.03 * float(want.abs().max()) + 1e-3
    o1, o2 = gemm.linear_dual(x, w1, w3, streamk=True, sk_ctas=ctas)
    assert _relerr(o1, _ref(x, w1)) < 1e-2 and _relerr(o2, _ref(x, w3)) < 1e-2
    torch.cuda.synchronize()
    assert _lib.read_status() == 0


def test_streamk_matches_tile_per_cta_kernel_on_rope_kv():
    """Fused QKV + RoPE + KV-cache scatter: same result as the tile-per-CTA kernel."""
    from easy_to_hard_b200.ops import _lib, gemm
    B, H, D, smax, dim = 16, 8, 128, 64, 1024
    x, wqkv = _case(B, 3 * H * D, dim, 3)
    ang = torch.rand(smax, D // 2, device="cuda") * 6.28
    freqs = torch.stack([ang.cos(), ang.sin()], -1).bfloat16()
    pos = torch.tensor([5], dtype=torch.int32, device="cuda")
    outs = []
    for sk in (False, True):
        kc = torch.zeros(B, H, smax, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        q = torch.zeros(B, H * D, device="cuda", dtype=torch.bfloat16)
        gemm.linear_qkv_rope(x, wqkv, q, freqs=freqs, pos_base=pos, sq=1, n_head=H, n_kv=H,
                             head_dim=D, kcache=kc, vcache=vc, streamk=sk)
        outs.append((q, kc, vc))
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    for a, b in zip(*outs):
        assert float((a.float() - b.float()).abs().max()) <= 0.02 * float(a.float().abs().max())
    assert float(outs[1][1][:, :, 5].float().abs().max()) > 0
