"""tcgen05 GEMM and its fused epilogues against fp32 PyTorch matmuls of the same bf16 inputs."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _check_status():
    from easy_to_hard_b200.ops import _lib
    torch.cuda.synchronize()
    assert _lib.read_status() == 0


def _close(got, want, rtol=2e-2, atol=None):
    want = want.float()
    got = got.float()
    if atol is None:
        atol = 2e-2 * want.abs().max().item() + 1e-3
    err = (got - want).abs().max().item()
    assert torch.allclose(got, want, rtol=rtol, atol=atol), f"max err {err}, atol {atol}"


SHAPES = [  # (T, F, K)
    (64, 4096, 4096), (64, 384, 256), (7, 130, 72), (300, 1000, 512), (512, 512, 1024),
    (64, 4096, 11008), (1, 256, 4096), (129, 128, 64),
]


@pytest.mark.parametrize("T,F,K", SHAPES)
@pytest.mark.parametrize("splitk", [None, 1, 2, 4, 8])
@pytest.mark.parametrize("tf", [128, 64])
def test_linear_bf16(T, F, K, splitk, tf):
    from easy_to_hard_b200.ops import gemm
    x, w = _mk(T, K, seed=1), _mk(F, K, scale=1 / math.sqrt(K), seed=2)
    kb = -(-K // 64)
    bn = None
    if splitk is not None and splitk > 1:
        if kb < splitk:
            pytest.skip("fewer K blocks than splits")
        bn = 64 if T <= 64 else 128
    if tf == 64 and (bn or (64 if T <= 64 else 128 if T <= 128 else 256)) == 256:
        bn = 128
    y = gemm.linear(x, w, splitk=splitk, bn=bn, tf=tf if splitk is not None else None)
    _check_status()
    _close(y, x.float() @ w.float().T)


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_linear_tile_widths_and_f32(bn):
    from easy_to_hard_b200.ops import gemm
    T, F, K = 515, 640, 1088
    x, w = _mk(T, K, seed=3), _mk(F, K, scale=1 / math.sqrt(K), seed=4)
    y = gemm.linear(x, w, out_dtype=torch.float32, bn=bn, splitk=1)
    _check_status()
    _close(y, x.float() @ w.float().T, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("T,splitk", [(64, 1), (64, 2), (64, 4), (200, 1), (1000, 1)])
@pytest.mark.parametrize("tf", [128, 64])
def test_swiglu_and_dual(T, splitk, tf):
    from easy_to_hard_b200.ops import gemm
    K, F = 512, 688
    x = _mk(T, K, seed=5)
    w1, w3 = _mk(F, K, scale=1 / math.sqrt(K), seed=6), _mk(F, K, scale=1 / math.sqrt(K), seed=7)
    y = gemm.linear_swiglu(x, w1, w3, splitk=splitk, tf=tf)
    g = (x.float() @ w1.float().T).bfloat16()
    u = (x.float() @ w3.float().T).bfloat16()
    _check_status()
    _close(y, torch.nn.functional.silu(g) * u)
    o1, o2 = gemm.linear_dual(x, w1, w3, splitk=splitk, tf=tf)
    _check_status()
    _close(o1, g)
    _close(o2, u)


def test_residual():
    from easy_to_hard_b200.ops import gemm
    T, F, K = 64, 1024, 2048
    x, w, r = _mk(T, K, seed=8), _mk(F, K, scale=1 / math.sqrt(K), seed=9), _mk(T, F, seed=10)
    y = gemm.linear_residual(x, w, r)
    _check_status()
    _close(y, r.float() + (x.float() @ w.float().T))


@pytest.mark.parametrize("T,F,K", [(256, 384, 512), (1000, 688, 256), (64, 4096, 4096)])
def test_dgrad_wgrad(T, F, K):
    from easy_to_hard_b200.ops import gemm
    x, w = _mk(T, K, seed=11), _mk(F, K, scale=1 / math.sqrt(K), seed=12)
    dy = _mk(T, F, scale=1 / math.sqrt(F), seed=13)
    dx = gemm.linear_dgrad(dy, w)
    _check_status()
    _close(dx, dy.float() @ w.float())
    dw = gemm.linear_wgrad(dy, x)
    _check_status()
    want = dy.float().T @ x.float()
    _close(dw, want, rtol=1e-3, atol=1e-3 * want.abs().max().item() + 1e-4)
    dw2 = gemm.linear_wgrad(dy, x, out=dw.clone(), accumulate=True)
    _check_status()
    _close(dw2, 2 * want, rtol=1e-3, atol=2e-3 * want.abs().max().item() + 1e-4)


@pytest.mark.parametrize("sq,B,n_head,n_kv,D", [(1, 64, 8, 8, 128), (16, 3, 8, 2, 64),
                                                 (1, 5, 4, 4, 64)])
@pytest.mark.parametrize("tf", [128, 64])
def test_qkv_rope_kv(sq, B, n_head, n_kv, D, tf):
    from easy_to_hard_b200.ops import gemm, reference
    dim, smax, pos0 = 512, 64, 7
    T = B * sq
    x = _mk(T, dim, seed=14)
    wqkv = _mk((n_head + 2 * n_kv) * D, dim, scale=1 / math.sqrt(dim), seed=15)
    freqs = reference.precompute_freqs_cis(smax, D, 10000.0, device="cuda")
    kc = torch.zeros(B + 1, n_kv, smax, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    q = torch.empty(T, n_head * D, dtype=torch.bfloat16, device="cuda")
    pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    gemm.linear_qkv_rope(x, wqkv, q, freqs=freqs, pos_base=pos, sq=sq, n_head=n_head, n_kv=n_kv,
                         head_dim=D, kcache=kc, vcache=vc, tf=tf)
    _check_status()
    qkv = (x.float() @ wqkv.float().T).bfloat16().view(B, sq, -1)
    qr, kr, vr = qkv.split([n_head * D, n_kv * D, n_kv * D], dim=-1)
    fc = freqs[pos0:pos0 + sq]
    qr = reference.apply_rotary_emb(qr.reshape(B, sq, n_head, D), fc)
    kr = reference.apply_rotary_emb(kr.reshape(B, sq, n_kv, D), fc)
    vr = vr.reshape(B, sq, n_kv, D)
    _close(q.view(B, sq, n_head, D), qr)
    _close(kc[:B, :, pos0:pos0 + sq].transpose(1, 2), kr)
    _close(vc[:B, :, pos0:pos0 + sq].transpose(1, 2), vr)
    assert kc[B].abs().sum().item() == 0 and kc[:, :, :pos0].abs().sum().item() == 0


@pytest.mark.parametrize("T,F,K", [(512, 512, 256), (700, 768, 1024), (1536, 1024, 2048 + 64),
                                   (3000, 256, 512)])
def test_cta_pair_tiles_match_fp32(T, F, K):
    """256 x 256 tiles on CTA pairs (cta_group::2): forward, dgrad, wgrad (bf16 and accumulated
    fp32), residual epilogue, ragged token counts, against fp32 PyTorch."""
    from easy_to_hard_b200.ops import _lib, gemm
    g = torch.Generator(device="cuda").manual_seed(T + F)
    x = (torch.randn(T, K, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(F, K, device="cuda", generator=g) * 0.05).bfloat16()
    dy = (torch.randn(T, F, device="cuda", generator=g) * 0.5).bfloat16()
    res = torch.randn(T, F, device="cuda", generator=g).bfloat16()

    def rel(got, want):
        return float((got.float() - want).abs().max() / want.abs().max())

    y = x.float() @ w.float().T
    assert rel(gemm.linear(x, w, pair=True), y) < 1e-2
    assert rel(gemm.linear(x, w, out_dtype=torch.float32, pair=True), y) < 2e-3
    assert rel(gemm.linear_residual(x, w, res, pair=True), res.float() + y.bfloat16().float()) < 1e-2
    assert rel(gemm.linear_dgrad(dy, w, pair=True), dy.float() @ w.float()) < 1e-2
    dw = dy.float().T @ x.float()
    if T % 64 == 0:
        out16 = torch.empty(F, K, device="cuda", dtype=torch.bfloat16)
        assert rel(gemm.linear_wgrad(dy, x, out=out16, pair=True), dw) < 1e-2
        acc = torch.ones(F, K, device="cuda")
        gemm.linear_wgrad(dy, x, out=acc, accumulate=True, pair=True)
        assert rel(acc, dw + 1.0) < 2e-3
    # same numbers as the single-CTA tiles up to accumulation order
    assert rel(gemm.linear(x, w, pair=True), gemm.linear(x, w, pair=False).float()) < 1e-2
    torch.cuda.synchronize()
    assert _lib.read_status() == 0


@pytest.mark.parametrize("T,F,K", [(64, 12288, 4096), (64, 1536, 4096), (64, 4096, 11008),
                                   (8, 6144, 2048), (1, 4002, 4096), (33, 1000, 512),
                                   (64, 4096, 512)])
def test_stream_tiles_of_lower_height_match_fp32(T, F, K):
    """Skinny GEMMs pick a feature-tile height between 64 and 128 rows (and a split-K factor)
    that fills one wave of the SMs; the result is the same product."""
    from easy_to_hard_b200.ops import gemm
    th = {12288: 88, 1536: 96, 4096: 112, 6144: 64, 4002: 72, 1000: 80}[F]
    x, w = _mk(T, K, seed=41), _mk(F, K, scale=0.05, seed=42)
    y = gemm.linear(x, w, th=th)
    _check_status()
    _close(y, x.float() @ w.float().t())
    res = _mk(T, F, seed=43)
    y2 = gemm.linear_residual(x, w, res, th=th, splitk=2 if K >= 2048 else 1)
    _check_status()
    _close(y2, (x.float() @ w.float().t()).bfloat16().float() + res.float())
    y32 = gemm.linear(x, w, out_dtype=torch.float32, th=th, kps=2)
    _check_status()
    _close(y32, x.float() @ w.float().t())


@pytest.mark.parametrize("T,F,K", [(64, 11008, 4096), (64, 1376, 4096), (5, 688, 256)])
def test_stream_tiles_dual_swiglu(T, F, K):
    from easy_to_hard_b200.ops import gemm
    assert gemm.pick_stream_tiles(11008, 4096, 64, True) == 80
    x = _mk(T, K, seed=44)
    w1, w3 = _mk(F, K, scale=0.05, seed=45), _mk(F, K, scale=0.05, seed=46)
    y = gemm.linear_swiglu(x, w1, w3, **({} if F == 11008 else dict(th=72)))
    _check_status()
    g = (x.float() @ w1.float().t()).bfloat16().float()
    u = (x.float() @ w3.float().t()).bfloat16().float()
    _close(y, torch.nn.functional.silu(g).bfloat16().float() * u)
