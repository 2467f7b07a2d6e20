"""tcgen05 flash attention against the fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(*shape, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, generator=g, device="cuda").bfloat16()


@pytest.mark.parametrize("B,H,Hkv,Sq,Sk,D,pad", [
    (2, 4, 4, 256, 256, 128, False), (1, 8, 2, 300, 300, 128, False), (3, 4, 4, 128, 128, 64, False),
    (2, 4, 4, 200, 200, 128, True), (2, 2, 2, 64, 192, 128, False), (1, 2, 1, 520, 520, 64, True),
    (2, 32, 32, 768, 768, 128, False)])
def test_flash_fwd(B, H, Hkv, Sq, Sk, D, pad):
    from easy_to_hard_b200.ops import _lib, flash, reference
    q = _mk(B, Sq, H, D, seed=1)
    k, v = _mk(B, Sk, Hkv, D, seed=2), _mk(B, Sk, Hkv, D, seed=3)
    left = (torch.randint(0, Sq // 2, (B,), device="cuda", dtype=torch.int32) if pad else None)
    out, lse = flash.flash_fwd(q, k, v, left, return_lse=True)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    off = Sk - Sq
    i = torch.arange(Sq, device="cuda")[:, None] + off
    j = torch.arange(Sk, device="cuda")[None, :]
    mask = (j <= i)[None].expand(B, Sq, Sk)
    if pad:
        mask = (mask & (j[None] >= left[:, None, None])) | (j == i)[None]
    want = reference.attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                               mask[:, None])
    got = out.transpose(1, 2)
    err = (got.float() - want.float()).abs().max().item()
    assert err < 3e-2, f"max err {err}"
    # log-sum-exp of the scaled, masked scores
    kk = k.transpose(1, 2).repeat_interleave(H // Hkv, 1).float()
    s = (q.transpose(1, 2).float() @ kk.transpose(-1, -2)) / D ** 0.5
    s = s.masked_fill(~mask[:, None], float("-inf"))
    assert torch.allclose(lse, torch.logsumexp(s, -1), rtol=1e-2, atol=2e-2)


def test_prefill_attention_cache_layout():
    from easy_to_hard_b200.ops import _lib, attention, reference
    B, S, H, D, smax = 3, 96, 4, 128, 160
    q = _mk(B, S, H, D, seed=4)
    kc, vc = _mk(B + 1, H, smax, D, seed=5), _mk(B + 1, H, smax, D, seed=6)
    left = torch.tensor([0, 5, 40], dtype=torch.int32, device="cuda")
    out = torch.empty(B, S, H * D, dtype=torch.bfloat16, device="cuda")
    attention.prefill_attention(q, kc, vc, left, out)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    mask = attention.prefill_mask(S, left, "cuda")
    want = reference.attention(q.transpose(1, 2), kc[:B, :, :S], vc[:B, :, :S], mask)
    err = (out.view(B, S, H, D).transpose(1, 2).float() - want.float()).abs().max().item()
    assert err < 3e-2, f"max err {err}"


@pytest.mark.parametrize("B,H,Hkv,S,D", [(2, 4, 4, 256, 128), (1, 8, 2, 300, 128),
                                         (2, 4, 4, 128, 64), (1, 2, 2, 768, 128)])
def test_flash_bwd(B, H, Hkv, S, D):
    from easy_to_hard_b200.ops import _lib, flash
    q, k, v = _mk(B, S, H, D, seed=7), _mk(B, S, Hkv, D, seed=8), _mk(B, S, Hkv, D, seed=9)
    d_o = _mk(B, S, H, D, seed=10)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    kk = kf.repeat_interleave(H // Hkv, 2)
    vv = vf.repeat_interleave(H // Hkv, 2)
    s = torch.einsum("bihd,bjhd->bhij", qf, kk) / D ** 0.5
    mask = torch.ones(S, S, dtype=torch.bool, device="cuda").tril()
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), -1)
    ref = torch.einsum("bhij,bjhd->bihd", p, vv)
    ref.backward(d_o.float())
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = flash.causal_attention(qg, kg, vg)
    out.backward(d_o)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    for got, want, name in ((qg.grad, qf.grad, "dq"), (kg.grad, kf.grad, "dk"),
                            (vg.grad, vf.grad, "dv")):
        scale = want.abs().max().item()
        err = (got.float() - want).abs().max().item()
        assert err < 3e-2 * scale + 2e-2, f"{name}: err {err} (scale {scale})"


@pytest.mark.parametrize("N,V,world", [(300, 32016, 1), (64, 1024, 1), (128, 1024, 4)])
def test_fused_ce_stats_and_grad(N, V, world):
    """Fused CE kernels vs fp32 PyTorch, incl. the shard-combine arithmetic of vocab parallel."""
    from easy_to_hard_b200.ops import loss
    g = torch.Generator(device="cuda").manual_seed(3)
    logits = torch.randn(N, V, generator=g, device="cuda") * 3
    tg = torch.randint(0, V, (N,), device="cuda", generator=g)
    temp = 0.7
    per = V // world
    m = torch.stack([loss.ce_stats(logits[:, r * per:(r + 1) * per].contiguous(), tg, temp,
                                   r * per) for r in range(world)])
    gm = m[..., 0].max(0).values
    w = torch.exp(m[..., 0] - gm)
    s, tgt, u = (m[..., 1] * w).sum(0), m[..., 2].sum(0), (m[..., 3] * w).sum(0)
    lse = gm + torch.log(s)
    ent = lse - u / s
    z = (logits / temp).requires_grad_(True)
    lp_ref = torch.log_softmax(z, -1)
    want_lp = lp_ref.gather(-1, tg[:, None]).squeeze(-1)
    want_ent = -(lp_ref.exp() * lp_ref).sum(-1)
    assert torch.allclose(tgt - lse, want_lp, rtol=1e-4, atol=1e-4)
    assert torch.allclose(ent, want_ent, rtol=1e-3, atol=1e-3)
    g_lp = torch.randn(N, generator=g, device="cuda")
    g_en = torch.randn(N, generator=g, device="cuda")
    (want_lp * g_lp + want_ent * g_en).sum().backward()
    want = z.grad / temp
    for r in range(world):
        dl = loss.ce_grad(logits[:, r * per:(r + 1) * per].contiguous(), tg, lse, ent, g_lp,
                          g_en, temp, r * per)
        ref = want[:, r * per:(r + 1) * per]
        assert (dl.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item() + 1e-3
