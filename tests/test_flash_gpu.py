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
