"""Fused reward head (ops/csrc/reward_head.cu): final RMSNorm + 2-row head + mean (+ weighted BCE)
against the same computation in PyTorch, and RewardModel scoring through it."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _ref(x, nw, hw, eps):
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).bfloat16() * nw.bfloat16()
    dots = y.float() @ hw.float().T                       # fp32 accumulation
    return dots, dots.bfloat16().float().mean(-1)


@pytest.mark.parametrize("rows,dim", [(37, 512), (64, 4096), (9, 1024), (5, 8192)])
def test_reward_head_matches_pytorch(rows, dim):
    from easy_to_hard_b200.ops import functional as Fn
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = torch.randn(rows, dim, device="cuda", generator=g).bfloat16()
    nw = (1 + 0.1 * torch.randn(dim, device="cuda", generator=g)).bfloat16()
    hw = (0.05 * torch.randn(2, dim, device="cuda", generator=g)).bfloat16()
    want_dots, want = _ref(x, nw, hw, 1e-5)
    reward, dots, _ = Fn.reward_head(x, nw, hw, 1e-5)
    assert float((dots - want_dots).abs().max()) < 2e-3 * float(want_dots.abs().max()) + 1e-4
    assert float((reward - want).abs().max()) < 1e-2 * float(want.abs().max()) + 1e-3
    # a subset of rows, labels and weights: weighted BCE sums
    idx = torch.tensor([rows - 1, 0, rows // 2], device="cuda", dtype=torch.int32)
    labels = torch.tensor([1.0, 0.0, 1.0], device="cuda")
    wts = torch.tensor([0.5, 2.0, 1.0], device="cuda")
    r2, _, acc = Fn.reward_head(x, nw, hw, 1e-5, index=idx, labels=labels, weights=wts)
    assert torch.equal(r2, reward[idx.long()])
    want_loss = (F.binary_cross_entropy_with_logits(r2, labels, reduction="none") * wts).sum()
    assert abs(float(acc[0]) - float(want_loss)) < 1e-4 * max(1.0, float(want_loss))
    assert abs(float(acc[1]) - float(wts.sum())) < 1e-6


def test_reward_head_slices_add_up():
    """Two column slices (a head sharded over its input dimension) sum to the whole."""
    from easy_to_hard_b200.ops import functional as Fn
    x = torch.randn(33, 2048, device="cuda").bfloat16()
    nw = torch.ones(2048, device="cuda").bfloat16()
    hw = (0.05 * torch.randn(2, 2048, device="cuda")).bfloat16()
    _, whole, _ = Fn.reward_head(x, nw, hw, 1e-5)
    _, a, _ = Fn.reward_head(x, nw, hw[:, :1024].contiguous(), 1e-5, k0=0, finalize=False)
    _, b, _ = Fn.reward_head(x, nw, hw[:, 1024:].contiguous(), 1e-5, k0=1024, finalize=False)
    assert float((a + b - whole).abs().max()) < 1e-3 * float(whole.abs().max()) + 1e-5


def test_reward_model_scores_through_the_fused_head():
    from easy_to_hard_b200.models.model import ModelArgs
    from easy_to_hard_b200.models.reward_model import (RewardArgs, RewardModel,
                                                      apply_reward_modeling_head)
    torch.manual_seed(0)
    args = ModelArgs(block_size=64, vocab_size=320, n_layer=2, n_head=4, dim=256,
                     intermediate_size=512)
    rm = RewardModel(RewardArgs(backbone_args=args)).to("cuda", torch.bfloat16)
    apply_reward_modeling_head(rm.backbone_model, init_sceheme="random")
    rm.eval()
    idx = torch.randint(0, 320, (3, 24), device="cuda")
    eos = torch.tensor([23, 10, 5], device="cuda")
    with torch.no_grad():
        fused_tok = rm(idx)
        fused_eos = rm(idx, eos_pos=eos)
    assert fused_tok.shape == (3, 24) and fused_eos.shape == (3,)
    assert torch.allclose(fused_eos, fused_tok[torch.arange(3), eos])
    with torch.enable_grad():                      # the autograd (module) path as the oracle
        ref_tok = rm(idx).detach()
    assert float((fused_tok - ref_tok).abs().max()) < 0.05 * float(ref_tok.abs().max()) + 0.02
