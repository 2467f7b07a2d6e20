"""Fused cache-less scoring passes (hidden states, log-probs / entropies, reward scores) and the
GAE kernel against plain PyTorch fp32 computations of the same quantities."""
import copy

import pytest
import torch

from test_engine_gpu import _model

pytestmark = pytest.mark.gpu


def _fp32_copy(model):
    m = copy.deepcopy(model).to(device="cpu", dtype=torch.float32).eval()
    m.freqs_cis, m.causal_mask, m.max_seq_length, m.max_batch_size = None, None, -1, -1
    return m


def test_fused_hidden_states_match_fp32_module():
    from easy_to_hard_b200.models import fused_block
    model = _model(kv=2)
    ids = torch.randint(0, 1024, (3, 200), device="cuda")
    assert fused_block.can_fuse(model, ids)
    got = fused_block.transformer_hidden(model, ids).float().cpu()
    ref = _fp32_copy(model)
    ref.setup_caches(3, 200, kv_cache=False)
    with torch.enable_grad():
        want = ref(ids.cpu(), torch.arange(200), fully_causal=True, return_hidden=True).detach()
    err = (got - want).abs().max() / want.abs().max()
    assert float(err) < 0.03, float(err)


@pytest.mark.parametrize("int8", [False, True], ids=["bf16", "int8"])
def test_policy_logprobs_and_entropies(int8):
    from types import SimpleNamespace
    from easy_to_hard_b200.models import rl_model
    from easy_to_hard_b200.models.quantize import WeightOnlyInt8QuantHandler
    model = _model()
    if int8:
        model = WeightOnlyInt8QuantHandler(model).convert_for_runtime_on_the_fly().cuda().eval()
    args = SimpleNamespace(temperature=0.7, target_max_len=16)
    tok = SimpleNamespace(pad_id=0, eos_id=2)
    B, Q, R = 4, 24, 16
    queries = torch.randint(3, 1024, (B, Q), device="cuda")
    queries[0, :7] = 0
    masks = queries.ne(0).long()
    responses = torch.randint(3, 1024, (B, R), device="cuda")
    responses[1, 10:] = 0
    policy = rl_model.make_policy_with_base_model(args, model, tok).eval()
    with torch.no_grad():
        out = policy(queries, masks, responses, temperature=0.7)
    # fp32 reference: dequantised weights, plain module path on the CPU
    ref = _fp32_copy(model) if not int8 else None
    if int8:
        from easy_to_hard_b200.models.fused_block import dense_weight
        ref = _fp32_copy(_model())
        for blk_r, blk_q in zip(ref.layers, model.layers):
            for name in ("wqkv", "wo"):
                getattr(blk_r.attention, name).weight.data.copy_(
                    dense_weight(getattr(blk_q.attention, name)).float().cpu())
            for name in ("w1", "w3", "w2"):
                getattr(blk_r.feed_forward, name).weight.data.copy_(
                    dense_weight(getattr(blk_q.feed_forward, name)).float().cpu())
    ref_policy = rl_model.make_policy_with_base_model(args, ref, tok).eval()
    ref.logprobs_and_entropy = None       # force the explicit-logits branch of the wrapper
    ref.setup_caches(B, Q + R + 8, kv_cache=False)
    with torch.enable_grad():
        want = ref_policy(queries.cpu(), masks.cpu(), responses.cpu(), temperature=0.7)
    for key, tol in (("logprobs", 0.08), ("entropies", 0.05)):
        a, b = out[key].float().cpu(), want[key].detach().float()
        assert a.shape == (B, R)
        assert float((a - b).abs().max()) < tol, (key, float((a - b).abs().max()))
    assert float(out["logprobs"][1, 10:].abs().max()) == 0.0          # padded labels score 0


@pytest.mark.parametrize("B,T", [(37, 512), (5, 45), (1, 1), (64, 33)])
def test_gae_kernel(B, T):
    from easy_to_hard_b200.trainers.ppo_trainer import gae
    torch.manual_seed(0)
    r, v = torch.randn(B, T), torch.randn(B, T)
    want_adv, want_ret = gae(r, v, 0.99, 0.95)
    adv, ret = gae(r.cuda(), v.cuda(), 0.99, 0.95)
    assert torch.allclose(adv.cpu(), want_adv, atol=2e-4, rtol=1e-4)
    assert torch.allclose(ret.cpu(), want_ret, atol=2e-4, rtol=1e-4)


def test_reward_model_scores_on_fused_path():
    from easy_to_hard_b200.models.reward_model import RewardModel, apply_reward_modeling_head
    model = _model()
    rm = RewardModel.__new__(RewardModel)
    torch.nn.Module.__init__(rm)
    rm.config, rm.backbone_model = None, model
    apply_reward_modeling_head(model, requires_grad=False, init_sceheme="random")
    model.output.weight.data = (torch.randn(2, 512, device="cuda") * 0.05).bfloat16()
    rm = rm.cuda().eval()
    ids = torch.randint(1, 1024, (4, 96), device="cuda")
    eos = torch.tensor([95, 40, 10, 77], device="cuda")
    with torch.no_grad():
        got = rm(ids, eos_pos=eos).float().cpu()
    ref = copy.deepcopy(rm).to(device="cpu", dtype=torch.float32)
    bb = ref.backbone_model
    bb.freqs_cis, bb.causal_mask, bb.max_seq_length, bb.max_batch_size = None, None, -1, -1
    with torch.enable_grad():
        want = ref(ids.cpu(), eos_pos=eos.cpu()).detach()
    assert got.shape == (4,)
    assert float((got - want).abs().max()) < 0.05
