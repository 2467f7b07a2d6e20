"""Packed int4 runtime layout (ops.gemm.Int4Weight) on CPU: codes survive the packing, and the
dequantised weight equals the checkpoint format's definition (models.quantize)."""
import pytest
import torch


def test_int4_weight_roundtrip_and_dequant_match_checkpoint_definition():
    from easy_to_hard_b200.models import quantize as qz
    from easy_to_hard_b200.ops.gemm import Int4Weight
    torch.manual_seed(0)
    w = (torch.randn(64, 512) * 0.05).bfloat16()
    q, sz = qz.group_quantize_tensor(w, 4, 128)                 # codes 0..15, [K/g, N, 2] bf16
    packed = Int4Weight.from_int(q, sz, 128)
    assert packed.q.dtype == torch.uint8 and packed.q.shape == (64, 256)
    assert torch.equal(packed.codes(), q)
    want = qz.group_dequantize_tensor(q, sz, 4, 128)
    assert torch.equal(packed.dequant(), want.to(torch.bfloat16))
    # word layout: 8 consecutive k as sum_j q[2j] << 4j | q[2j+1] << (16 + 4j)
    word = int(packed.q.view(torch.int32)[0, 0].item()) & 0xFFFFFFFF
    k = q[0, :8].tolist()
    expect = sum(k[2 * j] << (4 * j) | k[2 * j + 1] << (16 + 4 * j) for j in range(4))
    assert word == expect
    # through the tinygemm packing of the checkpoint and back
    tg = qz.pack_int4_tinygemm(q, 8)
    assert torch.equal(qz.unpack_int4_tinygemm(tg, 8), q)


def test_int4_checkpoint_shapes_follow_the_reference_padding_rule():
    """Input widths that fit the packed layout (4096, and the 7B FFN width 11008 = 86 groups of
    128) are stored unpadded; only widths that do not fit are padded to a multiple of 1024
    (models/quantize.py:460-475, 513-535 of the reference)."""
    import torch.nn as nn
    from easy_to_hard_b200.models import quantize as qz

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(4096, 16, bias=False)
            self.b = nn.Linear(11008, 16, bias=False)
            self.c = nn.Linear(1000, 16, bias=False)     # 1000 % 128 != 0: padded to 1024

    net = Net().to(torch.bfloat16)
    h = qz.WeightOnlyInt4QuantHandler(net, groupsize=128, inner_k_tiles=8)
    sd = h.create_quantized_state_dict()
    assert tuple(sd["a.weight"].shape) == (2, 32, 32, 4)
    assert tuple(sd["a.scales_and_zeros"].shape) == (32, 16, 2)
    assert tuple(sd["b.weight"].shape) == (2, 86, 32, 4)
    assert tuple(sd["b.scales_and_zeros"].shape) == (86, 16, 2)
    assert tuple(sd["c.weight"].shape) == (2, 8, 32, 4)
    assert tuple(sd["c.scales_and_zeros"].shape) == (8, 16, 2)
    rt = h.convert_for_runtime()
    assert not rt.a.padding and not rt.b.padding and rt.c.padding
    assert rt.b.in_features == 11008 and rt.c.in_features == 1024
    rt.load_state_dict(sd)                                  # shapes line up, strictly
    x = torch.randn(3, 11008).to(torch.bfloat16)
    w = qz.group_dequantize_tensor(qz.unpack_int4_tinygemm(sd["b.weight"]),
                                   sd["b.scales_and_zeros"], 4, 128)
    torch.testing.assert_close(rt.b(x).float(), (x.float() @ w.float().t()), atol=0.5, rtol=0.05)


def test_quantised_lm_head_in_a_file_is_expanded_at_load():
    """Files written from a model whose head is an nn.Linear carry output.weight int8 +
    output.scales (or packed int4 + scales_and_zeros); the loader turns them into bf16."""
    import torch.nn as nn
    from easy_to_hard_b200.models import quantize as qz

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.output = nn.Linear(256, 64, bias=False)

    torch.manual_seed(0)
    net = Net().to(torch.bfloat16)
    w = net.output.weight.detach().float()
    sd8 = qz.WeightOnlyInt8QuantHandler(net).create_quantized_state_dict()
    assert sd8["output.weight"].dtype == torch.int8 and "output.scales" in sd8
    out = qz.dequantize_head_in_state_dict(dict(sd8))
    assert "output.scales" not in out and out["output.weight"].dtype == torch.bfloat16
    assert float((out["output.weight"].float() - w).abs().max()) < 0.02 * float(w.abs().max())
    sd4 = qz.WeightOnlyInt4QuantHandler(net, 128, 8).create_quantized_state_dict()
    assert sd4["output.weight"].dtype == torch.int32
    out = qz.dequantize_head_in_state_dict(dict(sd4), 128)
    assert "output.scales_and_zeros" not in out and tuple(out["output.weight"].shape) == (64, 256)
    assert float((out["output.weight"].float() - w).abs().max()) < 0.1 * float(w.abs().max())


@pytest.mark.parametrize("world", [2, 4, 8])
def test_int4_feed_forward_shards_at_every_tp_degree(world):
    """11008 input features of w2 are 86 int4 groups: not divisible by 4 or 8. The intermediate
    dimension is padded with zero-weight features before sharding, so the summed partial
    outputs of the ranks equal the unsharded int4 layer."""
    import copy
    import torch.nn as nn
    from easy_to_hard_b200.models import quantize as qz, tp as tpm
    from easy_to_hard_b200.models.model import FeedForward, ModelArgs

    torch.manual_seed(0)
    cfg = ModelArgs(block_size=64, vocab_size=64, n_layer=1, n_head=2, dim=256,
                    intermediate_size=11008)
    holder = nn.Module()
    holder.ffn = FeedForward(cfg).to(torch.bfloat16)
    h = qz.WeightOnlyInt4QuantHandler(holder, 128, 8)
    sd = h.create_quantized_state_dict()
    h.convert_for_runtime()
    holder.load_state_dict(sd)
    x = (torch.randn(5, 256) * 0.5).to(torch.bfloat16)
    want = holder.ffn(x).float()
    total = torch.zeros_like(want)
    for rank in range(world):
        ffn = copy.deepcopy(holder.ffn)
        padded = tpm.pad_int4_ffn_for_tp(ffn, world)
        assert padded == (world in (4, 8))
        for name, style in (("w1", "colwise"), ("w3", "colwise"), ("w2", "rowwise")):
            tpm.shard_linear(getattr(ffn, name), style, world=world, rank=rank)
        assert ffn.w2.in_features == ffn.w1.out_features
        total += ffn(x).float()
    torch.testing.assert_close(total, want, atol=0.05, rtol=0.05)
