"""Packed int4 runtime layout (ops.gemm.Int4Weight) on CPU: codes survive the packing, and the
dequantised weight equals the checkpoint format's definition (models.quantize)."""
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
