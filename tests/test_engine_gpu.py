"""Decode engine against the plain module path of the same model: prefill logits, a few greedy
decode steps, left padding, and weight-only int8 / int4 checkpoints."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(dev="cuda", kv=None, dim=512, heads=4, ffn=1024, vocab=1024, layers=2):
    from easy_to_hard_b200.models.model import ModelArgs, Transformer
    torch.manual_seed(0)
    cfg = ModelArgs(block_size=256, vocab_size=vocab, n_layer=layers, n_head=heads, dim=dim,
                    intermediate_size=ffn, n_local_heads=kv if kv else -1)
    m = Transformer(cfg, freeze_tok_embeddings=True, freeze_output=True, freeze_norm=True)
    g = torch.Generator().manual_seed(1)
    for _, t in list(m.named_parameters()) + list(m.named_buffers()):
        if t.dim() == 2:
            t.data.copy_(torch.randn(t.shape, generator=g) * 0.04)
    return m.to(device=dev, dtype=torch.bfloat16).eval()


def _module_logits(model, prompt, left_pad):
    """Last-position logits of the eager module path with its own KV cache."""
    B, T = prompt.shape
    model.setup_caches(B, 64, kv_cache=True)
    with torch.enable_grad():      # keeps Transformer.forward off the fused scoring path
        out = model(prompt.long(), torch.arange(T, device=prompt.device),
                    left_pad_mask_pos=left_pad)
    return out[:, -1].float().detach()


def _engine_logits(model, prompt, left_pad):
    from easy_to_hard_b200.models.engine import DecodeEngine
    from easy_to_hard_b200.ops import _lib
    eng = DecodeEngine(model, prompt.shape[0], 64, use_graph=False)
    eng.prefill(prompt, left_pad, 0.0, None, 0, -1)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    return eng.logits[: prompt.shape[0]].float().clone(), eng


@pytest.mark.parametrize("kv", [None, 2], ids=["mha", "gqa"])
def test_prefill_logits_match_module_path(kv):
    model = _model(kv=kv)
    prompt = torch.randint(1, 1024, (3, 24), device="cuda", dtype=torch.int32)
    prompt[0, :5] = 0
    left = torch.tensor([5, 0, 0], device="cuda")
    want = _module_logits(copy.deepcopy(model), prompt, left)
    got, _ = _engine_logits(model, prompt, left)
    assert torch.allclose(got, want, atol=0.06, rtol=0.05), float((got - want).abs().max())
    assert torch.equal(got.argmax(-1), want.argmax(-1))


def test_greedy_generation_is_reproducible_and_in_range():
    from easy_to_hard_b200.models.engine import DecodeEngine
    model = _model()
    eng = DecodeEngine(model, 4, 64)
    prompt = torch.randint(1, 1024, (4, 16), device="cuda", dtype=torch.int32)
    a, steps = eng.generate(prompt, None, 12, 0.0, None, None, seed=3)
    b, _ = eng.generate(prompt, None, 12, 0.0, None, None, seed=99)
    torch.cuda.synchronize()
    assert steps == 11 and a.shape == (4, 28)
    assert torch.equal(a, b)                               # greedy ignores the seed
    assert torch.equal(a[:, :16], prompt) and int(a.max()) < 1024 and int(a.min()) >= 0


def test_new_seed_reuses_the_captured_graph_and_changes_the_samples():
    """The sampler's seed lives in device memory: generation calls with different seeds replay
    one captured graph (no capture per call, no growth of the graph cache) and still differ."""
    from easy_to_hard_b200.models.engine import DecodeEngine
    model = _model()
    eng = DecodeEngine(model, 4, 64)
    prompt = torch.randint(1, 1024, (4, 16), device="cuda", dtype=torch.int32)
    outs = []
    for seed in (1, 2, 3, 1):
        seq, _ = eng.generate(prompt, None, 24, temperature=1.0, top_k=50, seed=seed)
        outs.append(seq.clone())
    torch.cuda.synchronize()
    assert len(eng._graphs) == 1
    assert torch.equal(outs[0], outs[3])
    assert not torch.equal(outs[0], outs[1]) and not torch.equal(outs[1], outs[2])


def test_vocab_sharded_embedding_without_the_flag_is_refused():
    """An embedding table with V / tp rows indexed by global ids would read past its end: the
    engine refuses the combination instead of launching."""
    from easy_to_hard_b200.models.engine import DecodeEngine
    model = _model()
    model.tp_size = 2
    model.tok_embeddings.register_buffer("weight",
                                         model.tok_embeddings.weight[:512].contiguous())
    with pytest.raises((ValueError, RuntimeError, AssertionError)):
        DecodeEngine(model, 4, 64, reduce="nccl")


def test_int8_weight_only_engine_matches_module_path():
    from easy_to_hard_b200.models.quantize import WeightOnlyInt8QuantHandler
    model = _model()
    q8 = WeightOnlyInt8QuantHandler(copy.deepcopy(model)).convert_for_runtime_on_the_fly()
    q8 = q8.to("cuda").eval()
    prompt = torch.randint(1, 1024, (2, 20), device="cuda", dtype=torch.int32)
    want = _module_logits(copy.deepcopy(q8), prompt, None)
    got, eng = _engine_logits(q8, prompt, None)
    assert eng.W[0]["wqkv"][1] is not None and eng.W[0]["s13"].numel() == 2 * 1024
    assert torch.allclose(got, want, atol=0.08, rtol=0.05), float((got - want).abs().max())
    # and close to the unquantised model (8-bit weights)
    ref, _ = _engine_logits(model, prompt, None)
    assert float((got - ref).abs().max()) < 0.25


def test_int4_weights_are_unpacked_exactly():
    from easy_to_hard_b200.models import quantize as qz
    from easy_to_hard_b200.models.engine import DecodeEngine
    torch.manual_seed(0)
    w = (torch.randn(256, 1024) * 0.05).bfloat16()
    lin = qz.WeightOnlyInt4Linear(1024, 256, groupsize=128, inner_k_tiles=8, padding=True)
    packed, sz = qz.prepare_int4_weight_and_scales_and_zeros(w, 128, 8)
    lin.weight.copy_(packed)
    lin.scales_and_zeros.copy_(sz)
    lin = lin.cuda()
    from easy_to_hard_b200.ops.gemm import Int4Weight
    packed4, scale = DecodeEngine._dense(lin)
    q, sz_again = qz.group_quantize_tensor(w, 4, 128)
    assert torch.equal(sz_again, sz)
    want = qz.group_dequantize_tensor(q, sz, 4, 128).bfloat16()
    # the engine keeps the weight as packed nibbles (streamed as int4 by the decode GEMM)
    assert scale is None and isinstance(packed4, Int4Weight) and packed4.shape == (256, 1024)
    assert packed4.q.shape == (256, 512) and packed4.q.dtype == torch.uint8
    assert torch.equal(packed4.codes().cpu(), q)
    dense = packed4.dequant()
    assert torch.equal(dense.cpu(), want)
    assert float((dense.cpu().float() - w.float()).abs().max()) < 0.03


def test_int4_weight_only_engine_matches_module_path():
    from easy_to_hard_b200.models.quantize import WeightOnlyInt4QuantHandler
    from easy_to_hard_b200.ops.gemm import Int4Weight
    model = _model()
    h = WeightOnlyInt4QuantHandler(copy.deepcopy(model).cpu(), groupsize=128, inner_k_tiles=8)
    sd = h.create_quantized_state_dict()
    q4 = h.convert_for_runtime()
    q4.load_state_dict(sd, strict=False)
    q4 = q4.to("cuda").eval()
    prompt = torch.randint(1, 1024, (2, 20), device="cuda", dtype=torch.int32)
    want = _module_logits(copy.deepcopy(q4), prompt, None)
    got, eng = _engine_logits(q4, prompt, None)
    assert isinstance(eng.W[0]["wqkv"][0], Int4Weight)
    assert torch.allclose(got, want, atol=0.1, rtol=0.05), float((got - want).abs().max())
