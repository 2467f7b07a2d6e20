"""Checkpoint conversion scripts (round trip, agreement with a Hugging Face LLaMA) and the
data-preparation record shaping on synthetic inputs."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "data")):
    if p not in sys.path:
        sys.path.insert(0, p)


def _hf_state(n_layer=2, n_head=4, n_kv=2, dim=64, ffn=96, vocab=128):
    g = torch.Generator().manual_seed(0)
    hd = dim // n_head

    def r(*s):
        return torch.randn(*s, generator=g)
    st = {"model.embed_tokens.weight": r(vocab, dim), "model.norm.weight": r(dim),
          "lm_head.weight": r(vocab, dim)}
    for i in range(n_layer):
        b = f"model.layers.{i}."
        st[b + "self_attn.q_proj.weight"] = r(n_head * hd, dim)
        st[b + "self_attn.k_proj.weight"] = r(n_kv * hd, dim)
        st[b + "self_attn.v_proj.weight"] = r(n_kv * hd, dim)
        st[b + "self_attn.o_proj.weight"] = r(dim, dim)
        st[b + "self_attn.rotary_emb.inv_freq"] = r(hd // 2)
        st[b + "mlp.gate_proj.weight"] = r(ffn, dim)
        st[b + "mlp.up_proj.weight"] = r(ffn, dim)
        st[b + "mlp.down_proj.weight"] = r(dim, ffn)
        st[b + "input_layernorm.weight"] = r(dim)
        st[b + "post_attention_layernorm.weight"] = r(dim)
    return st


def test_hf_round_trip():
    from easy_to_hard_b200.models.model import ModelArgs
    from scripts.convert_checkpoint_to_hf import gptfast_to_hf
    from scripts.convert_hf_checkpoint import hf_to_gptfast
    cfg = ModelArgs(n_layer=2, n_head=4, n_local_heads=2, dim=64, intermediate_size=96,
                    vocab_size=128)
    hf = _hf_state()
    ours = hf_to_gptfast(hf, cfg)
    assert ours["layers.0.attention.wqkv.weight"].shape == ((4 + 2 * 2) * 16, 64)
    assert not any("inv_freq" in k or ".wq." in k for k in ours)
    back = gptfast_to_hf(ours, heads=(4, 2))
    for k, v in hf.items():
        if "inv_freq" in k:
            continue
        assert torch.equal(back[k], v), k


def test_converted_weights_reproduce_hf_llama_logits():
    transformers = pytest.importorskip("transformers")
    from easy_to_hard_b200.models.model import ModelArgs, Transformer
    from scripts.convert_hf_checkpoint import hf_to_gptfast
    hf_cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=96,
                                      num_hidden_layers=2, num_attention_heads=4,
                                      num_key_value_heads=2, rms_norm_eps=1e-5, rope_theta=10000.0,
                                      max_position_embeddings=64, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(hf_cfg).eval()
    cfg = ModelArgs(block_size=64, n_layer=2, n_head=4, n_local_heads=2, dim=64,
                    intermediate_size=96, vocab_size=128, rope_base=10000, norm_eps=1e-5)
    ours = Transformer(cfg)
    ours.load_state_dict(hf_to_gptfast(hf.state_dict(), cfg), strict=True)
    ours.eval()
    ids = torch.randint(0, 128, (2, 10))
    ours.setup_caches(2, 16, kv_cache=False)
    with torch.no_grad():
        want = hf(ids).logits
        got = ours(ids, torch.arange(10), fully_causal=True)
    assert torch.allclose(got.float(), want.float(), atol=2e-3, rtol=1e-3)


# ------------------------------------------------------------------------------- data prep

def _prm_record(problem):
    def comp(text, rating):
        return {"text": text, "rating": rating}
    return {"question": {"problem": problem},
            "label": {"steps": [
                {"completions": [comp("First step.", 1), comp("Bad step.", -1)],
                 "chosen_completion": 0, "human_completion": None},
                {"completions": [comp("Second step.", 0), comp("Second step.", 0)],
                 "chosen_completion": None, "human_completion": {"text": "Human step."}},
                {"completions": [comp("So x = 2.\n# Answer\n\n2", 1)],
                 "chosen_completion": 0, "human_completion": None}]}}


def test_prm800k_rm_and_sft_records():
    import prepare_prm800k_rm as rm
    import prepare_prm800k_sft as sft
    recs = rm.build([_prm_record("What is 1+1?")])
    assert [r["label"] for r in recs] == [1, 0, 1, 1]
    assert recs[0] == {"input": "What is 1+1?", "output_prefix": "", "output": "First step.\n\n",
                       "label": 1}
    assert recs[2]["output_prefix"] == "First step.\n\n"          # duplicate completion dropped
    assert recs[3]["output_prefix"] == "First step.\n\nHuman step.\n\n"
    assert recs[3]["output"] == "So x = 2.\n\n# Answer\n\n2"      # mark normalised, no splitter
    s = sft.build([_prm_record("What is 1+1?")])
    assert [r["is_eos"] for r in s] == [False, True]               # only ratings > 0 are kept
    assert s[1]["output_prefix"] == "First step.\n\nHuman step."
    assert s[1]["output"].startswith("\n\nSo x = 2.")


def test_metamath_reflow():
    import prepare_metamath as mm
    out = mm.reflow_response("We add. Then we get 4.\nThe answer is: 4")
    assert out == "We add.\n\nThen we get 4.\n\n# Answer\n\n4"
    meta = [{"type": "MATH_AnsAug", "original_question": "easy q", "query": "q1",
             "response": "A. B.\nThe answer is: 1"},
            {"type": "MATH_AnsAug", "original_question": "hard q", "query": "q2",
             "response": "A.\nThe answer is: 2"},
            {"type": "GSM_Rephrased", "original_question": "g", "query": "q3",
             "response": "A.\nThe answer is: 3"}] * 3
    train = [{"problem": "easy q", "level": "Level 2"}, {"problem": "hard q", "level": "Level 5"}]
    selected, pruned = mm.build(meta, train, pruned_numbers=2)
    assert len(selected) == 6 and len(pruned) == 4
    assert all("# Answer" in ex["output"] for ex in selected)


def test_shepherd_steps_and_labels():
    import prepare_metamath_shepherd as sh
    mark = sh.STEP_MARK
    item = {"task": "MATH",
            "input": f"Find x. Step 1: Add one. {mark}\nStep 2: The answer is: 3 {mark}",
            "label": "Find x. Step 1: Add one. +\nStep 2: The answer is: 3 -"}
    rec = sh.convert_item(item, easy_keys={"Findx."})
    assert rec["input"] == "Find x." and rec["level"] == "easy"
    assert rec["label"] == [1, 0] and len(rec["output"]) == 2
    assert rec["output"][1].endswith("# Answer\n\n3")


def test_ppo_prompts():
    import prepare_ppo_test as pt
    import prepare_ppo_train_valid as ptv
    rows = [{"problem": f"p{i}", "answer": str(i), "subject": "Algebra", "level": 1 + i % 5}
            for i in range(10)]
    out = pt.build(rows)
    assert out[0]["input"] == "# Question\n\np0\n\n# Solution\n\n"
    assert [r["answer"] for r in out[:5]] == ["0", "1", "2", "Unavailable", "Unavailable"]
    assert len(pt.build(rows, skip_unavailable=True)) == 6
    original = {r["input"] for r in out[:4]}
    train, valid = ptv.build(rows, rows[:3], original, lambda s: 10)
    assert len(train) + len(valid) == 10 and 1 <= len(valid) <= 3
    assert all(v["input"] in original for v in valid)
