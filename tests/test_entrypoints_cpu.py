"""End-to-end runs of the training entry points on CPU: a tiny random ``model.pth`` in the
gpt-fast layout, a sentencepiece ``tokenizer.model`` trained on the spot, a few JSON records,
one epoch, checkpoint written, resume picks it up."""
import json
import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

WORDS = ("solve add subtract number answer question solution step therefore equals two three "
         "four five six seven eight nine ten the of is we get so then x y z sum product").split()


def _sentence(g, n):
    return " ".join(WORDS[int(i)] for i in torch.randint(0, len(WORDS), (n,), generator=g))


@pytest.fixture(scope="module")
def workspace(tmp_path_factory):
    import sentencepiece as spm
    from easy_to_hard_b200.models.model import Transformer
    root = tmp_path_factory.mktemp("ws")
    model_dir = root / "tiny-llama"
    model_dir.mkdir()
    g = torch.Generator().manual_seed(0)
    corpus = root / "corpus.txt"
    corpus.write_text("\n".join(_sentence(g, 12) for _ in range(400)) +
                      "\n# Question\n\n# Solution\n\n0 1 2 3 4 5 6 7 8 9 + - = .\n")
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(model_dir / "tokenizer"),
                                   vocab_size=400, model_type="bpe", bos_id=1, eos_id=2,
                                   unk_id=0, pad_id=-1, byte_fallback=True,
                                   normalization_rule_name="identity",
                                   remove_extra_whitespaces=False,
                                   character_coverage=1.0, minloglevel=2)
    torch.manual_seed(0)
    m = Transformer.from_name("tiny-llama")
    for p in m.parameters():
        if p.dim() == 2:
            torch.nn.init.normal_(p, std=0.05)
    torch.save(m.state_dict(), model_dir / "model.pth")

    sft = [{"query": _sentence(g, 8), "output": _sentence(g, 10)} for _ in range(8)]
    (root / "sft.json").write_text(json.dumps(sft))
    prm = [{"input": _sentence(g, 8), "output_prefix": "", "output": _sentence(g, 6) + "\n\n",
            "label": int(i % 2)} for i in range(8)]
    (root / "prm.json").write_text(json.dumps(prm))
    pairs = [{"input": _sentence(g, 6), "output_1": _sentence(g, 5), "output_2": _sentence(g, 5),
              "preference": 1 + int(i % 2)} for i in range(8)]
    (root / "pairs.json").write_text(json.dumps(pairs))
    return root


def _args(workspace, save_dir, **kw):
    from easy_to_hard_b200.utils.arguments import Arguments
    from easy_to_hard_b200.utils.hf_argparser import HfArgumentParser
    argv = ["--do_train", "--checkpoint_path", str(workspace / "tiny-llama" / "model.pth"),
            "--source_max_len", "32", "--target_max_len", "32", "--total_max_len", "64",
            "--per_device_train_batch_size", "4", "--micro_train_batch_size", "2",
            "--learning_rate", "1e-3", "--num_train_epochs", "1", "--save_strategy", "epoch",
            "--save_dir", str(save_dir), "--param_dtype", "fp32", "--optim_dtype", "fp32",
            "--compute_dtype", "fp32", "--report_to", "none", "--seed", "1"]
    for k, v in kw.items():
        argv += [f"--{k}"] + ([] if v is True else [str(v)])
    return HfArgumentParser((Arguments,)).parse_args_into_dataclasses(argv)[0]


def test_train_sft_end_to_end_and_resume(workspace, tmp_path):
    import train_sft
    save = tmp_path / "sft"
    rec = train_sft.main(_args(workspace, save, dataset=str(workspace / "sft.json"),
                               dataset_format="metamath"))
    assert 3.0 < rec["loss"] < 8.0 and rec["grad_norm"] > 0
    files = sorted(os.listdir(save))
    assert "epoch_1_step_2_rank_0.pt" in files and "last_checkpoint" in files
    ck = torch.load(save / "epoch_1_step_2_rank_0.pt", weights_only=False)
    assert set(ck) >= {"model", "optimizer", "scheduler", "epoch", "global_step"}
    assert all("layers." in k for k in ck["model"])            # only trainable tensors
    assert "layers.0.attention.wqkv.weight" in ck["optimizer"]["state"]
    # a second run resumes: nothing is left to train, the final checkpoint is rewritten
    rec2 = train_sft.main(_args(workspace, save, dataset=str(workspace / "sft.json"),
                                dataset_format="metamath", resume_from_checkpoint=True))
    assert rec2 == {}


def test_train_rm_pointwise_end_to_end(workspace, tmp_path):
    import train_rm_pointwise
    save = tmp_path / "prm"
    rec = train_rm_pointwise.main(_args(workspace, save, dataset=str(workspace / "prm.json"),
                                        dataset_format="prm-v2",
                                        profile=str(tmp_path / "trace")))
    assert 0.3 < rec["loss"] < 1.5
    # --profile: a chrome trace of the steps after the first one
    assert any(f.startswith("trace") and f.endswith(".json") for f in os.listdir(tmp_path))
    ck = torch.load(save / "epoch_1_step_2_rank_0.pt", weights_only=False)
    assert "backbone_model.output.weight" in ck["model"]
    assert ck["model"]["backbone_model.output.weight"].shape == (2, 256)


def test_train_rm_pairwise_end_to_end(workspace, tmp_path):
    import train_rm_pairwise
    save = tmp_path / "orm"
    rec = train_rm_pairwise.main(_args(workspace, save, dataset=str(workspace / "pairs.json")))
    assert 0.3 < rec["loss"] < 1.5 and 0.0 <= rec["accuracy"] <= 1.0
    assert (save / "epoch_1_step_2_rank_0.pt").exists()


@pytest.mark.parametrize("variant", ["dpo", "ipo", "rpo_average"])
def test_train_rl_dpo_end_to_end(workspace, tmp_path, variant):
    import train_rl_dpo
    save = tmp_path / "dpo"
    rec = train_rl_dpo.main(_args(workspace, save, dataset=str(workspace / "pairs.json"),
                                  dpo_variant=variant, dpo_beta=0.1))
    assert rec["loss"] >= 0 and 0.0 <= rec["accuracy"] <= 1.0
    if variant == "dpo":       # policy == reference at the start: loss starts at ln 2
        assert abs(rec["loss"] - 0.693) < 0.1
    assert (save / "epoch_1_step_2_rank_0.pt").exists()


def _read_jsonl(path):
    with open(path) as fh:
        return [json.loads(ln) for ln in fh if ln.strip()]


def test_inference_generate_main_two_dp_ranks_and_resume(workspace, tmp_path):
    """The batched-generation entry point end to end: prompts sorted by length and repeated per
    sample, batches dealt round-robin to two data-parallel (gloo) ranks, both appending to one
    jsonl under flock; --resume_generation only produces what is missing."""
    import mp_workers as W
    g = torch.Generator().manual_seed(4)
    prompts = [{"prompt": _sentence(g, 3 + i)} for i in range(5)]
    pfile = tmp_path / "prompts.json"
    pfile.write_text(json.dumps(prompts))
    out = tmp_path / "gen" / "out.jsonl"
    kw = dict(checkpoint=str(workspace / "tiny-llama" / "model.pth"), prompt_file=str(pfile),
              output_file=str(out))
    W.run(W.generate_main, 2, str(tmp_path / "r1"), **kw)
    rows = _read_jsonl(out)
    # 5 prompts x 2 samples = 10, padded to a multiple of the batch size by repeating the first
    assert len(rows) == 10
    assert all(set(r) == {"idx", "sample_idx", "prompt", "output"} for r in rows)
    per_idx = {}
    for r in rows:
        per_idx.setdefault(r["idx"], []).append(r["sample_idx"])
        assert r["prompt"] == prompts[r["idx"]]["prompt"] and isinstance(r["output"], str)
    assert sorted(per_idx) == [0, 1, 2, 3, 4]
    assert all(sorted(v) == [0, 1] for v in per_idx.values())
    # drop three finished lines, then resume: exactly the missing samples are regenerated
    kept = rows[:7]
    out.write_text("".join(json.dumps(r) + "\n" for r in kept))
    W.run(W.generate_main, 2, str(tmp_path / "r2"), resume=True, **kw)
    rows2 = _read_jsonl(out)
    assert rows2[:7] == kept and len(rows2) >= 10
    count = {}
    for r in rows2:
        count[r["idx"]] = count.get(r["idx"], 0) + 1
    assert all(count[i] >= 2 for i in range(5))
    # nothing left: a further resume appends nothing
    W.run(W.generate_main, 2, str(tmp_path / "r3"), resume=True, **kw)
    assert len(_read_jsonl(out)) == len(rows2)
