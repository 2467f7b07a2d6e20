"""The training and scoring entry points end to end on one GPU (CUDA kernels throughout: fused
block forward / backward, fused CE and log-prob kernels, AdamW kernel, CUDA-graph decode engine
for the PPO rollout, reward-head kernel): tiny random ``model.pth``, a tokenizer trained on the
spot, a few JSON records."""
import json
import os

import pytest
import torch

from test_entrypoints_cpu import WORDS, _args, _sentence, workspace  # noqa: F401  (fixtures)

pytestmark = pytest.mark.gpu


def _gpu_args(workspace, save, **kw):  # noqa: F811
    a = dict(param_dtype="fp32", optim_dtype="fp32", compute_dtype="bf16")
    a.update(kw)
    return _args(workspace, save, **a)


def _status_ok():
    from easy_to_hard_b200.ops import _lib
    torch.cuda.synchronize()
    assert _lib.read_status() == 0


def test_train_sft_on_gpu(workspace, tmp_path):  # noqa: F811
    import train_sft
    rec = train_sft.main(_gpu_args(workspace, tmp_path / "sft", dataset=str(workspace / "sft.json"),
                                   dataset_format="metamath"))
    assert 3.0 < rec["loss"] < 8.0 and rec["grad_norm"] > 0
    assert "epoch_1_step_2_rank_0.pt" in os.listdir(tmp_path / "sft")
    _status_ok()


def test_train_rm_pointwise_on_gpu(workspace, tmp_path):  # noqa: F811
    import train_rm_pointwise
    rec = train_rm_pointwise.main(_gpu_args(workspace, tmp_path / "prm",
                                            dataset=str(workspace / "prm.json"),
                                            dataset_format="prm-v2"))
    assert 0.3 < rec["loss"] < 1.5
    _status_ok()


def test_inference_reward_on_gpu(workspace, tmp_path):  # noqa: F811
    import inference_reward as ir
    samples = [{"idx": i, "sample_idx": k,
                "prompt": "# Question\n\nadd two three\n\n# Solution\n\n",
                "output": "we get five\n\nso the sum is five\n\n# Answer\n\n5"}
               for i in range(2) for k in range(3)]
    pf = tmp_path / "samples.jsonl"
    pf.write_text("\n".join(json.dumps(s) for s in samples) + "\n")
    out, best = tmp_path / "scored.jsonl", tmp_path / "best.jsonl"
    ir.main(pf, out, batch_size=4, checkpoint_path=workspace / "tiny-llama" / "model.pth",
            compile=False, aggregate="min", best_of_n_file=best)
    recs = [json.loads(x) for x in out.read_text().splitlines()]
    # six samples in batches of four: the first one is repeated to fill the last batch, as the
    # reference does (inference_reward.py:251-252), so it is scored and written more than once
    assert len({(r["idx"], r["sample_idx"]) for r in recs}) == 6
    assert all(len(r["reward"]) == 2 for r in recs)
    assert len(best.read_text().splitlines()) == 2
    _status_ok()


def test_train_rl_ppo_on_gpu(workspace, tmp_path):  # noqa: F811
    """One PPO run (two steps) with policy, value, reference and reward model on the GPU: the
    rollout goes through the CUDA-graph decode engine, scoring and training through the fused
    kernels."""
    import train_rl_ppo
    from easy_to_hard_b200.utils.arguments import Arguments
    from easy_to_hard_b200.utils.hf_argparser import HfArgumentParser
    g = torch.Generator().manual_seed(3)
    data = [{"input": "# Question\n\n" + _sentence(g, 5) + "\n\n# Solution\n\n",
             "answer": str(i % 7), "gt_answer": str(i % 7), "level": 1 + i % 3}
            for i in range(16)]
    (tmp_path / "ppo.json").write_text(json.dumps(data))
    save = tmp_path / "ppo"
    ckpt = str(workspace / "tiny-llama" / "model.pth")
    argv = ["--do_train", "--base_checkpoint_path", ckpt, "--dataset", str(tmp_path / "ppo.json"),
            "--source_max_len", "24", "--target_max_len", "8", "--total_max_len", "32",
            "--rollout_batch_size", "8", "--rollout_per_device_batch_size", "8",
            "--step_batch_size", "8", "--step_per_device_batch_size", "4",
            "--reward_model_per_device_batch_size", "8", "--per_device_eval_batch_size", "8",
            "--noptepochs", "1", "--num_train_epochs", "1", "--learning_rate", "1e-4",
            "--save_strategy", "steps", "--save_steps", "2", "--save_dir", str(save),
            "--param_dtype", "fp32", "--optim_dtype", "fp32", "--compute_dtype", "bf16",
            "--report_to", "none", "--seed", "1", "--kl_coef", "0.01", "--gamma", "1.0",
            "--lam", "0.95", "--whitening_async_stats", "per_gpu", "--temperature", "1.0",
            "--max_grad_norm", "1.0", "--stop_token", r"\n\n# Answer\n\n",
            "--ref_policy_model_bits", "8", "--reward_model_bits", "8"]
    args = HfArgumentParser((Arguments,)).parse_args_into_dataclasses(argv)[0]
    history = train_rl_ppo.main(args)
    assert len(history) == 2
    for stats in history:
        assert "ppo/loss/policy" in stats and "ppo/loss/value" in stats
        assert stats["ppo/loss/grad_norm_policy"] >= 0.0
        assert all(v == v for v in stats.values() if isinstance(v, float))     # no NaN
    assert "policy_step_2_rank_0.pt" in os.listdir(save)
    _status_ok()
