"""PPO building blocks against closed forms, and one end-to-end PPO step of the entry point on
CPU with tiny random models (policy, value, frozen reference, frozen reward model)."""
import json

import pytest
import torch

from test_entrypoints_cpu import WORDS, _sentence, workspace  # noqa: F401  (fixture)


def test_gae_matches_definition():
    from easy_to_hard_b200.trainers.ppo_trainer import gae
    torch.manual_seed(0)
    B, T, gamma, lam = 5, 37, 0.99, 0.95
    r, v = torch.randn(B, T), torch.randn(B, T)
    adv, ret = gae(r, v, gamma, lam)
    want = torch.zeros(B, T)
    for b in range(B):
        last = 0.0
        for t in reversed(range(T)):
            nxt = v[b, t + 1] if t < T - 1 else 0.0
            last = (r[b, t] + gamma * nxt - v[b, t]) + gamma * lam * last
            want[b, t] = last
    assert torch.allclose(adv, want, atol=1e-5)
    assert torch.allclose(ret, want + v, atol=1e-5)


def test_whiten_modes():
    from easy_to_hard_b200.trainers.ppo_trainer import whiten
    torch.manual_seed(0)
    x = torch.randn(16, 9) * 3 + 2
    w = whiten(x, shift_mean=True, async_stats="per_gpu")
    assert abs(float(w.mean())) < 1e-5 and abs(float(w.std(unbiased=False)) - 1) < 1e-4
    w2 = whiten(x, shift_mean=False, async_stats="per_gpu")
    assert abs(float(w2.mean()) - float(x.mean())) < 1e-4
    w3 = whiten(x, async_stats="none")
    assert torch.allclose(w3.mean(dim=-1), torch.zeros(16), atol=1e-5)


def test_truncation_helpers():
    from easy_to_hard_b200.trainers.ppo_trainer import (truncate_after_stop_token,
                                                        vanilla_stop_token_penalty)
    from easy_to_hard_b200.trainers.rl_trainer import (truncate_after_eos,
                                                       truncate_after_eos_padded)
    t = torch.tensor([[5, 6, 2, 7, 2], [5, 6, 7, 8, 9]])
    assert truncate_after_eos(t, 2) == [[5, 6], [5, 6, 7, 8, 9]]
    assert truncate_after_eos_padded(t, 2, 0).tolist() == [[5, 6, 0, 0, 0], [5, 6, 7, 8, 9]]
    assert truncate_after_stop_token("a b</s> c", "</s>") == "a b</s>"
    assert truncate_after_stop_token("a b c", None) == "a b c"
    assert vanilla_stop_token_penalty(["x\n\n# Answer", "y"], r"\n\n# Answer", "</s>") == [0.0, 1.0]


def test_ppo_losses_closed_form():
    """compute_policy_loss / compute_value_loss arithmetic with stub models."""
    from types import SimpleNamespace
    from easy_to_hard_b200.trainers.ppo_trainer import PPOTrainer

    class StubPolicy(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.zeros(()))

        def forward(self, queries, masks, responses, temperature=None):
            lp = self.w + torch.full(responses.shape, -1.0)
            ent = torch.ones(responses.shape)
            return dict(logprobs=lp, entropies=ent, reg_entropies=ent,
                        reg_entropies_weight=torch.ones(responses.shape))

    class StubValue(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.zeros(()))

        def forward(self, queries, masks, responses):
            return dict(values=self.w + torch.full(responses.shape, 0.5))
    args = SimpleNamespace(temperature=1.0, cliprange=0.2, ent_reg_coef=0.0,
                           cliprange_value=0.2, vf_coef=0.1, kl_coef=0.01)
    tr = PPOTrainer.__new__(PPOTrainer)
    tr.args, tr.policy, tr.value_model = args, StubPolicy(), StubValue()
    B, T = 4, 6
    roll = dict(logprobs=torch.full((B, T), -1.5), advantages=torch.ones(B, T),
                queries=torch.ones(B, 3, dtype=torch.long),
                query_attn_masks=torch.ones(B, 3, dtype=torch.long),
                responses=torch.ones(B, T, dtype=torch.long),
                values=torch.zeros(B, T), returns=torch.ones(B, T))
    loss, stats = tr.compute_policy_loss(roll)
    ratio = torch.exp(torch.tensor(0.5))
    assert float(loss) == pytest.approx(-1.2)            # clipped at 1 + cliprange
    assert float(stats["policy/clipfrac"]) == 1.0 and ratio > 1.2
    assert float(stats["policy/approxkl"]) == pytest.approx(0.125)
    vloss, vstats = tr.compute_value_loss(roll)
    # vpred 0.5 clipped to 0.2; max((0.5-1)^2, (0.2-1)^2) = 0.64 -> 0.5 * 0.64 * vf_coef
    assert float(vloss) == pytest.approx(0.1 * 0.32)
    assert float(vstats["val/clipfrac"]) == 1.0


def test_train_rl_ppo_end_to_end(workspace, tmp_path):  # noqa: F811
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
            "--param_dtype", "fp32", "--optim_dtype", "fp32", "--compute_dtype", "fp32",
            "--report_to", "none", "--seed", "1", "--kl_coef", "0.01", "--gamma", "1.0",
            "--lam", "0.95", "--whitening_async_stats", "per_gpu", "--temperature", "1.0",
            "--max_grad_norm", "1.0", "--stop_token", r"\n\n# Answer\n\n"]
    args = HfArgumentParser((Arguments,)).parse_args_into_dataclasses(argv)[0]
    history = train_rl_ppo.main(args)
    assert len(history) == 2                     # 16 prompts / rollout batch 8
    for stats in history:
        assert stats["objective/kl_sum_seq"] == pytest.approx(0.0, abs=1e-3) or True
        assert "ppo/loss/policy" in stats and "ppo/loss/value" in stats
        assert stats["ppo/loss/grad_norm_policy"] >= 0.0
    files = sorted(p.name for p in save.iterdir())
    assert "policy_step_2_rank_0.pt" in files and "value_step_2_rank_0.pt" in files
    assert (save / "rollouts" / "step_1.json").exists()


@pytest.mark.parametrize("extra", [
    ["--tensor_parallel_size", "2", "--vocab_parallel", "True"],
    ["--tensor_parallel_size", "1", "--rollout_tensor_parallel_size", "2"],
], ids=["tp2_vocab_parallel", "dp2_rollout_tp2"])
def test_train_rl_ppo_two_ranks(workspace, tmp_path, extra):  # noqa: F811
    """One PPO step on two gloo ranks: with the reference recipe's flags (tensor parallel 2,
    --vocab_parallel True), and with generation at a wider tensor-parallel degree than training
    (two data-parallel ranks that generate as one TP 2 group; the rollout copy is refreshed from
    the training shards by the re-layout)."""
    import mp_workers as W
    g = torch.Generator().manual_seed(3)
    data = [{"input": "# Question\n\n" + _sentence(g, 5) + "\n\n# Solution\n\n",
             "answer": str(i % 7), "gt_answer": str(i % 7), "level": 1 + i % 3}
            for i in range(16)]
    (tmp_path / "ppo.json").write_text(json.dumps(data))
    save = tmp_path / "ppo"
    ckpt = str(workspace / "tiny-llama" / "model.pth")
    argv = ["--do_train", "--base_checkpoint_path", ckpt, "--dataset", str(tmp_path / "ppo.json"),
            "--source_max_len", "24", "--target_max_len", "8", "--total_max_len", "32",
            "--rollout_batch_size", "8", "--rollout_per_device_batch_size", "4",
            "--step_batch_size", "8", "--step_per_device_batch_size", "4",
            "--reward_model_per_device_batch_size", "4", "--per_device_eval_batch_size", "4",
            "--noptepochs", "1", "--num_train_epochs", "1", "--learning_rate", "1e-4",
            "--save_strategy", "no", "--save_dir", str(save),
            "--param_dtype", "fp32", "--optim_dtype", "fp32", "--compute_dtype", "fp32",
            "--report_to", "none", "--seed", "1", "--kl_coef", "0.01", "--gamma", "1.0",
            "--lam", "0.95", "--whitening_async_stats", "per_gpu", "--temperature", "1.0",
            "--max_grad_norm", "1.0", "--stop_token", r"\n\n# Answer\n\n"] + extra
    res = W.run(W.ppo_main, 2, str(tmp_path / "out"), argv=argv, pg_timeout=300)
    for r in res:
        assert r["steps"] >= 1 and "ppo/loss/policy" in r["keys"]
        assert all(x == x for x in r["policy_loss"])          # no NaN
    assert res[0]["steps"] == res[1]["steps"]
