"""Speculative decoding of ``interactive.py`` on CPU with tiny random models."""
import torch

import interactive as it
from test_entrypoints_cpu import workspace  # noqa: F401  (fixture)


def _model(seed, name="tiny-llama"):
    from easy_to_hard_b200.models.model import Transformer
    torch.manual_seed(seed)
    m = Transformer.from_name(name)
    for p in m.parameters():
        if p.dim() == 2:
            torch.nn.init.normal_(p, std=0.05)
    return m.eval()


def test_identical_draft_is_always_accepted():
    target, draft = _model(0), _model(0)
    prompt = torch.randint(0, 1024, (12,), dtype=torch.int)
    torch.manual_seed(1)
    seq, stats = it.generate(target, prompt, 20, interactive=False, draft_model=draft,
                             speculate_k=4, temperature=0.8, top_k=50)
    assert seq.shape == (32,) and torch.equal(seq[:12], prompt)
    counts = stats["accept_counts"]
    assert sum(counts[:-1]) == 0 and counts[-1] >= 3       # every round yields k + 1 tokens


def test_different_draft_still_produces_valid_tokens():
    target, draft = _model(0), _model(7)
    prompt = torch.randint(0, 1024, (8,), dtype=torch.int)
    torch.manual_seed(2)
    seq, stats = it.generate(target, prompt, 16, interactive=False, draft_model=draft,
                             speculate_k=3, temperature=1.0, top_k=None)
    assert seq.shape == (24,) and int(seq.min()) >= 0 and int(seq.max()) < 1024
    assert sum(stats["accept_counts"]) >= 4


def test_speculative_matches_plain_when_nearly_greedy():
    """At a very low temperature both paths follow the target's argmax."""
    target, draft = _model(0), _model(0)
    prompt = torch.randint(0, 1024, (8,), dtype=torch.int)
    plain, _ = it.generate(target, prompt, 12, interactive=False, draft_model=None,
                           temperature=1e-4, top_k=1)
    spec, _ = it.generate(target, prompt, 12, interactive=False, draft_model=draft,
                          speculate_k=4, temperature=1e-4, top_k=1)
    assert torch.equal(plain, spec)


def test_main_runs(workspace, capsys):  # noqa: F811
    m = it.main(prompt="add two three", num_samples=1, max_new_tokens=8, top_k=20,
                temperature=0.8, checkpoint_path=workspace / "tiny-llama" / "model.pth",
                draft_checkpoint_path=workspace / "tiny-llama" / "model.pth", speculate_k=3)
    assert len(m["tokens_per_sec"]) == 1
    assert "Mean Accepted" in capsys.readouterr().out
