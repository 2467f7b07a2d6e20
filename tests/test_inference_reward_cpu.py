"""Step-boundary scoring, aggregation and best-of-N selection of ``inference_reward``; an
end-to-end CPU run against the workspace of the entry-point tests."""
import json
import math

import pytest
import torch

import inference_reward as ir
from test_entrypoints_cpu import workspace  # noqa: F401  (fixture)

NL, EOS = 13, 2


def _seq(prompt_steps, out_steps, answer=None, eos=True):
    """Token ids for bos + steps joined by blank lines; every word is a distinct id >= 100."""
    ids, nxt = [1], [100]

    def words(n):
        for _ in range(n):
            ids.append(nxt[0])
            nxt[0] += 1
    for n in prompt_steps:
        words(n)
        ids.extend([NL, NL])
    for n in out_steps:
        words(n)
        ids.extend([NL, NL])
    if answer is not None:
        words(2)                    # "# Answer"
        ids.extend([NL, NL])
        words(answer)
    if eos:
        ids.append(EOS)
    return ids


def test_step_scores_are_read_at_first_newline_of_each_gap():
    ids = _seq([3, 2], [4, 5, 3], answer=1)
    scores = [float(i) for i in range(len(ids))]
    prompt = "q q q\n\ns s\n\n"
    output = "a a a a\n\nb b b b b\n\nc c c\n\n# Answer\n\n7"
    got, pretty = ir.post_process_newline_scores(ids + [0, 0, 0], scores + [0, 0, 0], prompt,
                                                 output, False, newline_id=NL, eos_id=EOS)
    bounds = ir.find_step_boundaries(ids, NL)
    assert len(bounds) == 6
    assert got == [float(bounds[2]), float(bounds[3]), float(bounds[4])]
    assert pretty.startswith("q q q")
    # with the answer: the last step is replaced by the score at the token before EOS
    got2, _ = ir.post_process_newline_scores(ids, scores, prompt, output, True, newline_id=NL,
                                             eos_id=EOS)
    assert got2 == [float(bounds[2]), float(bounds[3]), float(len(ids) - 2)]
    # no EOS at the end: the answer is marked broken
    got3, _ = ir.post_process_newline_scores(ids[:-1], scores[:-1], prompt, output, True,
                                             newline_id=NL, eos_id=EOS)
    assert got3[-1] == ir.BROKEN_ANSWER_SCORE


def test_run_of_three_newlines_is_one_boundary():
    assert ir.find_step_boundaries([5, NL, NL, NL, 6, NL, NL], NL) == [1, 5]


def test_aggregation_and_best_of_n():
    assert ir.aggregate_step_scores([], "min") == 0.0
    s = [0.0, 2.0, -1.0]
    sig = [1 / (1 + math.exp(-x)) for x in s]
    assert ir.aggregate_step_scores(s, "min") == pytest.approx(min(sig))
    assert ir.aggregate_step_scores(s, "prod") == pytest.approx(sig[0] * sig[1] * sig[2])
    assert ir.aggregate_step_scores(s, "last") == pytest.approx(sig[2])
    recs = [dict(idx=0, sample_idx=0, aggregate_reward=0.2),
            dict(idx=0, sample_idx=1, aggregate_reward=0.7),
            dict(idx=1, sample_idx=0, aggregate_reward=0.5),
            dict(idx=1, sample_idx=1, aggregate_reward=0.5)]
    best = ir.select_best_of_n(recs)
    assert [(b["idx"], b["sample_idx"]) for b in best] == [(0, 1), (1, 0)]


def test_inference_reward_end_to_end(workspace, tmp_path):  # noqa: F811
    samples = []
    for idx in range(2):
        for k in range(3):
            samples.append({"idx": idx, "sample_idx": k,
                            "prompt": "# Question\n\nadd two three\n\n# Solution\n\n",
                            "output": "we get five\n\nso the sum is five\n\n# Answer\n\n5"})
    pf = tmp_path / "samples.jsonl"
    pf.write_text("\n".join(json.dumps(s) for s in samples) + "\n")
    out, best = tmp_path / "scored.jsonl", tmp_path / "best.jsonl"
    ir.main(pf, out, batch_size=4, checkpoint_path=workspace / "tiny-llama" / "model.pth",
            compile=False, aggregate="min", best_of_n_file=best)
    recs = [json.loads(x) for x in out.read_text().splitlines()]
    assert {(r["idx"], r["sample_idx"]) for r in recs} == {(i, k) for i in range(2)
                                                            for k in range(3)}
    for r in recs:
        assert len(r["reward"]) == 2 and 0.0 <= r["aggregate_reward"] <= 1.0
    assert len(best.read_text().splitlines()) == 2
    # resume: nothing new is written
    ir.main(pf, out, batch_size=4, checkpoint_path=workspace / "tiny-llama" / "model.pth",
            compile=False, resume_generation=True, aggregate="min")
    assert len(out.read_text().splitlines()) >= 6
