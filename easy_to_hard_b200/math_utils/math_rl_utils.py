"""Reward shaping for math RL (behaviour of the reference's math_utils/math_rl_utils.py).

* ``post_process_math_rollouts``: pull the predicted answer out of each rollout (after the
  ``\\n\\n# Answer\\n\\n`` stop string, or the last ``\\boxed{}``), grade it against the
  ground truth decoded from the ``answer ;;; gt_answer ;;; level`` side channel, and return
  symbolic rewards plus per-level accuracy counters.
* ``post_process_math_prm_scores``: locate the step boundaries (two consecutive newline tokens)
  inside prompt+response token sequences and take, per reasoning step, the minimum of the three
  reward-model scores around the boundary.
* ``math_stop_token_penalty``: graded 0 / 0.5 / 0.75 / 1.0 penalty for how well the final answer
  is announced.
* ``shape_math_process_rewards``: turn step scores into dense token rewards (``min`` / ``prod``
  scheme) and add the terminal reward.
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..trainers import common_utils
from . import grader

UNAVAILABLE_REWARD = 0.25     # symbolic reward when no label can be checked
POSITIVE_STEP_BUDGET = 0.25   # spread evenly over the steps of a solution
LEVELS = (1, 2, 3, 4, 5)


def rank0_print(*args):
    if int(os.environ.get("LOCAL_RANK", 0)) == 0:
        print(*args)


def _parse_stop_token(stop_token: Optional[str], default: str) -> str:
    if stop_token is None:
        return default
    return stop_token.replace(r"\n", "\n").replace(r"\\", "\\")


def _calculate_outcome_accuracy(predicted_answers: List[str], gt_answers: List[str],
                                answers: List[str], levels: List[int], outcome_reward: bool,
                                easy_outcome_reward: bool, device):
    assert len(predicted_answers) == len(answers)
    assert not (outcome_reward and easy_outcome_reward), \
        "Cannot use both outcome_reward and easy_outcome_reward."
    with common_utils.DisableLogger():
        accuracy = [1.0 if grader.grade_answer(p, g) else 0.0
                    for p, g in zip(predicted_answers, gt_answers)]
        if outcome_reward:
            symbolic = list(accuracy)
        elif easy_outcome_reward:
            symbolic = [UNAVAILABLE_REWARD if a == "Unavailable"
                        else (1.0 if grader.grade_answer(p, a) else 0.0)
                        for p, a in zip(predicted_answers, answers)]
        else:
            symbolic = [UNAVAILABLE_REWARD] * len(predicted_answers)
    out = {"symbolic_rewards": torch.tensor(symbolic, device=device),
           "outcome_accuracy": torch.tensor(accuracy, device=device)}
    lv = torch.tensor(levels, device=device)
    acc = out["outcome_accuracy"]
    for level in LEVELS:
        hit = (lv == level).to(acc.dtype)
        out[f"level_{level}_counts"] = hit
        out[f"level_{level}_accuracy"] = hit * acc
    return out, symbolic


def last_boxed_only_string(string: str) -> Optional[str]:
    """The last ``\\boxed{...}`` (balanced braces) of ``string``."""
    start = string.rfind("\\boxed")
    if start < 0:
        return None
    depth = 0
    for i in range(start, len(string)):
        if string[i] == "{":
            depth += 1
        elif string[i] == "}":
            depth -= 1
            if depth == 0:
                return string[start: i + 1]
    return None


def remove_boxed(s: Optional[str]) -> Optional[str]:
    left = "\\boxed{"
    if s is None or not s.startswith(left) or not s.endswith("}"):
        return None
    return s[len(left):-1]


def post_process_math_rollouts(text_responses: List[str], answer_gt_levels, tokenizer,
                               stop_token: Optional[str], outcome_reward: bool,
                               easy_outcome_reward: bool, device):
    stop = _parse_stop_token(stop_token, tokenizer.eos_token)
    predicted = []
    for text in text_responses:
        answer = "No answer found."
        if "\n\n" in stop:
            if stop in text:
                answer = text.split(stop)[1].split(tokenizer.eos_token)[0]
        elif stop == "\\boxed{}":
            boxed = remove_boxed(last_boxed_only_string(text.split(tokenizer.eos_token)[0]))
            if boxed is not None:
                answer = boxed
        else:
            raise ValueError(f"Unknown stop token: {stop}")
        predicted.append(answer)
    answers, gts, levels = [], [], []
    for line in tokenizer.batch_decode(answer_gt_levels, skip_special_tokens=True):
        parts = line.split(";;;")
        assert len(parts) == 3, line
        answers.append(parts[0].strip())
        gts.append(parts[1].strip())
        levels.append(int(parts[2].strip()))
    metrics, _ = _calculate_outcome_accuracy(predicted, gts, answers, levels, outcome_reward,
                                             easy_outcome_reward, device)
    return metrics


def _pair_positions(tokens: List[int], newline_id: int) -> List[int]:
    """Start indices of non-overlapping (newline, newline) token pairs, left to right."""
    out, i = [], 0
    while i + 1 < len(tokens):
        if tokens[i] == newline_id and tokens[i + 1] == newline_id:
            out.append(i)
            i += 2
        else:
            i += 1
    return out


def _post_process_newline_scores(encoded_full_seq, scores, prompt: str, output: str,
                                 str_splitter: str = "\n\n", newline_id: int = 13):
    """[(offset of the boundary inside the response, min of 3 scores)] for every step of
    ``output`` except the last two segments (the announced answer), plus a readable trace.
    Returns ([], "Parsing error") when text and token boundaries disagree."""
    if str_splitter != "\n\n":
        raise ValueError(f"Unknown str_splitter: {str_splitter}")
    tokens = list(encoded_full_seq)
    n_prompt, n_out = prompt.count(str_splitter), output.count(str_splitter)
    pairs = _pair_positions(tokens, newline_id)
    assert n_prompt + n_out <= len(pairs), (
        f"Something wrong: {n_prompt} + {n_out} v.s. {len(pairs)}\n===\n{prompt}\n===\n{output}")
    assert n_prompt >= 1, "the prompt must end with a step delimiter"
    prompt_len = pairs[n_prompt - 1] + 2          # tokens up to and incl. the last prompt pair
    rest = pairs[n_prompt:]
    if len(rest) != n_out:
        return [], "Parsing error"
    trace = [prompt.strip()]
    found = []
    segments = output.split(str_splitter)
    for i, seg in enumerate(segments):
        if i < n_out - 1:
            pos = rest[i] + 2                      # first token after this boundary
            if pos < prompt_len + 4:               # too close to the prompt to carry a score
                found.append((pos - 2 - prompt_len, -4.44))
                trace.append(f"{seg} (-4.44)")
            else:
                tri = (scores[pos - 3], scores[pos - 2], scores[pos - 1])
                found.append((pos - 2 - prompt_len, min(tri)))
                trace.append(f"{seg} ({tri[0]},{tri[1]},{tri[2]})")
        else:
            trace.append(seg)
    return found, str_splitter.join(trace)


def post_process_math_prm_scores(sequences: torch.Tensor, rewards: torch.Tensor,
                                 text_queries: List[str], text_responses: List[str], tokenizer):
    seqs, scores = sequences.tolist(), rewards.tolist()
    assert len(seqs) == len(scores)
    newline_id = tokenizer.encode("\n\n\n", bos=False, eos=False)[-1]
    packed = [_post_process_newline_scores(seqs[i], scores[i], text_queries[i],
                                           text_responses[i], newline_id=newline_id)
              for i in range(len(seqs))]
    if packed:
        rank0_print("=" * 20)
        rank0_print("Reward:", packed[0][1])
        rank0_print("=" * 20)
    return [p[0] for p in packed]


def math_stop_token_penalty(text_responses: List[str], stop_token: Optional[str],
                            eos_token: str) -> List[float]:
    stop = _parse_stop_token(stop_token, eos_token)
    out = []
    for text in text_responses:
        if stop not in text:
            out.append(1.0)
        elif "\n\n" in stop:
            body, tail = text.split(stop, 1)
            body, tail = body.strip(), tail.split(eos_token)[0]
            last = body.split("\n\n")[-1]
            if tail.strip() == "":
                out.append(1.0)
            elif "\\boxed{" + tail + "}" in body:
                out.append(0.0)            # answer boxed in the solution
            elif f"${tail}$" in last or f"${tail}.$" in last:
                out.append(0.5)            # answer in math mode on the last line
            elif tail in last:
                out.append(0.75)           # answer at least appears on the last line
            else:
                out.append(1.0)
        elif stop == "\\boxed{}":
            out.append(0.0 if "\\boxed" in text else 1.0)
        else:
            raise ValueError(f"Unknown stop token: {stop}")
    return out


def _post_terminating_reward(reward_outputs: Dict[str, torch.Tensor], responses: torch.Tensor,
                             penalize_no_stop_token: bool, relative_stop_token_penalty: bool,
                             stop_token_penalty, penalty_reward_value: float):
    if not penalize_no_stop_token:
        return reward_outputs
    pen = torch.tensor(stop_token_penalty, device=responses.device)
    rewards = reward_outputs["rewards"]
    if relative_stop_token_penalty:
        rewards = rewards + pen * penalty_reward_value
    else:
        rewards[pen > 0.0] = penalty_reward_value
    reward_outputs["rewards"] = rewards
    return reward_outputs


def _step_rewards(step_scores: List[float], scheme: str, upper: float) -> List[float]:
    """A step is charged only when it sets a new minimum (of the score itself, or of the running
    product) below ``upper``; every step also earns an equal share of a small positive budget."""
    running, floor, out = 1.0, upper, []
    for s in step_scores:
        if scheme == "min":
            v = s
        elif scheme == "prod":
            running *= s
            v = running
        else:
            raise ValueError(f"Unknown process_reward_scheme: {scheme}")
        if v < floor:
            out.append(v - floor)
            floor = v
        else:
            out.append(0.0)
    share = POSITIVE_STEP_BUDGET / (len(step_scores) + 1e-6)
    return [x + share for x in out]


def shape_math_process_rewards(symbolic_rewards: torch.Tensor, queries: torch.Tensor,
                               responses: torch.Tensor, tokenizer, device,
                               new_line_scores: List[List[Tuple[int, float]]],
                               stop_token_penalty, penalty_reward_value: float,
                               penalize_no_stop_token: bool, relative_stop_token_penalty: bool,
                               process_reward_scheme: str, process_reward_upper_bound: float,
                               apply_process_reward: bool, apply_terminal_process_reward: bool,
                               process_reward_scale: float):
    """Returns (dense rewards [B, T] or None, per-sequence reward [B], responses)."""
    dense = np.zeros((responses.size(0), responses.size(1)), dtype=float)
    for b, steps in enumerate(new_line_scores):
        assert all(pos >= 0 for pos, _ in steps)
        probs = [1.0 / (1.0 + math.exp(-s)) for _, s in steps]
        vals = _step_rewards(probs, process_reward_scheme, process_reward_upper_bound)
        for (pos, _), v in zip(steps, vals):   # split over the two newline tokens
            dense[b, pos] = v / 2.0
            dense[b, pos + 1] = v / 2.0
        if b == 0:
            rank0_print("=" * 20)
            rank0_print("Normalized Scores:", vals)
            rank0_print("=" * 20)
    terminal = _post_terminating_reward(
        {"rewards": symbolic_rewards.clone()}, responses, penalize_no_stop_token,
        relative_stop_token_penalty, stop_token_penalty, penalty_reward_value)["rewards"]
    if not (apply_process_reward or apply_terminal_process_reward):
        return None, terminal, responses
    shaped = torch.tensor(dense, device=device) * process_reward_scale
    last = (responses != tokenizer.pad_id).sum(dim=1) - 1
    shaped[torch.arange(queries.size(0), device=responses.device), last] += terminal
    if apply_process_reward:
        return shaped, shaped.sum(dim=1), responses
    return None, shaped.sum(dim=1), responses
