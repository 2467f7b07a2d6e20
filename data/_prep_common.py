"""Helpers shared by the data-preparation scripts of this directory (MATH / PRM800K / MetaMath /
Math-Shepherd munging for SFT, reward-model and PPO training). Everything that does the actual
record shaping takes plain Python data, so it runs (and is tested) without any download."""
from __future__ import annotations

import glob
import json
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Set, Tuple

QUESTION_FORMATS = {
    "prm800k": "# Question\n\n{question}\n\n# Solution\n\n",
    "deepseek": ("User: {question}\nPlease reason step by step, and put your final answer within "
                 "\\boxed{{}}.\n\nAssistant:"),
}
ANSWER_MARK = "# Answer\n\n"


def read_jsonl(path: str) -> List[dict]:
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


def write_json(path: str, records, indent: Optional[int] = 2) -> None:
    with open(path, "w") as f:
        json.dump(records, f, indent=indent)
    print(f"Saved {len(records)} records to {path}")


def question_template(name: str) -> str:
    if name not in QUESTION_FORMATS:
        raise ValueError("Unknown question format")
    return QUESTION_FORMATS[name]


def parse_levels(levels: str) -> List[str]:
    return [s.strip() for s in levels.split(",") if s.strip()]


def make_length_fn(tokenizer_path: Optional[str]) -> Callable[[str], int]:
    """Token counter for length filters: a local ``tokenizer.model`` / HF tokenizer directory via
    ``AcceleraTokenizer``, else a whitespace count scaled by 1.3 (no download is attempted)."""
    if tokenizer_path:
        import os
        import sys
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        from easy_to_hard_b200.models.tokenizer_utils import AcceleraTokenizer
        tok = AcceleraTokenizer(tokenizer_path)
        return lambda s: len(tok.encode(s, bos=True, eos=False))
    return lambda s: int(1.3 * len(s.split())) + 1


def math_problem_sets(train: Sequence[dict], test: Sequence[dict], levels: Sequence[str]
                      ) -> Tuple[Set[str], Set[str]]:
    """(all MATH problems, train problems whose ``Level k`` is in ``levels``)."""
    all_problems = {ex["problem"] for ex in list(train) + list(test)}
    wanted = {ex["problem"] for ex in train if f"Level {ex['level']}" in levels}
    return all_problems, wanted


def select_prm_annotations(files_pattern: str, all_problems: Set[str], wanted: Set[str]
                           ) -> List[dict]:
    """PRM800K annotation records whose problem is an easy-level train problem or is not a MATH
    problem at all (held-out MATH problems of other levels are dropped)."""
    out, skipped = [], 0
    for path in sorted(glob.glob(files_pattern)):
        for rec in read_jsonl(path):
            problem = rec["question"]["problem"]
            if problem in wanted or problem not in all_problems:
                out.append(rec)
            else:
                skipped += 1
    print(f"Number of PRM annotations: {len(out)} (skipped {skipped})")
    return out


def normalise_answer_mark(text: str) -> str:
    """``# Answer`` always ends up preceded by exactly one blank line."""
    if ANSWER_MARK in text and "\n" + ANSWER_MARK not in text:
        text = text.replace(ANSWER_MARK, "\n" + ANSWER_MARK)
    if "\n" + ANSWER_MARK in text and "\n\n" + ANSWER_MARK not in text:
        text = text.replace("\n" + ANSWER_MARK, "\n\n" + ANSWER_MARK)
    return text


def walk_prm_steps(record: dict) -> Iterator[Tuple[dict, Optional[str]]]:
    """Yield (step, text that continues the chosen trajectory) for the steps of one PRM800K
    record; the continuation is the chosen completion, else the human completion, else the only
    completion; iteration stops where the trajectory cannot be continued."""
    for step in record["label"]["steps"]:
        if step["completions"] is None:
            return
        if step["chosen_completion"] is not None:
            nxt = step["completions"][step["chosen_completion"]]["text"]
        elif step["human_completion"] is not None:
            nxt = step["human_completion"]["text"]
        elif len(step["completions"]) == 1:
            nxt = step["completions"][0]["text"]
        else:
            nxt = None
        yield step, nxt
        if nxt is None:
            return


def filter_by_length(records: Iterable[dict], length_fn: Callable[[str], int], limit: int
                     ) -> List[dict]:
    kept = [ex for ex in records
            if length_fn(ex["input"] + ex["output_prefix"]) + length_fn(ex["output"]) <= limit]
    print(f"Number of filtered PRM annotations: {len(kept)}")
    return kept


def ppo_record(ex: dict, template: str, levels: Sequence[str]) -> dict:
    """One PPO prompt: the ground-truth answer is only revealed (``answer``) for the allowed
    difficulty levels; ``gt_answer`` is kept for evaluation."""
    gt = ex["answer"]
    return {"input": template.format(question=ex["problem"]),
            "answer": gt if f"Level {ex['level']}" in levels else "Unavailable",
            "gt_answer": gt, "subject": ex["subject"], "level": ex["level"]}
