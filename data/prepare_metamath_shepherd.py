"""Math-Shepherd (MATH part) -> step-labelled reward-model records ``{input, output: [steps],
label: [0/1 per step], level: easy|hard}`` (data/prepare_metamath_shepherd.py of the reference).
A question counts as easy when it matches (exactly, or on a 5..49 character prefix that no hard
question shares) a MetaMath question derived from a Level 1-3 MATH problem. The step tag
``Step k:`` is removed, the Shepherd step marker splits the steps and carries the +/- label,
and ``The answer is:`` becomes a ``# Answer`` paragraph.

    python data/prepare_metamath_shepherd.py --output_1to5_path all.json --output_1to3_path easy.json \
        [--shepherd_path shepherd.jsonl --metamath_path MetaMathQA.jsonl --math_train_path train.jsonl]
"""
from __future__ import annotations

import argparse
import os
import random
import re
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _prep_common import read_jsonl, write_json  # noqa: E402

STEP_MARK = "ки"
PREFIX_LENGTHS = range(5, 50)


def easy_question_index(metamath, math_train):
    easy_problems = {ex["problem"] for ex in math_train
                     if ex["level"] in ("Level 1", "Level 2", "Level 3")}
    easy, hard = [], []
    for ex in metamath:
        if "MATH" in ex["type"]:
            (easy if ex["original_question"] in easy_problems else hard).append(ex)
    hard_keys, easy_keys = set(), set()
    for ex in hard:
        q = ex["original_question"].replace(" ", "")
        hard_keys.add(q)
        hard_keys.update(q[:n] for n in PREFIX_LENGTHS)
    for ex in easy:
        q = ex["original_question"].replace(" ", "")
        easy_keys.add(q)
        easy_keys.update(q[:n] for n in PREFIX_LENGTHS if q[:n] not in hard_keys)
    return easy_keys


def convert_item(item, easy_keys):
    if " Step 1: " not in item["input"]:
        return None
    question, solution = item["input"].split(" Step 1: ", 1)
    solution = "Step 1: " + solution
    labelled = "Step 1: " + item["label"].split(" Step 1: ", 1)[1]
    key = question.replace(" ", "")
    is_easy = key in easy_keys or any(key[:n] in easy_keys for n in PREFIX_LENGTHS)
    steps, labels = [], []
    for step in solution.split(STEP_MARK):
        if not step:
            continue
        steps.append(re.sub(r"Step \d+: ", "\n\n", step).strip())
        labelled = labelled[len(step):]
        if not labelled:
            steps.pop()
            break
        if labelled[0] not in "+-":
            raise ValueError("label error")
        labels.append(1 if labelled[0] == "+" else 0)
        labelled = labelled[1:]
    fixed = []
    for s in steps:
        parts = s.split("The answer is: ")
        fixed.append(parts[0].strip() + "\n\n# Answer\n\n" + parts[1].strip()
                     if len(parts) == 2 else s)
    return {"input": question, "output": fixed, "label": labels,
            "level": "easy" if is_easy else "hard"}


def build(shepherd, metamath, math_train, seed=0):
    easy_keys = easy_question_index(metamath, math_train)
    out = [r for r in (convert_item(it, easy_keys) for it in shepherd if it["task"] == "MATH")
           if r is not None]
    random.Random(seed).shuffle(out)
    easy = [r for r in out if r["level"] == "easy"]
    print("all data:", len(out), "level 1-3:", len(easy))
    return out, easy


def main(output_1to5_path, output_1to3_path, shepherd_path=None, metamath_path=None,
         math_train_path=None):
    if shepherd_path and metamath_path and math_train_path:
        shepherd, metamath, math_train = (read_jsonl(shepherd_path), read_jsonl(metamath_path),
                                          read_jsonl(math_train_path))
    else:
        from datasets import load_dataset
        shepherd = load_dataset("peiyi9979/Math-Shepherd")["train"]
        metamath = load_dataset("meta-math/MetaMathQA")["train"]
        math_train = load_dataset("hendrycks/competition_math")["train"]
    everything, easy = build(shepherd, metamath, math_train)
    write_json(output_1to5_path, everything, indent=None)
    write_json(output_1to3_path, easy)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--output_1to5_path", required=True)
    ap.add_argument("--output_1to3_path", required=True)
    ap.add_argument("--shepherd_path", default=None)
    ap.add_argument("--metamath_path", default=None)
    ap.add_argument("--math_train_path", default=None)
    main(**vars(ap.parse_args()))
