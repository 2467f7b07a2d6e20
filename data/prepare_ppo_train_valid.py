"""MATH train split -> PPO training prompts plus a validation set drawn from the problems that
also occur in the original MATH test split, matched per (subject, level) to the PRM800K test
split (data/prepare_ppo_train_valid.py of the reference).

    python data/prepare_ppo_train_valid.py --train_output_path train_ppo.json \
        --valid_output_path valid_ppo.json --train_math_path math_splits/train.jsonl \
        --test_math_path math_splits/test.jsonl [--original_test_path competition_math_test.jsonl]
"""
from __future__ import annotations

import argparse
import os
import random
import sys
from collections import Counter

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _prep_common import (make_length_fn, parse_levels, ppo_record, question_template,  # noqa: E402
                          read_jsonl, write_json)

MAX_PROMPT_TOKENS = 512 - 16


def build(train_records, test_records, original_test_inputs, length_fn,
          question_format="prm800k", levels="Level 1, Level 2, Level 3", skip_unavailable=False,
          metamath_inputs=frozenset(), seed=42):
    template, lv = question_template(question_format), parse_levels(levels)
    outputs = [ppo_record(ex, template, lv) for ex in train_records]
    budget = Counter((ex["subject"], ex["level"]) for ex in test_records)
    random.Random(seed).shuffle(outputs)
    train, valid, too_long, skipped = [], [], 0, 0
    for rec in outputs:
        if rec["input"] in metamath_inputs:
            skipped += 1
            continue
        key = (rec["subject"], rec["level"])
        if length_fn(rec["input"]) > MAX_PROMPT_TOKENS:
            too_long += 1
            train.append(rec)
        elif budget[key] > 0 and rec["input"] in original_test_inputs:
            valid.append(rec)
            budget[key] -= 1
        else:
            train.append(rec)
    if skip_unavailable:
        train = [r for r in train if r["answer"] != "Unavailable"]
    print("Train:", len(train), "Valid:", len(valid), "MetaMath skipped:", skipped,
          "Over lengthed examples:", too_long)
    print("Count levels in train:", dict(Counter(r["level"] for r in train)))
    return train, valid


def main(train_output_path, valid_output_path, train_math_path, test_math_path,
         original_test_path=None, metamath_path=None, tokenizer_path=None, skip_unavailable=False,
         question_format="prm800k", levels="Level 1, Level 2, Level 3",
         remove_metamath_problems=False, seed=42):
    template = question_template(question_format)
    if original_test_path is not None:
        original = {template.format(question=ex["problem"]) for ex in read_jsonl(original_test_path)}
    else:
        from datasets import load_dataset
        original = {template.format(question=ex["problem"])
                    for ex in load_dataset("hendrycks/competition_math")["test"]}
    metamath = frozenset()
    if remove_metamath_problems:
        if metamath_path is not None:
            rows = read_jsonl(metamath_path)
        else:
            from datasets import load_dataset
            rows = load_dataset("meta-math/MetaMathQA")["train"]
        metamath = frozenset(template.format(question=ex["query"]) for ex in rows)
    train, valid = build(read_jsonl(train_math_path), read_jsonl(test_math_path), original,
                         make_length_fn(tokenizer_path), question_format, levels,
                         skip_unavailable, metamath, seed)
    write_json(train_output_path, train)
    write_json(valid_output_path, valid)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    for name in ("train_output_path", "valid_output_path", "train_math_path", "test_math_path"):
        ap.add_argument(f"--{name}", required=True)
    ap.add_argument("--original_test_path", default=None,
                    help="jsonl of the original MATH test split (else fetched with `datasets`)")
    ap.add_argument("--metamath_path", default=None)
    ap.add_argument("--tokenizer_path", default=None)
    ap.add_argument("--skip_unavailable", action="store_true")
    ap.add_argument("--question_format", default="prm800k")
    ap.add_argument("--levels", default="Level 1, Level 2, Level 3")
    ap.add_argument("--remove_metamath_problems", action="store_true")
    ap.add_argument("--seed", type=int, default=42)
    main(**vars(ap.parse_args()))
