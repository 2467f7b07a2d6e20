"""PRM800K step annotations -> pointwise reward-model records ``{input, output_prefix, output,
label}`` (data/prepare_prm800k_rm.py of the reference): every rated completion of every step
becomes one example whose prefix is the chosen trajectory so far; ratings 0 and 1 are merged
into label 1, -1 is label 0; duplicates of the same full text are dropped; examples longer than
768 - 32 tokens are filtered out.

    python data/prepare_prm800k_rm.py --train_math_path math_splits/train.jsonl \
        --test_math_path math_splits/test.jsonl --prm_data_pattern "prm800k/data/*train.jsonl" \
        --output_path prm_rm.json [--tokenizer_path ckpts/llemma-7b/tokenizer.model]
"""
from __future__ import annotations

import argparse
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _prep_common import (ANSWER_MARK, filter_by_length, make_length_fn,  # noqa: E402
                          math_problem_sets, normalise_answer_mark, parse_levels, read_jsonl,
                          select_prm_annotations, walk_prm_steps, write_json)

MAX_TOTAL_TOKENS = 768 - 32


def build(annotations, splitter="\n\n"):
    out, seen = [], set()
    for rec in annotations:
        question, prefix = rec["question"]["problem"], ""
        for step, nxt in walk_prm_steps(rec):
            for comp in step["completions"]:
                text, rating = comp["text"], comp["rating"]
                if rating is None:
                    continue
                text = normalise_answer_mark(text)
                if "\n\n" + ANSWER_MARK in text:
                    text = text.strip()
                elif len(text) == 0:
                    break
                full = prefix + text
                if full in seen:
                    continue
                seen.add(full)
                tail = splitter
                if text.endswith("Mr.") or text.endswith("Mrs.") or ANSWER_MARK in text:
                    tail = ""
                out.append({"input": question, "output_prefix": prefix, "output": text + tail,
                            "label": 1 if rating >= 0 else 0})
            if nxt is None:
                break
            prefix = prefix + nxt + splitter
    print(f"Number of extended PRM annotations: {len(out)} "
          f"(label 1: {sum(r['label'] for r in out)})")
    return out


def main(train_math_path, test_math_path, prm_data_pattern, output_path,
         levels="Level 1, Level 2, Level 3", splitter="\n\n", tokenizer_path=None, seed=0):
    all_p, wanted = math_problem_sets(read_jsonl(train_math_path), read_jsonl(test_math_path),
                                      parse_levels(levels))
    records = build(select_prm_annotations(prm_data_pattern, all_p, wanted), splitter)
    random.Random(seed).shuffle(records)
    write_json(output_path, filter_by_length(records, make_length_fn(tokenizer_path),
                                             MAX_TOTAL_TOKENS))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    for name in ("train_math_path", "test_math_path", "prm_data_pattern", "output_path"):
        ap.add_argument(f"--{name}", required=True)
    ap.add_argument("--levels", default="Level 1, Level 2, Level 3")
    ap.add_argument("--splitter", default="\n\n")
    ap.add_argument("--tokenizer_path", default=None)
    ap.add_argument("--seed", type=int, default=0)
    main(**vars(ap.parse_args()))
