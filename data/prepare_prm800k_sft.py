"""PRM800K step annotations -> next-step SFT records ``{input, output_prefix, output, is_eos}``
(data/prepare_prm800k_sft.py of the reference): only completions rated +1 are kept, the prefix
is the chosen trajectory so far joined by blank lines, ``is_eos`` marks completions that contain
the final ``# Answer``; examples longer than 768 tokens are filtered out.

    python data/prepare_prm800k_sft.py --output_path prm_sft.json \
        --prm_data_pattern "prm800k/data/*train.jsonl" --train_math_path math_splits/train.jsonl \
        --test_math_path math_splits/test.jsonl
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

MAX_TOTAL_TOKENS = 768


def build(annotations, splitter="\n\n"):
    out, seen = [], set()
    for rec in annotations:
        question, prefix = rec["question"]["problem"], ""
        for step, nxt in walk_prm_steps(rec):
            for comp in step["completions"]:
                text, rating = comp["text"], comp["rating"]
                if rating is not None and rating < 0:
                    continue
                text = normalise_answer_mark(text)
                full = text if prefix == "" else prefix + splitter + text
                if full in seen:
                    continue
                join, add = splitter, not text.startswith("\n\n" + ANSWER_MARK)
                if prefix.endswith("Mr.") or prefix.endswith("Mrs."):
                    join, add = " ", True
                if rating is not None and rating > 0:
                    out.append({"input": question, "output_prefix": prefix,
                                "output": join + text if (prefix != "" and add) else text,
                                "is_eos": ANSWER_MARK in text})
                    seen.add(full)
            if nxt is None:
                break
            prefix = nxt if prefix == "" else prefix + splitter + nxt
    print(f"Number of extended PRM annotations: {len(out)}")
    return out


def main(output_path, prm_data_pattern, train_math_path, test_math_path,
         levels="Level 1, Level 2, Level 3", splitter="\n\n", tokenizer_path=None, seed=0):
    all_p, wanted = math_problem_sets(read_jsonl(train_math_path), read_jsonl(test_math_path),
                                      parse_levels(levels))
    records = build(select_prm_annotations(prm_data_pattern, all_p, wanted), splitter)
    random.Random(seed).shuffle(records)
    write_json(output_path, filter_by_length(records, make_length_fn(tokenizer_path),
                                             MAX_TOTAL_TOKENS))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    for name in ("output_path", "prm_data_pattern", "train_math_path", "test_math_path"):
        ap.add_argument(f"--{name}", required=True)
    ap.add_argument("--levels", default="Level 1, Level 2, Level 3")
    ap.add_argument("--splitter", default="\n\n")
    ap.add_argument("--tokenizer_path", default=None)
    ap.add_argument("--seed", type=int, default=0)
    main(**vars(ap.parse_args()))
