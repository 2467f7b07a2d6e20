"""MATH test problems -> PPO evaluation prompts (data/prepare_ppo_test.py of the reference).

    python data/prepare_ppo_test.py --output_path test_ppo.json \
        --test_math_path prm800k/math_splits/test.jsonl [--question_format prm800k|deepseek]
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _prep_common import (parse_levels, ppo_record, question_template, read_jsonl,  # noqa: E402
                          write_json)


def build(test_records, question_format="prm800k", levels="Level 1, Level 2, Level 3",
          skip_unavailable=False):
    template, lv = question_template(question_format), parse_levels(levels)
    out = [ppo_record(ex, template, lv) for ex in test_records]
    if skip_unavailable:
        out = [r for r in out if r["answer"] != "Unavailable"]
    return out


def main(output_path, test_math_path, skip_unavailable=False, question_format="prm800k",
         levels="Level 1, Level 2, Level 3"):
    out = build(read_jsonl(test_math_path), question_format, levels, skip_unavailable)
    print("Test:", len(out))
    write_json(output_path, out)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--output_path", required=True)
    ap.add_argument("--test_math_path", required=True)
    ap.add_argument("--skip_unavailable", action="store_true")
    ap.add_argument("--question_format", default="prm800k")
    ap.add_argument("--levels", default="Level 1, Level 2, Level 3")
    main(**vars(ap.parse_args()))
