"""MetaMathQA -> SFT records in the step-per-paragraph format (data/prepare_metamath.py of the
reference): MATH-derived items are kept only when their original question is an easy-level MATH
train problem, the response is re-flowed so that every sentence is its own paragraph and the
final answer follows ``# Answer``; a pruned copy keeps at most ``pruned_numbers`` responses per
query.

    python data/prepare_metamath.py --output_path metamath.json --pruned_output_path pruned.json \
        [--metamath_path MetaMathQA.jsonl --math_train_path competition_math_train.jsonl]
"""
from __future__ import annotations

import argparse
import os
import random
import sys
from collections import defaultdict

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _prep_common import parse_levels, read_jsonl, write_json  # noqa: E402

ABBREVIATIONS = ("Mr.", "Dr.", "Ms.", "Mrs.", "St.", "Prof.")


def reflow_response(response: str) -> str:
    """One sentence per paragraph, display maths kept on one line, answer after ``# Answer``."""
    body, answer = response.split("The answer is: ")[:2]
    out = body.split("####")[0].strip() + "\n\n# Answer\n\n" + answer
    for a, b in (("\\[ ", "\\["), (" \\]", "\\]"), ("\n", "\n\n"), (".\n", ".\n\n"),
                 (". ", ".\n\n"), (".$", ".$\n\n"), ("\\]", "\\]\n\n")):
        out = out.replace(a, b)
    for _ in range(10):
        out = out.replace("\n\n\n", "\n\n").replace("\n ", "\n")
    for a, b in ((",\n\n", ", "), ("\n\n$", " $"), ("\n\n\\]", " \\]"), ("\\[\n\n", "\\[ "),
                 ("$ $", "$$")):
        out = out.replace(a, b)
    out = out.strip()
    for abbr in ABBREVIATIONS:
        out = out.replace(abbr + "\n\n", abbr + " ")
    return out


def build(metamath, math_train, levels="Level 1, Level 2, Level 3", pruned_numbers=8, epoch=1,
          seed=0):
    lv = parse_levels(levels)
    easy = {ex["problem"] for ex in math_train if ex["level"] in lv}
    rng = random.Random(seed)
    selected = [dict(ex) for ex in metamath
                if "MATH" not in ex["type"] or ex["original_question"] in easy]
    rng.shuffle(selected)
    for ex in selected:
        ex["output"] = reflow_response(ex["response"])
    by_query = defaultdict(list)
    for ex in selected:
        by_query[ex["query"]].append(ex)
    pruned = []
    for rows in by_query.values():
        pruned.extend((rows * epoch)[: pruned_numbers * epoch])
    rng.shuffle(pruned)
    print("Before pruning:", len(selected), "After pruning:", len(pruned))
    return selected, pruned


def main(output_path, pruned_output_path, pruned_numbers=8, epoch=1,
         levels="Level 1, Level 2, Level 3", metamath_path=None, math_train_path=None):
    if metamath_path and math_train_path:
        metamath, math_train = read_jsonl(metamath_path), read_jsonl(math_train_path)
    else:
        from datasets import load_dataset
        metamath = load_dataset("meta-math/MetaMathQA")["train"]
        math_train = load_dataset("hendrycks/competition_math")["train"]
    selected, pruned = build(metamath, math_train, levels, pruned_numbers, epoch)
    write_json(output_path, selected)
    write_json(pruned_output_path, pruned)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--output_path", required=True)
    ap.add_argument("--pruned_output_path", required=True)
    ap.add_argument("--pruned_numbers", type=int, default=8)
    ap.add_argument("--epoch", type=int, default=1)
    ap.add_argument("--levels", default="Level 1, Level 2, Level 3")
    ap.add_argument("--metamath_path", default=None)
    ap.add_argument("--math_train_path", default=None)
    main(**vars(ap.parse_args()))
