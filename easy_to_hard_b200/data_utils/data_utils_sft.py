"""SFT data module (reference: data_utils/data_utils_sft.py:52-374).

Sequence layout per example: the source is left-padded / left-truncated to ``source_max_len``
and the target right-padded to ``target_max_len``; they are concatenated and the leading pad of
the source is rotated to the tail, so every row is ``[source, target, pad...]``, cut to
``total_max_len``. Labels are pad on the source (unless ``train_on_source``) and on the padding.
The target is tokenised with a leading "\\n" that is stripped again, which keeps SentencePiece
from inserting its word-initial marker at the start of the target.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Sequence

import torch

from ..trainers import common_utils as utils

ALPACA_PROMPT_DICT = {
    "prompt_input": (
        "Below is an instruction that describes a task, paired with an input that provides "
        "further context. Write a response that appropriately completes the request.\n\n"
        "### Instruction:\n{instruction}\n\n### Input:\n{input}\n\n### Response:\n"),
    "prompt_no_input": (
        "Below is an instruction that describes a task. "
        "Write a response that appropriately completes the request.\n\n"
        "### Instruction:\n{instruction}\n\n### Response:\n"),
}
DROMEDARY_PROMPT_DICT = {
    "prompt_input": "{meta_prompt}\n{instruction}\n\n{input}\n\n### Dromedary",
    "prompt_no_input": "{meta_prompt}\n{instruction}\n\n### Dromedary",
}

_HUB_DATASETS = {
    "alpaca": ("tatsu-lab/alpaca", {}),
    "alpaca-clean": ("yahma/alpaca-cleaned", {}),
    "chip2": ("laion/OIG", {"data_files": "unified_chip2.jsonl"}),
    "self-instruct": ("yizhongw/self_instruct", {"name": "self_instruct"}),
    "hh-rlhf": ("Anthropic/hh-rlhf", {}),
    "longform": ("akoksal/LongForm", {}),
    "oasst1": ("timdettmers/openassistant-guanaco", {}),
}


def preprocess_for_sft(instances: Sequence[Dict], tokenizer, source_max_len: int,
                       target_max_len: int, total_max_len, train_on_source: bool,
                       add_eos_to_target: bool, add_eos_to_marked_target: bool,
                       return_win_rate: bool = False) -> Dict[str, torch.Tensor]:
    sources = [ex["input"] for ex in instances]
    targets = ["\n" + ex["output"] for ex in instances]
    lead = len(tokenizer(["\n"], add_bos=False, add_eos=False)["input_ids"][0])
    src = tokenizer(sources, max_length=source_max_len, padding="max_length", truncation=True,
                    add_bos=True, add_eos=False, padding_side="left", truncation_side="left")
    marked = None
    if add_eos_to_marked_target and "is_eos" in instances[0]:
        marked = [ex["is_eos"] for ex in instances]
    tgt = tokenizer(targets, max_length=target_max_len + lead, padding="max_length",
                    truncation=True, add_bos=False, add_eos=add_eos_to_target, marked_eos=marked,
                    padding_side="right", truncation_side="right")
    pad = tokenizer.pad_id
    ids, labels = [], []
    for n_src, s_ids, t_ids in zip(src["length"], src["input_ids"], tgt["input_ids"]):
        t_ids = t_ids[lead:]
        n_pad = len(s_ids) - n_src
        row = (s_ids + t_ids)[n_pad:] + [pad] * n_pad       # leading pad moves to the tail
        lab = row if train_on_source else [pad] * n_src + t_ids + [pad] * n_pad
        if total_max_len is not None:
            row, lab = row[:total_max_len], lab[:total_max_len]
        ids.append(row)
        labels.append(lab)
    input_ids = torch.tensor(ids)
    out = {"input_ids": input_ids, "attention_mask": input_ids.ne(pad),
           "labels": torch.tensor(labels)}
    if return_win_rate:
        wr = [ex.get("win_rate", 0.5) for ex in instances]
        out["win_rate"] = torch.tensor(wr).view(-1, 1)
    return out


@dataclass
class DataCollatorForCausalLM:
    tokenizer: object
    source_max_len: int
    target_max_len: int
    total_max_len: int
    train_on_source: bool
    add_eos_to_target: bool
    add_eos_to_marked_target: bool

    def __call__(self, instances: Sequence[Dict]) -> Dict[str, torch.Tensor]:
        return preprocess_for_sft(instances, self.tokenizer, self.source_max_len,
                                  self.target_max_len, self.total_max_len, self.train_on_source,
                                  self.add_eos_to_target, self.add_eos_to_marked_target)


def extract_alpaca_dataset(example):
    key = "prompt_input" if example.get("input", "") != "" else "prompt_no_input"
    return {"input": ALPACA_PROMPT_DICT[key].format(**example)}


def extract_dromedary_dataset(example, meta_prompts):
    assert "example_id" in example
    meta = meta_prompts[int(example["example_id"]) % len(meta_prompts)]
    key = "prompt_input" if example.get("input", "") != "" else "prompt_no_input"
    return {"input": DROMEDARY_PROMPT_DICT[key].format(meta_prompt=meta, **example),
            "output": "\n" + example["output"]}


def _question_answer(example, q_head, a_head, a_sep):
    if example["output_prefix"] == "":
        out = {"input": q_head + example["input"] + a_head[:len(a_head) - len(a_sep)],
               "output": a_sep + example["output"]}
    else:
        out = {"input": q_head + example["input"] + a_head + example["output_prefix"],
               "output": example["output"]}
    if "is_eos" in example:
        out["is_eos"] = example["is_eos"]
    return out


def extract_prm_dataset(example):
    """``Question: ...\\n\\nAnswer: prefix`` -> next step."""
    if example["output_prefix"] == "":
        out = {"input": "Question: " + example["input"],
               "output": "\n\nAnswer: " + example["output"]}
    else:
        out = {"input": "Question: " + example["input"] + "\n\nAnswer: "
               + example["output_prefix"], "output": example["output"]}
    if "is_eos" in example:
        out["is_eos"] = example["is_eos"]
    return out


def extract_prm_v2_dataset(example):
    """``# Question\\n\\n...\\n\\n# Solution\\n\\nprefix`` -> next step (PRM800K-style SFT)."""
    return _question_answer(example, "# Question\n\n", "\n\n# Solution\n\n", "\n\n")


def extract_metamath_dataset(example):
    return {"input": "# Question\n\n" + example["query"] + "\n\n# Solution",
            "output": "\n\n" + example["output"], "is_eos": True}


def _load(dataset_name: str, args):
    if dataset_name in _HUB_DATASETS:
        from datasets import load_dataset
        repo, kw = _HUB_DATASETS[dataset_name]
        return load_dataset(repo, **kw)
    if dataset_name == "vicuna":
        raise NotImplementedError("Vicuna data was not released.")
    if os.path.exists(dataset_name):
        args.dataset_format = args.dataset_format or "alpaca"
        try:
            return utils.local_dataset(dataset_name)
        except Exception as e:
            raise ValueError(f"Error loading dataset from {dataset_name}") from e
    raise NotImplementedError(f"Dataset {dataset_name} not implemented yet.")


def _format(dataset, fmt, args):
    if fmt in ("alpaca", "alpaca-clean") or (fmt is None and args.dataset in ("alpaca",
                                                                              "alpaca-clean")):
        dataset = dataset.map(extract_alpaca_dataset, remove_columns=["instruction"])
    elif fmt == "hh-rlhf" or (fmt is None and args.dataset == "hh-rlhf"):
        dataset = dataset.map(lambda x: {"input": "", "output": x["chosen"]})
    elif fmt == "prm":
        dataset = dataset.map(extract_prm_dataset)
    elif fmt == "prm-v2":
        dataset = dataset.map(extract_prm_v2_dataset)
    elif fmt == "metamath":
        dataset = dataset.map(extract_metamath_dataset)
    elif fmt != "mapped":
        raise ValueError(f"Unsupported dataset format: {fmt}")
    keep = {"input", "output", "is_eos"}
    return dataset.remove_columns([c for c in dataset.column_names["train"] if c not in keep])


def make_sft_data_module(tokenizer, args) -> Dict:
    """Dataset(s) with ``input`` / ``output`` (/``is_eos``) columns plus the collator."""
    dataset = _format(_load(args.dataset, args), args.dataset_format, args)
    train_dataset = eval_dataset = None
    if args.do_eval:
        if "eval" in dataset:
            eval_dataset = dataset["eval"]
        else:
            print("Splitting train dataset in train and validation according to "
                  "`eval_dataset_size`")
            dataset = dataset["train"].train_test_split(test_size=args.eval_dataset_size,
                                                        shuffle=True, seed=42)
            eval_dataset = dataset["test"]
        if args.max_eval_samples is not None and len(eval_dataset) > args.max_eval_samples:
            eval_dataset = eval_dataset.select(range(args.max_eval_samples))
    if args.do_train:
        train_dataset = dataset["train"]
        if args.max_train_samples is not None and len(train_dataset) > args.max_train_samples:
            train_dataset = train_dataset.select(range(args.max_train_samples))
    collator = DataCollatorForCausalLM(tokenizer, args.source_max_len, args.target_max_len,
                                       args.total_max_len, args.train_on_source,
                                       args.add_eos_to_target, args.add_eos_to_marked_target)
    return dict(train_dataset=train_dataset, eval_dataset=eval_dataset, data_collator=collator)
