"""Pointwise (process) reward-model data (reference: data_utils/data_utils_rm_pointwise.py).

Every example is a prompt plus one solution step (``prm`` / ``prm-v2`` / ``prm-v3``: one 0/1
label) or all steps of a solution joined by `` ;;; `` (``prm-v4``: one label per step). The
collators produce ``input_ids``, per-token ``labels`` and per-token loss ``weights``: 1 on the
tokens of a step (all of them with ``train_on_every_token``, otherwise the last three of each
step), 0 on the prompt and the padding.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Sequence

import torch
from torch.nn.utils.rnn import pad_sequence

from ..trainers import common_utils as utils

SPLITTER = " ;;; "


def _step_weights(n_tokens: int, every_token: bool) -> List[int]:
    if every_token or n_tokens <= 3:
        return [1] * n_tokens
    return [0] * (n_tokens - 3) + [1] * 3


def _encode_pair(tokenizer, sources, targets, source_max_len, target_max_len):
    lead = len(tokenizer(["\n"], add_bos=False, add_eos=False)["input_ids"][0])
    src = tokenizer(sources, max_length=source_max_len, padding="max_length", truncation=True,
                    add_bos=True, add_eos=False, padding_side="left", truncation_side="left")
    tgt = tokenizer(["\n" + t for t in targets], max_length=target_max_len + lead,
                    padding="max_length", truncation=True, add_bos=False, add_eos=False,
                    padding_side="right", truncation_side="right")
    return lead, src, tgt


@dataclass
class DataCollatorForPointwiseRewardModeling:
    tokenizer: object
    source_max_len: int
    target_max_len: int
    total_max_len: int
    train_on_every_token: bool

    def __call__(self, instances: Sequence[Dict]) -> Dict[str, torch.Tensor]:
        pad = self.tokenizer.pad_id
        lead, src, tgt = _encode_pair(self.tokenizer, [ex["input"] for ex in instances],
                                      [ex["output"] for ex in instances], self.source_max_len,
                                      self.target_max_len)
        ids, weights = [], []
        for n_src, n_tgt, s_ids, t_ids in zip(src["length"], tgt["length"], src["input_ids"],
                                              tgt["input_ids"]):
            real = n_tgt - lead
            t_ids = t_ids[lead:]
            n_pad = len(s_ids) - n_src
            row = (s_ids + t_ids)[n_pad:] + [pad] * n_pad
            w = ([0] * n_src + _step_weights(real, self.train_on_every_token)
                 + [0] * (len(t_ids) - real + n_pad))
            if self.total_max_len is not None:
                row, w = row[:self.total_max_len], w[:self.total_max_len]
            ids.append(torch.tensor(row))
            weights.append(torch.tensor(w))
        input_ids = pad_sequence(ids, batch_first=True, padding_value=pad)
        labels = torch.tensor([ex["label"] for ex in instances]).view(-1, 1)
        return {"input_ids": input_ids, "attention_mask": input_ids.ne(pad),
                "weights": pad_sequence(weights, batch_first=True, padding_value=0).float(),
                "labels": labels.repeat(1, input_ids.shape[1]).contiguous()}


@dataclass
class DataCollatorForPointwiseRewardModelingV2:
    """Multi-step examples: ``output`` and ``label`` are `` ;;; ``-joined lists."""
    tokenizer: object
    source_max_len: int
    target_max_len: int
    total_max_len: int
    train_on_every_token: bool

    def __call__(self, instances: Sequence[Dict]) -> Dict[str, torch.Tensor]:
        pad = self.tokenizer.pad_id
        steps = [ex["output"].split(SPLITTER) for ex in instances]
        step_labels = [[int(x) for x in ex["label"].split(SPLITTER)] for ex in instances]
        flat = [s for ss in steps for s in ss]
        lead, src, tgt = _encode_pair(self.tokenizer, [ex["input"] for ex in instances], flat,
                                      self.source_max_len, self.target_max_len)
        ids, weights, labels = [], [], []
        cursor = 0
        for i, (n_src, s_ids) in enumerate(zip(src["length"], src["input_ids"])):
            row = s_ids[len(s_ids) - n_src:]
            w, lab = [0] * n_src, [0] * n_src
            for k, step_label in enumerate(step_labels[i][:len(steps[i])]):
                n_tgt = tgt["length"][cursor + k]
                piece = tgt["input_ids"][cursor + k][lead:n_tgt]
                row = row + piece
                w += _step_weights(len(piece), self.train_on_every_token)
                lab += [step_label] * len(piece)
            cursor += len(steps[i])
            if self.total_max_len is not None:
                row, w, lab = (x[:self.total_max_len] for x in (row, w, lab))
                fill = self.total_max_len - len(row)
                row, w, lab = row + [pad] * fill, w + [0] * fill, lab + [0] * fill
            assert len(row) == len(w) == len(lab)
            ids.append(torch.tensor(row))
            weights.append(torch.tensor(w))
            labels.append(torch.tensor(lab))
        input_ids = pad_sequence(ids, batch_first=True, padding_value=pad)
        return {"input_ids": input_ids, "attention_mask": input_ids.ne(pad),
                "weights": pad_sequence(weights, batch_first=True, padding_value=0).float(),
                "labels": pad_sequence(labels, batch_first=True, padding_value=0).long()}


def extract_prm_dataset(example):
    if example["output_prefix"] == "":
        out = {"input": "Question: " + example["input"],
               "output": "\n\nAnswer: " + example["output"]}
    else:
        out = {"input": "Question: " + example["input"] + "\n\nAnswer: "
               + example["output_prefix"], "output": example["output"]}
    out["label"] = example["label"]
    return out


def extract_prm_v2_dataset(example):
    head = "# Question\n\n" + example["input"] + "\n\n# Solution"
    if example["output_prefix"] == "":
        out = {"input": head, "output": "\n\n" + example["output"]}
    else:
        out = {"input": head + "\n\n" + example["output_prefix"], "output": example["output"]}
    out["label"] = example["label"]
    return out


def extract_prm_v3_dataset(example):
    head = "# Question\n\n" + example["input"] + "\n\n# Solution\n\n"
    return {"input": head + (example["output_prefix"] or ""), "output": example["output"],
            "label": example["label"]}


def extract_prm_v4_dataset(example):
    steps = [s + "\n\n" for s in example["output"][:-1]] + [example["output"][-1]]
    assert len(steps) == len(example["label"])
    assert all(SPLITTER not in s for s in steps)
    head = "# Question\n\n" + example["input"] + "\n\n# Solution\n\n"
    if example.get("output_prefix") is not None:
        head += example["output_prefix"]
    return {"input": head, "output": SPLITTER.join(steps),
            "label": SPLITTER.join(str(x) for x in example["label"])}


_EXTRACTORS = {"prm": extract_prm_dataset, "prm-v2": extract_prm_v2_dataset,
               "prm-v3": extract_prm_v3_dataset, "prm-v4": extract_prm_v4_dataset}


def split_and_cap(dataset, args):
    """Shared train / eval selection of the data modules."""
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
    return train_dataset, eval_dataset


def make_pointwise_reward_modeling_data_module(tokenizer, args) -> Dict:
    if not os.path.exists(args.dataset):
        raise NotImplementedError(f"Dataset {args.dataset} not implemented yet.")
    try:
        dataset = utils.local_dataset(args.dataset)
    except Exception as e:
        raise ValueError(f"Error loading dataset from {args.dataset}") from e
    if args.dataset_format not in _EXTRACTORS:
        raise ValueError(f"Unsupported dataset format: {args.dataset_format}")
    dataset = dataset.map(_EXTRACTORS[args.dataset_format])
    keep = {"input", "output", "label"}
    dataset = dataset.remove_columns([c for c in dataset.column_names["train"] if c not in keep])
    train_dataset, eval_dataset = split_and_cap(dataset, args)
    cls = (DataCollatorForPointwiseRewardModelingV2 if args.dataset_format == "prm-v4"
           else DataCollatorForPointwiseRewardModeling)
    collator = cls(tokenizer, args.source_max_len, args.target_max_len, args.total_max_len,
                   args.train_on_every_token)
    return dict(train_dataset=train_dataset, eval_dataset=eval_dataset, data_collator=collator)
