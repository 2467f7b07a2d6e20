"""RL (PPO) prompt data (reference: data_utils/data_utils_ppo.py:31-214).

``QueryDataset`` holds left-padded prompt token ids (prompts longer than ``source_max_len`` are
dropped) and, per prompt, the tokenised string ``"{answer} ;;; {gt_answer} ;;; {level}"`` that
the trainer decodes again for symbolic outcome grading."""
from __future__ import annotations

import logging
import os
from typing import Dict

import torch
from torch.utils.data import Dataset

from ..trainers import common_utils as utils

logger = logging.getLogger(__name__)


class QueryDataset(Dataset):
    def __init__(self, dataset, tokenizer, query_len: int):
        super().__init__()
        records = dataset.to_pandas().to_dict("records") if hasattr(dataset, "to_pandas") \
            else list(dataset)
        pad = tokenizer.pad_id

        def enc(text):
            return torch.tensor(tokenizer(text, truncation=False)["input_ids"][0])

        pairs = []
        for rec in records:
            q = enc(rec["input"])
            if len(q) <= query_len:
                pairs.append((q, enc(f"{rec['answer']} ;;; {rec['gt_answer']} ;;; "
                                     f"{rec['level']}")))
        logger.warning("Filtered out %d instances out of %d that exceed length limit.",
                       len(records) - len(pairs), len(records))
        assert pairs, "no prompt fits into source_max_len"
        self.queries = torch.stack([utils.left_pad(q, (query_len,), value=pad)
                                    for q, _ in pairs])
        width = max(len(a) for _, a in pairs)
        self.answers = torch.stack([utils.left_pad(a, (width,), value=pad) for _, a in pairs])
        self.query_attn_masks = self.queries.ne(pad).long()
        self.list_dict_data = records

    def __getitem__(self, i):
        return dict(queries=self.queries[i], query_attn_masks=self.query_attn_masks[i],
                    answers=self.answers[i])

    def __len__(self):
        return len(self.queries)


def _load(name: str):
    if not os.path.exists(name):
        raise NotImplementedError(f"Dataset {name} not implemented yet.")
    try:
        ds = utils.local_dataset(name)
    except Exception as e:
        raise ValueError(f"Error loading dataset from {name}") from e
    keep = {"input", "answer", "gt_answer", "level"}
    return ds.remove_columns([c for c in ds.column_names["train"] if c not in keep])


def make_rl_data_module(tokenizer, args) -> Dict:
    dataset = _load(args.dataset)
    eval_dataset = test_dataset = None
    if args.do_eval:
        if args.eval_dataset is not None:
            eval_dataset = _load(args.eval_dataset)["train"]
        else:
            print("Splitting train dataset in train and validation according to "
                  "`eval_dataset_size`")
            dataset = dataset["train"].train_test_split(test_size=args.eval_dataset_size,
                                                        shuffle=True, seed=42)
            eval_dataset = dataset["test"]
        if args.max_eval_samples is not None and len(eval_dataset) > args.max_eval_samples:
            eval_dataset = eval_dataset.select(range(args.max_eval_samples))
    if args.do_test:
        if args.test_dataset is None:
            raise NotImplementedError("Must specify test dataset if `do_test` is True.")
        test_dataset = _load(args.test_dataset)["train"]
    train_dataset = dataset["train"]
    if args.max_train_samples is not None and len(train_dataset) > args.max_train_samples:
        train_dataset = train_dataset.select(range(args.max_train_samples))

    def wrap(ds):
        return None if ds is None else QueryDataset(ds, tokenizer, args.source_max_len)

    return dict(train_dataset=wrap(train_dataset), eval_dataset=wrap(eval_dataset),
                test_dataset=wrap(test_dataset),
                data_collator=utils.DataCollatorForStackableDataset())
