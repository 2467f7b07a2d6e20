"""DPO preference data (reference: data_utils/data_utils_dpo.py:29-165): every pair is
re-ordered into (winner, loser) by ``preference`` in {1, 2}, each side goes through the SFT
preprocessing, and optional ``is_eos_{1,2}`` / ``win_rate_{1,2}`` columns follow their side."""
from __future__ import annotations

from typing import Dict

import torch
from torch.utils.data import Dataset

from ..trainers import common_utils as utils
from .data_utils_sft import extract_alpaca_dataset, preprocess_for_sft


def preprocess_for_dpo(args, dataset, tokenizer, reorder_wl: bool = True) -> Dict[str, torch.Tensor]:
    records = dataset.to_pandas().to_dict("records") if hasattr(dataset, "to_pandas") \
        else list(dataset)
    extras = [k for k in ("is_eos", "win_rate") if records and f"{k}_1" in records[0]]

    def side(rec, want_winner: bool):
        first = (rec["preference"] == 1) if reorder_wl else True
        take_1 = first if want_winner else not first
        sfx = "1" if take_1 else "2"
        out = {k: rec[k] for k in ("instruction", "input") if k in rec}
        out["output"] = rec[f"output_{sfx}"]
        for k in extras:
            out[k] = rec[f"{k}_{sfx}"]
        if args.dataset_format == "alpaca":
            out.update(extract_alpaca_dataset(out))
        elif args.dataset_format is not None:
            raise ValueError(f"Unknown dataset format: {args.dataset_format}")
        return out

    def encode(rows):
        return preprocess_for_sft(rows, tokenizer, args.source_max_len, args.target_max_len,
                                  args.total_max_len, args.train_on_source,
                                  args.add_eos_to_target, args.add_eos_to_marked_target,
                                  return_win_rate=True)

    tw = encode([side(r, True) for r in records])
    tl = encode([side(r, False) for r in records])
    return dict(input_ids_w=tw["input_ids"], labels_w=tw["labels"], win_rate_w=tw["win_rate"],
                input_ids_l=tl["input_ids"], labels_l=tl["labels"], win_rate_l=tl["win_rate"])


class DPODataset(Dataset):
    def __init__(self, args, dataset, tokenizer):
        super().__init__()
        self.tensors = preprocess_for_dpo(args, dataset, tokenizer)

    def __len__(self):
        return len(next(iter(self.tensors.values())))

    def __getitem__(self, i) -> Dict[str, torch.Tensor]:
        return {k: v[i] for k, v in self.tensors.items()}


def make_dpo_data_module(tokenizer, args) -> dict:
    train = utils.local_dataset(args.dataset)["train"]
    train_dataset = DPODataset(args, train, tokenizer)
    eval_dataset = None
    if args.eval_size > 0:
        train_dataset, eval_dataset = utils.split_train_into_train_and_eval(
            train_dataset, args.eval_size, args.seed)
    return dict(train_dataset=train_dataset, eval_dataset=eval_dataset,
                data_collator=utils.DataCollatorForStackableDataset())
