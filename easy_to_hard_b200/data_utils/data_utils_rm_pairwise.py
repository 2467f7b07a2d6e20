"""Pairwise reward-model data (reference: data_utils/data_utils_rm_pairwise.py:53-239):
``input_ids`` ``[N, 2, seq]`` right-padded (bos + prompt + output_k [+ eos]) and ``choice``
``[N, 1]`` with preference 1 -> 0 and 2 -> 1 (1 means output_2 is preferred)."""
from __future__ import annotations

import logging
from typing import Dict, Optional, Sequence

import torch
from torch.utils.data import Dataset

from ..trainers import common_utils as utils
from .data_utils_sft import ALPACA_PROMPT_DICT

logger = logging.getLogger(__name__)


def format_prompt(example: Dict[str, str], prompt_dict: Optional[Dict[str, str]]) -> str:
    if prompt_dict is None:
        return "{input}".format(**example)
    assert "instruction" in example, "Internal error: example missing required keys."
    key = "prompt_input" if example.get("input", "") != "" else "prompt_no_input"
    return prompt_dict[key].format(**example)


def format_output(example: dict, output_key: str = "output") -> str:
    return example[output_key]


def _tokenize_fn(strings: Sequence[str], tokenizer, max_length: int,
                 end_sequence_with_eos: bool) -> torch.Tensor:
    enc = tokenizer(list(strings), max_length=max_length, padding="max_length", truncation=True,
                    add_bos=True, add_eos=bool(end_sequence_with_eos), padding_side="right",
                    truncation_side="right")
    return torch.tensor(enc["input_ids"])


def preprocess_for_reward_modeling(data, tokenizer, end_sequence_with_eos: bool = False,
                                   max_length: Optional[int] = None,
                                   query_len: Optional[int] = None,
                                   response_len: Optional[int] = None,
                                   prompt_dict: Optional[Dict[str, str]] = None):
    records = data.to_pandas().to_dict("records") if hasattr(data, "to_pandas") else list(data)
    choice = torch.tensor([[{1: 0, 2: 1}[r["preference"]]] for r in records])
    if max_length is None:
        max_length = query_len + response_len
    logger.warning("Tokenizing %d pairs...", len(records))
    sides = [_tokenize_fn([format_prompt(r, prompt_dict) + format_output(r, key)
                           for r in records], tokenizer, max_length, end_sequence_with_eos)
             for key in ("output_1", "output_2")]
    return dict(input_ids=torch.stack(sides, dim=1), choice=choice,
                metadata=dict(mean_choice=choice.float().mean().item()))


class PairwiseRewardModelingDataset(Dataset):
    def __init__(self, data, tokenizer, end_sequence_with_eos: bool = False,
                 max_length: Optional[int] = None, query_len: Optional[int] = None,
                 response_len: Optional[int] = None, prompt_dict=None):
        super().__init__()
        d = preprocess_for_reward_modeling(data, tokenizer, end_sequence_with_eos, max_length,
                                           query_len, response_len, prompt_dict)
        self.input_ids, self.choice, self.metadata = d["input_ids"], d["choice"], d["metadata"]

    def __len__(self):
        return len(self.input_ids)

    def __getitem__(self, i) -> Dict[str, torch.Tensor]:
        return dict(input_ids=self.input_ids[i], choice=self.choice[i])


def make_pairwise_reward_modeling_data_module(tokenizer, args):
    train = utils.local_dataset(args.dataset)["train"]
    if args.dataset_format == "alpaca":
        prompt_dict = ALPACA_PROMPT_DICT
    elif args.dataset_format is None:
        prompt_dict = None
    else:
        raise ValueError(f"Unsupported dataset_format: {args.dataset_format}."
                         "Only alpaca and None are supported.")
    train_dataset = PairwiseRewardModelingDataset(
        train, tokenizer, end_sequence_with_eos=args.add_eos_to_target,
        max_length=args.total_max_len, query_len=args.source_max_len,
        response_len=args.target_max_len, prompt_dict=prompt_dict)
    eval_dataset = None
    if args.eval_size > 0:
        train_dataset, eval_dataset = utils.split_train_into_train_and_eval(
            train_dataset, args.eval_size, args.seed)
    return dict(train_dataset=train_dataset, eval_dataset=eval_dataset,
                data_collator=utils.DataCollatorForStackableDataset())
