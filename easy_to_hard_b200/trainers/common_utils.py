"""Small helpers shared by the trainers and data modules (API of the reference's
trainers/common_utils.py:38-254): sequence / dict utilities, tensor padding, seeding, an
endless data loader, the local-JSON dataset loader."""
from __future__ import annotations

import logging
import os
import random
import tempfile
from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.utils.data import DataLoader, Dataset, random_split


def alleq(items: Sequence, same: Callable = lambda a, b: a == b) -> bool:
    """True when every element equals the first under ``same``."""
    return all(same(items[0], other) for other in items[1:])


def zip_(*seqs: Sequence):
    """``zip`` that insists on equal lengths."""
    if not seqs:
        return []
    assert alleq(seqs, lambda a, b: len(a) == len(b)), "sequences differ in length"
    return zip(*seqs)


def mean(*seqs):
    vals = [float(np.mean(s)) for s in seqs]
    return vals[0] if len(vals) == 1 else vals


def flatten_dict(nested: dict, sep: str = ".", postprocess_fn: Callable = lambda *a: a) -> dict:
    """{"a": {"b": 1}} -> {"a.b": postprocess_fn(1)}."""
    flat = {}
    stack = [("", nested)]
    while stack:
        prefix, node = stack.pop()
        for key, val in node.items():
            if sep in key:
                raise ValueError(f"separator '{sep}' not allowed to be in key '{key}'")
            if isinstance(val, dict):
                stack.append((prefix + key + sep, val))
            else:
                flat[prefix + key] = postprocess_fn(val)
    return flat


def unpack_dict(d: Dict, keys: Sequence[str], return_type: type = tuple):
    if return_type in (tuple, list):
        return return_type(d[k] for k in keys)
    if return_type is dict:
        return {k: d[k] for k in keys}
    raise ValueError(f"Unknown return_type: {return_type}")


def merge_dict(dicts: Sequence[dict], merge_fn: Callable = lambda *a: a) -> dict:
    """Dicts with the same keys -> one dict of merged value lists."""
    if not dicts:
        return {}
    return {k: merge_fn([d[k] for d in dicts]) for k in dicts[0]}


def prepare_inputs(data, device):
    """Move every tensor of a (nested) container to ``device``."""
    if isinstance(data, Mapping):
        return type(data)({k: prepare_inputs(v, device) for k, v in data.items()})
    if isinstance(data, (tuple, list)):
        return type(data)(prepare_inputs(v, device) for v in data)
    if torch.is_tensor(data):
        return data.to(device)
    return data


def pad_inputs_on_batch(data: Sequence[torch.Tensor], per_device_batch_size: int):
    """Repeat row 0 until the batch is a multiple of ``per_device_batch_size``."""
    n = data[0].size(0)
    extra = (-n) % per_device_batch_size
    out = []
    for t in data:
        assert t.size(0) == n
        if extra:
            t = torch.cat([t, t[:1].expand(extra, *t.shape[1:])], dim=0)
        out.append(t)
    return out


def pad(inputs: torch.Tensor, target_size, value=0.0, left: bool = True) -> torch.Tensor:
    spec = []
    for want, have in reversed(list(zip_(target_size, inputs.size()))):
        gap = want - have
        spec += [gap, 0] if left else [0, gap]
    return F.pad(inputs, pad=spec, value=value)


def left_pad(inputs, target_size, value=0.0):
    return pad(inputs, target_size, value, left=True)


def right_pad(inputs, target_size, value=0.0):
    return pad(inputs, target_size, value, left=False)


def manual_seed(args_or_seed, fix_cudnn: bool = False) -> None:
    seed = getattr(args_or_seed, "seed", args_or_seed)
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    os.environ["PYTHONHASHSEED"] = str(seed)
    if fix_cudnn:
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False


class InfiniteLoader:
    """Iterates a DataLoader forever, bumping the sampler's epoch on every wrap-around."""

    def __init__(self, loader: DataLoader):
        self.loader, self.epoch = loader, 0
        self._it = iter(loader)

    def __iter__(self):
        return self

    def __next__(self):
        try:
            return next(self._it)
        except StopIteration:
            self.epoch += 1
            sampler = getattr(self.loader, "sampler", None)
            if dist.is_initialized() and hasattr(sampler, "set_epoch"):
                sampler.set_epoch(self.epoch)
            self._it = iter(self.loader)
            return next(self._it)


class DisableLogger:
    def __enter__(self):
        logging.disable(logging.CRITICAL)

    def __exit__(self, *exc):
        logging.disable(logging.NOTSET)


@dataclass
class DataCollatorForStackableDataset:
    def __call__(self, instances: Sequence[Dict]) -> Dict[str, torch.Tensor]:
        return {k: torch.stack([inst[k] for inst in instances]) for k in instances[0]}


def local_dataset(dataset_name: str):
    """Load a local ``.json`` file as a Hugging Face ``DatasetDict`` with a ``train`` split."""
    if not dataset_name.endswith(".json"):
        raise ValueError(f"Unsupported dataset format: {dataset_name}")
    from datasets import load_dataset
    cache = os.path.join(tempfile.gettempdir(), f"{os.getuid()}_cache", "huggingface", "datasets")
    return load_dataset("json", data_files=dataset_name, cache_dir=cache)


def split_train_into_train_and_eval(train_dataset: Dataset, eval_size: int,
                                    seed: int) -> Tuple[Dataset, Dataset]:
    assert eval_size < len(train_dataset), \
        "Requested eval_size cannot be equal/larger than original train data size."
    gen = torch.Generator().manual_seed(seed)
    return tuple(random_split(train_dataset, [len(train_dataset) - eval_size, eval_size],
                              generator=gen))
