"""Tokenizer front-end with the calling convention of the reference's ``AcceleraTokenizer``
(models/tokenizer_utils.py:251-610): SentencePiece ``tokenizer.model`` files (LLaMA family:
pad=-1, unk=0, bos=1, eos=2) or a Hugging Face tokenizer directory (deepseek-math), ids clamped
below the model's vocabulary size, left/right padding and truncation, ``marked_eos`` per-sample
EOS control, and ``batch_encode_tokens`` which builds the left-padded prompt tensor plus
``left_pad_mask_pos`` of batched generation.

``ByteTokenizer`` is a dependency-free stand-in (UTF-8 bytes + specials) used by tests and by
the synthetic end-to-end scripts when no tokenizer file exists.
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Union

import torch


class BatchEncoding(dict):
    """Dict of ``input_ids`` / ``attention_mask`` / ``length`` with attribute access and an
    optional conversion to tensors (``tensor_type="pt"``)."""

    def __init__(self, data: Optional[Dict[str, Any]] = None, tensor_type: Optional[str] = None):
        super().__init__(data or {})
        if tensor_type is not None:
            self.convert_to_tensors(tensor_type)

    def __getattr__(self, item):
        try:
            return self[item]
        except KeyError as e:
            raise AttributeError(item) from e

    def convert_to_tensors(self, tensor_type: str = "pt") -> "BatchEncoding":
        if str(tensor_type).lower() not in ("pt", "tensortype.pytorch"):
            raise ValueError(f"only PyTorch tensors are supported, got {tensor_type!r}")
        for k, v in list(self.items()):
            if not torch.is_tensor(v):
                try:
                    self[k] = torch.tensor(v)
                except (ValueError, TypeError) as e:
                    raise ValueError(
                        f"cannot build a tensor for {k!r}: sequences of different length need "
                        "padding=True/'max_length' and/or truncation") from e
        return self

    def to(self, device) -> "BatchEncoding":
        for k, v in list(self.items()):
            if torch.is_tensor(v):
                self[k] = v.to(device)
        return self


class ByteTokenizer:
    """UTF-8 byte-level tokenizer: ids 0..3 are unk/bos/eos/newline-free specials, byte b maps
    to id b + 4. Mirrors the small part of the SentencePiece API that AcceleraTokenizer uses."""

    def __init__(self, vocab_size: int = 260):
        self._vocab = max(vocab_size, 260)

    def vocab_size(self):
        return self._vocab

    get_piece_size = vocab_size

    def bos_id(self):
        return 1

    def eos_id(self):
        return 2

    def pad_id(self):
        return -1

    def unk_id(self):
        return 0

    def encode(self, s):
        if isinstance(s, (list, tuple)):
            return [self.encode(x) for x in s]
        return [b + 4 for b in s.encode("utf-8")]

    def decode(self, ids):
        return bytes(i - 4 for i in ids if 4 <= i < 260).decode("utf-8", errors="replace")


class AcceleraTokenizer:
    def __init__(self, tokenizer: Union[str, Path, Any] = None, model_vocab_size: int = 32000):
        self.hf_model = None
        self.sp_model = None
        if isinstance(tokenizer, (str, Path)) and str(tokenizer).endswith(".model"):
            from sentencepiece import SentencePieceProcessor
            tokenizer = SentencePieceProcessor(model_file=str(tokenizer))
        if hasattr(tokenizer, "bos_id") and callable(tokenizer.bos_id):
            sp = tokenizer
            self.sp_model = sp
            self.model_vocab_size = model_vocab_size
            self.n_words = sp.vocab_size()
            self.bos_id, self.eos_id = sp.bos_id(), sp.eos_id()
            self.pad_id, self.unk_id = sp.pad_id(), sp.unk_id()
            self.bos_token, self.eos_token = "<s>", "</s>"
        else:
            from transformers import AutoTokenizer
            hf = AutoTokenizer.from_pretrained(str(tokenizer))
            self.hf_model = hf
            if hf.pad_token_id is None or hf.unk_token_id is None:
                hf.add_special_tokens({"pad_token": "<pad>", "unk_token": "<unk>"})
            # deepseek-math: 100000 base entries + bos/eos + the two added specials
            self.model_vocab_size = max(model_vocab_size, len(hf))
            self.n_words = self.model_vocab_size
            self.bos_id, self.eos_id = hf.bos_token_id, hf.eos_token_id
            self.pad_id, self.unk_id = hf.pad_token_id, hf.unk_token_id
            self.bos_token, self.eos_token = hf.bos_token, hf.eos_token
        self.pad_token, self.unk_token = "<pad>", "<unk>"

    # ------------------------------------------------------------------ encoding
    def _clamp(self, ids: List[int]) -> List[int]:
        top = self.model_vocab_size - 1
        return [i if i <= top else top for i in ids]

    def encode(self, s: str, bos: bool, eos: bool) -> List[int]:
        assert isinstance(s, str)
        ids = (self.sp_model.encode(s) if self.sp_model is not None
               else self.hf_model.encode(s, add_special_tokens=False))
        ids = ([self.bos_id] if bos else []) + list(ids) + ([self.eos_id] if eos else [])
        return self._clamp(ids)

    def batch_encode(self, batch_s: Sequence[str], bos: Sequence[bool], eos: Sequence[bool]):
        assert len(batch_s) == len(bos) == len(eos)
        if self.sp_model is not None:
            raw = self.sp_model.encode(list(batch_s))
        else:
            raw = self.hf_model(list(batch_s), add_special_tokens=False)["input_ids"]
        out = []
        for ids, b, e in zip(raw, bos, eos):
            out.append(self._clamp(([self.bos_id] if b else []) + list(ids)
                                   + ([self.eos_id] if e else [])))
        return out

    def __call__(self, text=None, add_bos: bool = True, add_eos: bool = False,
                 marked_eos: Optional[List[bool]] = None, padding: Union[bool, str] = False,
                 truncation: bool = False, max_length: Optional[int] = None,
                 return_tensors: Optional[str] = None, padding_side: str = "right",
                 truncation_side: str = "right") -> BatchEncoding:
        if not isinstance(text, (list, tuple)):
            ids = self.encode(text, bos=add_bos, eos=add_eos)
            return BatchEncoding({"input_ids": [ids], "attention_mask": [[1] * len(ids)],
                                  "length": [len(ids)]}, tensor_type=return_tensors)
        n = len(text)
        eos_flags = [add_eos] * n if marked_eos is None else list(marked_eos)
        assert len(eos_flags) == n
        seqs = self.batch_encode(text, [add_bos] * n, eos_flags)
        if truncation:
            if truncation_side not in ("left", "right"):
                raise ValueError(f"Invalid truncation side: {truncation_side}")
            seqs = [s[-max_length:] if truncation_side == "left" else s[:max_length]
                    for s in seqs]
        lengths = [len(s) for s in seqs]
        if padding is True or padding == "longest":
            width = max(lengths)
        elif padding == "max_length":
            assert max_length is not None
            width = max_length
        else:
            width = None
        masks = [[1] * n_ for n_ in lengths]
        if width is not None:
            if padding_side not in ("left", "right"):
                raise ValueError(f"Invalid padding side: {padding_side}")
            left = padding_side == "left"
            for i, (s, m) in enumerate(zip(seqs, masks)):
                fill = max(width - len(s), 0)
                seqs[i] = [self.pad_id] * fill + s if left else s + [self.pad_id] * fill
                masks[i] = [0] * fill + m if left else m + [0] * fill
        return BatchEncoding({"input_ids": seqs, "attention_mask": masks, "length": lengths},
                             tensor_type=return_tensors)

    # ------------------------------------------------------------------ decoding
    def decode(self, t, skip_special_tokens: bool = True) -> str:
        if torch.is_tensor(t):
            t = t.tolist()
        t = [x for x in t if x != self.pad_id]
        if self.sp_model is None:
            return self.hf_model.decode(t, skip_special_tokens=skip_special_tokens)
        return self.sp_convert_tokens_to_string(t, skip_special_tokens=skip_special_tokens)

    def sp_convert_tokens_to_string(self, tokens, skip_special_tokens: bool = False) -> str:
        """Decode with SentencePiece, rendering (or dropping) the special ids ourselves."""
        names = {self.bos_id: self.bos_token, self.eos_id: self.eos_token,
                 self.pad_id: self.pad_token}
        if self.unk_id != self.pad_id:
            names[self.unk_id] = self.unk_token
        pieces, run = [], []
        n_pieces = self.sp_model.get_piece_size()
        for tok in tokens:
            if tok >= n_pieces or tok < 0:
                # the model's vocabulary may be padded beyond the tokenizer's (Llemma: 32016
                # rows for 32000 pieces); such ids decode to nothing instead of raising
                continue
            if tok in names:
                if not skip_special_tokens:
                    pieces.append(self.sp_model.decode(run) + names[tok])
                    run = []
            else:
                run.append(tok)
        if run:
            pieces.append(self.sp_model.decode(run))
        return "".join(pieces)

    def batch_decode(self, sequences, skip_special_tokens: bool = False, **kwargs) -> List[str]:
        if torch.is_tensor(sequences):
            sequences = sequences.tolist()
        if self.sp_model is None:
            return self.hf_model.batch_decode(sequences, skip_special_tokens=skip_special_tokens,
                                              **kwargs)
        return [self.decode(s, skip_special_tokens=skip_special_tokens) for s in sequences]


def batch_encode_tokens(tokenizer: AcceleraTokenizer, strings: List[str], bos: bool = True,
                        eos: bool = False, device="cuda", padding_side: str = "left"):
    """Left padding returns ``(ids int32 [B, T], left_pad_mask_pos int32 [B] or None)``; right
    padding returns the ids only. Pad id falls back to unk when the tokenizer has none."""
    assert padding_side in ("left", "right")
    rows = [tokenizer.encode(s, bos=bos, eos=eos) for s in strings]
    width = max(len(r) for r in rows)
    pad = tokenizer.pad_id if tokenizer.pad_id >= 0 else tokenizer.unk_id
    fills = [width - len(r) for r in rows]
    if padding_side == "left":
        ids = torch.tensor([[pad] * f + r for f, r in zip(fills, rows)], dtype=torch.int,
                           device=device)
        if not any(fills):
            return ids, None
        return ids, torch.tensor(fills, dtype=torch.int, device=device)
    return torch.tensor([r + [pad] * f for f, r in zip(fills, rows)], dtype=torch.int,
                        device=device)
