"""Tokenizer wrapper with the Megatron-style surface the framework expects (``eod``, ``pad``,
``vocab_size``, ``tokenize`` / ``detokenize``) over a Hugging Face tokenizer, plus a tiny
vocabulary-free tokenizer for synthetic runs (ids in, ids out).
Reference: ``mindspeed_rl/utils/tokenizer.py:20-342``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence


class BaseTokenizer:
    name = "base"

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError

    def tokenize(self, text: str) -> List[int]:
        raise NotImplementedError

    def detokenize(self, ids: Sequence[int]) -> str:
        raise NotImplementedError

    @property
    def eod(self) -> Optional[int]:
        raise NotImplementedError

    @property
    def pad(self) -> Optional[int]:
        raise NotImplementedError


class HuggingFaceTokenizer(BaseTokenizer):
    """``pad`` defaults to ``eos`` when the model defines no pad token."""

    def __init__(self, tokenizer_name_or_path: str, prompt_type: Optional[str] = None,
                 prompt_type_path: Optional[str] = None, use_fast: bool = True, padding_side: str = "right",
                 trust_remote_code: bool = False, enable_thinking: bool = False, **kw):
        from transformers import AutoTokenizer

        self.tokenizer = AutoTokenizer.from_pretrained(tokenizer_name_or_path, use_fast=use_fast,
                                                       padding_side=padding_side,
                                                       trust_remote_code=trust_remote_code, **kw)
        self.name = "HuggingFaceTokenizer"
        self.template = None
        if prompt_type and prompt_type_path:
            from ..datasets.templates import fix_model_tokenizer

            self.template = fix_model_tokenizer(self.tokenizer, prompt_type.strip(), prompt_type_path.strip(),
                                                enable_thinking)
        if self.tokenizer.pad_token_id is None:
            self.tokenizer.pad_token = self.tokenizer.eos_token

    @property
    def vocab_size(self) -> int:
        return len(self.tokenizer)

    @property
    def vocab(self):
        return self.tokenizer.get_vocab()

    def tokenize(self, text: str, **kw) -> List[int]:
        return self.tokenizer.encode(text, **kw)

    def detokenize(self, ids, **kw) -> str:
        return self.tokenizer.decode(ids, **kw)

    def decode(self, ids, **kw) -> str:
        return self.tokenizer.decode(ids, **kw)

    def encode(self, text, **kw):
        return self.tokenizer.encode(text, **kw)

    @property
    def eod(self):
        return self.tokenizer.eos_token_id

    @property
    def eos_token_id(self):
        return self.tokenizer.eos_token_id

    @property
    def pad(self):
        return self.tokenizer.pad_token_id

    @property
    def pad_token_id(self):
        return self.tokenizer.pad_token_id

    @property
    def cls(self):
        return self.tokenizer.cls_token_id

    @property
    def sep(self):
        return self.tokenizer.sep_token_id

    @property
    def mask(self):
        return self.tokenizer.mask_token_id


class IdentityTokenizer(BaseTokenizer):
    """Token ids are their own text ("12 7 33"): used with synthetic prompts and rule rewards."""

    name = "IdentityTokenizer"

    def __init__(self, vocab_size: int, eos_token_id: Optional[int] = None, pad_token_id: int = 0):
        self._vocab = vocab_size
        self._eos = vocab_size - 1 if eos_token_id is None else eos_token_id
        self._pad = pad_token_id
        self.tokenizer = self

    @property
    def vocab_size(self) -> int:
        return self._vocab

    def __len__(self):
        return self._vocab

    def tokenize(self, text: str, **kw) -> List[int]:
        return [int(t) for t in text.split()]

    encode = tokenize

    def detokenize(self, ids, skip_special_tokens: bool = False, **kw) -> str:
        ids = [int(i) for i in ids]
        if skip_special_tokens:
            ids = [i for i in ids if i not in (self._eos, self._pad)]
        return " ".join(str(i) for i in ids)

    decode = detokenize

    @property
    def eod(self):
        return self._eos

    eos_token_id = eod

    @property
    def pad(self):
        return self._pad

    pad_token_id = pad
    bos_token_id = None

    def convert_tokens_to_ids(self, token):
        return int(token)


def get_tokenizer(tokenizer_model: str, tokenizer_type: str = "HuggingFaceTokenizer", prompt_type=None,
                  prompt_type_path=None, eos_token_id=None, pad_token_id=None, vocab_size=None, **kw):
    """Factory used by the CLIs (``tokenizer_type: PretrainedFromHF | HuggingFaceTokenizer | Identity``)."""
    if tokenizer_type in ("Identity", "IdentityTokenizer", "NullTokenizer"):
        return IdentityTokenizer(vocab_size or 32000, eos_token_id, pad_token_id or 0)
    return HuggingFaceTokenizer(tokenizer_model, prompt_type, prompt_type_path, **kw)
