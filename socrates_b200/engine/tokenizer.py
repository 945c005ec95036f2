"""A stand-in tokenizer for models with random weights.

It offers the part of the tokenizer surface that the engine uses (the same part the
reference's test stub offers, tests/tiny.py:41-55): `all_special_ids`,
`apply_chat_template`, calling it on text, and `decode`.  Text becomes one id per
UTF-8 byte, folded into the vocabulary; id 0 is the only special id.
"""

from __future__ import annotations

from typing import List


class ByteTokenizer:
    all_special_ids = [0]

    def __init__(self, vocab_size: int):
        if vocab_size < 2:
            raise ValueError("a vocabulary of at least 2 ids is needed")
        self.vocab_size = vocab_size

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True,
                            enable_thinking=False) -> str:
        return messages[0]["content"]

    def encode(self, text: str) -> List[int]:
        return [1 + (b % (self.vocab_size - 1)) for b in text.encode("utf-8")] or [1]

    def __call__(self, text: str, return_tensors=None):
        from types import SimpleNamespace
        ids = self.encode(text)
        if return_tensors == "pt":
            import torch
            return SimpleNamespace(input_ids=torch.tensor([ids], dtype=torch.long))
        return SimpleNamespace(input_ids=[ids])

    def decode(self, ids) -> str:
        return " ".join(str(int(i)) for i in ids)
