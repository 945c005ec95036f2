"""Tokenizers for the entry point.

`load_tokenizer(model_dir, vocab)` gives what the engine turns text into ids with:

* a model folder that carries `tokenizer.json` (or `tokenizer_config.json`) is read with
  `transformers.AutoTokenizer`, offline, as the reference reads its checkpoint's
  tokenizer (model/inference_paged.py:67-70); prompts then go through its chat template
  and outputs are decoded to text (:139-143, 242-251);
* a folder without one (random weights) gets `ByteTokenizer`, which needs no files.

What the engine uses of either: `all_special_ids`, `apply_chat_template`, calling it on
text (`.input_ids`), `decode`, and `chat_template` (None: prompts are taken as they are).
"""

from __future__ import annotations

from pathlib import Path
from types import SimpleNamespace
from typing import List

TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json")


class ByteTokenizer:
    """Text as UTF-8 bytes: byte b is id b + 1, id 0 ends a text and is the only special id.

    With a vocabulary of at least 257 ids this is lossless and `decode` returns text (ids
    beyond the bytes print as <id>); a smaller vocabulary folds the bytes into 1..vocab-1
    and `decode` prints the ids."""

    all_special_ids = [0]
    chat_template = None              # a prompt is tokenised as it is

    def __init__(self, vocab_size: int):
        if vocab_size < 2:
            raise ValueError("a vocabulary of at least 2 ids is needed")
        self.vocab_size = vocab_size
        self.lossless = vocab_size >= 257

    def apply_chat_template(self, messages, **_) -> str:
        return "\n".join(m["content"] for m in messages)

    def encode(self, text: str) -> List[int]:
        raw = text.encode("utf-8") or b" "
        if self.lossless:
            return [b + 1 for b in raw]
        return [1 + b % (self.vocab_size - 1) for b in raw]

    def __call__(self, text: str, return_tensors=None):
        ids = self.encode(text)
        if return_tensors == "pt":
            import torch
            return SimpleNamespace(input_ids=torch.tensor([ids], dtype=torch.long))
        return SimpleNamespace(input_ids=ids)

    def decode(self, ids) -> str:
        ids = [int(i) for i in ids]
        if not self.lossless:
            return " ".join(str(i) for i in ids)
        out, run = [], bytearray()
        for i in ids:
            if 1 <= i <= 256:
                run.append(i - 1)
                continue
            if run:
                out.append(run.decode("utf-8", errors="replace"))
                run = bytearray()
            out.append(f"<{i}>")
        if run:
            out.append(run.decode("utf-8", errors="replace"))
        return "".join(out)


def encode_prompt(tok, prompt: str) -> List[int]:
    """Token ids of one user prompt: through the tokenizer's chat template where it has one
    (one user message, generation prompt added, thinking off, as the reference asks for it,
    model/inference_paged.py:139-143), then tokenised."""
    text = prompt
    if getattr(tok, "chat_template", "") is not None:        # None: the tokenizer has no template
        text = tok.apply_chat_template([{"role": "user", "content": prompt}], tokenize=False,
                                       add_generation_prompt=True, enable_thinking=False)
    got = tok(text).input_ids
    got = got.tolist() if hasattr(got, "tolist") else list(got)
    return [int(i) for i in (got[0] if got and isinstance(got[0], (list, tuple)) else got)]


def has_tokenizer_files(model_dir) -> bool:
    return any((Path(model_dir) / f).exists() for f in TOKENIZER_FILES)


def load_tokenizer(model_dir, vocab_size: int):
    """The folder's own tokenizer if it has one, else a ByteTokenizer over `vocab_size` ids."""
    if not has_tokenizer_files(model_dir):
        return ByteTokenizer(vocab_size)
    from transformers import AutoTokenizer          # tokenizer only; no model code of that package is used
    tok = AutoTokenizer.from_pretrained(str(model_dir), local_files_only=True)
    if len(tok) > vocab_size:
        raise ValueError(f"the tokenizer in {model_dir} has {len(tok)} ids, the model's vocabulary {vocab_size}")
    return tok
