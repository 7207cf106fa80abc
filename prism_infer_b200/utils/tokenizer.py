"""Tokenizer loading.  A checkpoint directory with tokenizer files uses Hugging Face
``AutoTokenizer``; random-init models (no files) use ``IdTokenizer``, which maps text made
of integers to those ids and hashes any other word into the non-special vocabulary, so the
public text API works offline with synthetic weights."""

from __future__ import annotations

import os
import zlib
from typing import Sequence


class IdTokenizer:
    def __init__(self, vocab_size: int, reserved: Sequence[int] = (), eos_token_id: int | None = None) -> None:
        self.vocab_size = vocab_size
        self.reserved = set(int(r) for r in reserved)
        self.eos_token_id = eos_token_id
        self._usable = min([vocab_size] + [r for r in self.reserved]) if self.reserved else vocab_size

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        out = []
        for word in text.split():
            if word.lstrip("-").isdigit() and 0 <= int(word) < self.vocab_size:
                out.append(int(word))
            else:
                out.append(zlib.crc32(word.encode("utf-8")) % max(1, self._usable))
        return out or [0]

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return " ".join(str(int(i)) for i in ids if not (skip_special_tokens and int(i) in self.reserved))

    def __call__(self, text: str, **_: object) -> dict[str, list[int]]:
        return {"input_ids": self.encode(text)}


def load_tokenizer(model: str, arch) -> object:
    if not model.startswith("random:") and any(
        os.path.exists(os.path.join(model, f)) for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json")
    ):
        from transformers import AutoTokenizer

        return AutoTokenizer.from_pretrained(model, use_fast=True)
    reserved = (arch.image_token_id, arch.video_token_id, arch.vision_start_token_id, arch.vision_end_token_id,
                arch.eos_token_id)
    return IdTokenizer(arch.text.vocab_size, reserved, arch.eos_token_id)
