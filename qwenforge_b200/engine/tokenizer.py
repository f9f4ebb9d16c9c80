"""Text in and out of the engine. The model library works on token ids; strings are a convenience of
the entry point, as in the reference (student_engine.py:365-374, :1218-1239, :1373-1378).

A model folder with tokenizer files gets its own tokenizer (through the `transformers` tokenizer
loader the reference uses, which is not model code). A folder without them (random weights) gets a
byte tokenizer: UTF-8 bytes are token ids, so any text round-trips for vocabularies of at least 256."""
from __future__ import annotations

from pathlib import Path
from typing import Optional, Sequence


class ByteTokenizer:
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    def __init__(self, vocab_size: int):
        self.vocab_size = vocab_size

    def encode_prompt(self, text: str) -> list[int]:
        return [b % self.vocab_size for b in text.encode("utf-8")]

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(int(i) % 256 for i in ids).decode("latin-1")


class FolderTokenizer:
    """The folder's own tokenizer with its chat template (student_engine.py:1218-1225)."""

    def __init__(self, model_dir, local_files_only: bool):
        from transformers import AutoTokenizer  # tokenizer loader only; no model code is imported

        self.tok = AutoTokenizer.from_pretrained(str(model_dir), trust_remote_code=False,
                                                 local_files_only=local_files_only)
        self.bos_token_id = self.tok.bos_token_id
        self.eos_token_id = self.tok.eos_token_id

    def encode_prompt(self, text: str) -> list[int]:
        if getattr(self.tok, "chat_template", None):
            text = self.tok.apply_chat_template([{"role": "user", "content": text}], tokenize=False,
                                                add_generation_prompt=True)
        return list(self.tok(text, add_special_tokens=False)["input_ids"])

    def decode(self, ids: Sequence[int]) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=True)


def load_tokenizer(model_dir, vocab_size: int, local_files_only: bool = True):
    model_dir = Path(model_dir)
    if any((model_dir / name).exists() for name in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
        return FolderTokenizer(model_dir, local_files_only)
    return ByteTokenizer(vocab_size)
