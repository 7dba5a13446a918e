"""Tokenizers: a protocol, a byte-level tokenizer for tests, and an adapter over a
HuggingFace ``tokenizers`` file.

Parity: reference ``src/tilerl/tokenizer.py`` (protocol, ``ByteTokenizer``, HF adapter).
"""
from __future__ import annotations

from typing import List, Optional, Protocol, Sequence


class Tokenizer(Protocol):
    eos_id: Optional[int]
    vocab_size: int

    def encode(self, text: str) -> List[int]: ...

    def decode(self, ids: Sequence[int]) -> str: ...


class ByteTokenizer:
    """One token per UTF-8 byte, plus a few named specials above 255 so chat templates,
    ``<think>`` handling and stop tokens can be exercised without a vocabulary file."""

    SPECIALS = ("<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>",
                "<|endoftext|>")

    def __init__(self, vocab_size: int = 320):
        self.vocab_size = vocab_size
        self.special_ids = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.id_special = {v: k for k, v in self.special_ids.items()}
        self.eos_id = self.special_ids["<|im_end|>"]
        self.think_ids = (self.special_ids["<think>"], self.special_ids["</think>"])

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        i = 0
        while i < len(text):
            for s, sid in self.special_ids.items():
                if text.startswith(s, i):
                    out.append(sid)
                    i += len(s)
                    break
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def decode(self, ids: Sequence[int]) -> str:
        parts: List[str] = []
        buf = bytearray()
        for t in ids:
            t = int(t)
            if t < 256:
                buf.append(t)
                continue
            if buf:
                parts.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
            parts.append(self.id_special.get(t, ""))
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)


class HFTokenizer:
    """Adapter over a ``tokenizer.json`` (HuggingFace ``tokenizers``)."""

    def __init__(self, path: str):
        from tokenizers import Tokenizer as _T
        import os
        f = path if path.endswith(".json") else os.path.join(path, "tokenizer.json")
        self.tok = _T.from_file(f)
        self.vocab_size = self.tok.get_vocab_size()
        self.eos_id = None
        for name in ("<|im_end|>", "<|endoftext|>", "</s>"):
            i = self.tok.token_to_id(name)
            if i is not None:
                self.eos_id = i
                break
        a, b = self.tok.token_to_id("<think>"), self.tok.token_to_id("</think>")
        self.think_ids = (a, b) if a is not None and b is not None else None

    def encode(self, text: str) -> List[int]:
        return self.tok.encode(text, add_special_tokens=False).ids

    def decode(self, ids: Sequence[int]) -> str:
        return self.tok.decode([int(i) for i in ids], skip_special_tokens=False)


def load_tokenizer(path: Optional[str], vocab_size: int = 320):
    if path:
        return HFTokenizer(path)
    return ByteTokenizer(vocab_size)
