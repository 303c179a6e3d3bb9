"""Tokenizers and the streaming UTF-8-safe detokenizer.

`HFTokenizer` wraps a Hugging Face `tokenizer.json` (the official checkpoint ships one); `ByteTokenizer` is a
self-contained byte-level tokenizer with the same special tokens, used by tests and by random-weight serving.
`StreamingDecoder` only releases text that ends on a complete UTF-8 sequence, so a multi-byte character split across
tokens is never emitted half-way (reference: rust/crates/ds41rt-loader/src/tokenizer.rs).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

SPECIALS = ["<｜begin▁of▁sentence｜>", "<｜end▁of▁sentence｜>", "<｜▁pad▁｜>"]
CHAT_SPECIALS = ["<｜User｜>", "<｜Assistant｜>", "<think>", "</think>", "<｜DSML｜", "</｜DSML｜"]


class ByteTokenizer:
    """ids: 0 BOS, 1 EOS, 2 PAD, 3..258 raw bytes, then the chat specials."""

    def __init__(self, vocab_size: Optional[int] = None, extra_specials: Sequence[str] = ()):
        self.bos, self.eos, self.pad = 0, 1, 2
        self.special: Dict[str, int] = {}
        nxt = 259
        for s in list(CHAT_SPECIALS) + list(extra_specials):
            self.special[s] = nxt
            nxt += 1
        self.vocab_size = max(vocab_size or nxt, nxt)
        self.think_end = self.special["</think>"]
        self._by_id = {v: k for k, v in self.special.items()}

    def token_bytes(self) -> List[bytes]:
        table = [b""] * self.vocab_size
        for b in range(256):
            table[3 + b] = bytes([b])
        for s, i in self.special.items():
            table[i] = s.encode("utf-8")
        return table

    def encode(self, text: str, add_bos: bool = False) -> List[int]:
        out = [self.bos] if add_bos else []
        i = 0
        keys = sorted(self.special, key=len, reverse=True)
        while i < len(text):
            for s in keys:
                if text.startswith(s, i):
                    out.append(self.special[s])
                    i += len(s)
                    break
            else:
                out.extend(3 + b for b in text[i].encode("utf-8"))
                i += 1
        return out

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        out = bytearray()
        for t in ids:
            if 3 <= t < 259:
                out.append(t - 3)
            elif t in self._by_id:
                out.extend(self._by_id[t].encode("utf-8"))
        return bytes(out)

    def decode(self, ids: Sequence[int]) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")


class HFTokenizer:
    def __init__(self, path: str, think_end_id: int = 128822):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(path)
        self.vocab_size = self.tk.get_vocab_size()
        self.bos, self.eos, self.pad = 0, 1, 2
        self.think_end = think_end_id

    def encode(self, text: str, add_bos: bool = False) -> List[int]:
        ids = self.tk.encode(text, add_special_tokens=False).ids
        return ([self.bos] if add_bos else []) + ids

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        return self.tk.decode(list(ids), skip_special_tokens=False).encode("utf-8")

    def decode(self, ids: Sequence[int]) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=False)

    def token_bytes(self) -> List[bytes]:
        from ..runtime.grammar import byte_level_vocab
        vocab = self.tk.get_vocab(with_added_tokens=True)
        return byte_level_vocab(vocab, self.vocab_size).token_bytes


class StreamingDecoder:
    """Incremental detokenizer: feed token ids, get the text that is safe to emit."""

    def __init__(self, tokenizer):
        self.tk = tokenizer
        self.pending = b""

    def push(self, ids: Sequence[int]) -> str:
        data = self.pending + self.tk.decode_bytes(ids)
        # find the longest prefix that ends on a complete UTF-8 sequence
        cut = len(data)
        for back in range(1, min(4, len(data)) + 1):
            b = data[-back]
            if b & 0xC0 == 0x80:
                continue                      # continuation byte, keep looking for the lead byte
            need = 1 if b < 0x80 else 2 if b >> 5 == 0b110 else 3 if b >> 4 == 0b1110 else 4 if b >> 3 == 0b11110 else 1
            if need > back:
                cut = len(data) - back        # incomplete sequence at the tail
            break
        self.pending = data[cut:]
        return data[:cut].decode("utf-8", errors="replace")

    def flush(self) -> str:
        out = self.pending.decode("utf-8", errors="replace")
        self.pending = b""
        return out
