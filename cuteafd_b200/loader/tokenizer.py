"""Tokenizers: a Hugging Face `tokenizer.json` when the snapshot ships one, else a byte-level fallback
(ids 0..255 = bytes, 256 = BOS, 257 = EOS) so the server and tests work without any model files.
Streaming decode holds back incomplete UTF-8 so SSE chunks never split a character
(reference: cuteafd-loader/src/tokenizer.rs, incremental detokenizer in serve.rs:260-291)."""
from __future__ import annotations

from pathlib import Path


class ByteTokenizer:
    bos_id, eos_id, vocab_size = 256, 257, 258

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: list[int]) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")


class HFTokenizer:
    def __init__(self, path: str):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(path)
        self.vocab_size = self.tk.get_vocab_size()
        self.eos_id = self.bos_id = None

    def encode(self, text: str) -> list[int]:
        return self.tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids: list[int]) -> str:
        return self.tk.decode(ids, skip_special_tokens=True)


def load_tokenizer(snapshot: str | None):
    if snapshot:
        f = Path(snapshot) / "tokenizer.json"
        if f.exists():
            try:
                return HFTokenizer(str(f))
            except Exception:
                pass
    return ByteTokenizer()


class StreamDecoder:
    """Incremental detokeniser: emits only text that later tokens cannot change."""

    def __init__(self, tok):
        self.tok, self.ids, self.sent = tok, [], 0

    def push(self, new_ids: list[int]) -> str:
        self.ids += new_ids
        text = self.tok.decode(self.ids)
        if text.endswith("�"):          # incomplete multi-byte sequence: wait for the rest
            text = text.rstrip("�")
        out, self.sent = text[self.sent:], max(self.sent, len(text))
        return out
