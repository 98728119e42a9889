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


def _eos_ids(snapshot: Path, tk) -> list[int]:
    """End-of-sequence ids of a snapshot: `generation_config.json` / `config.json` (`eos_token_id`, int or list), else the
    id of `eos_token` named in `tokenizer_config.json`."""
    import json
    ids: list[int] = []
    for name in ("generation_config.json", "config.json"):
        f = snapshot / name
        if f.exists():
            try:
                v = json.loads(f.read_text()).get("eos_token_id")
            except Exception:
                v = None
            for x in (v if isinstance(v, list) else [v]):
                if isinstance(x, int) and x not in ids:
                    ids.append(x)
    f = snapshot / "tokenizer_config.json"
    if f.exists():
        try:
            tok = json.loads(f.read_text()).get("eos_token")
            tok = tok.get("content") if isinstance(tok, dict) else tok
            i = tk.token_to_id(tok) if isinstance(tok, str) else None
            if i is not None and i not in ids:
                ids.append(i)
        except Exception:
            pass
    return ids


class HFTokenizer:
    def __init__(self, path: str):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(path)
        self.vocab_size = self.tk.get_vocab_size()
        eos = _eos_ids(Path(path).parent, self.tk)
        self.eos_id = eos[0] if eos else None
        self.stop_ids = tuple(eos[1:])                 # further ids that end a turn (e.g. <|im_end|> next to <|endoftext|>)
        self.bos_id = None

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
