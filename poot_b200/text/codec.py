"""Text codec: tokenizer + streaming detokeniser.

Three sources, as in the reference (crates/poot-text/src/tokenize.rs:1-2): a HF ``tokenizer.json`` (through the
``tokenizers`` library), the tokenizer embedded in a GGUF header (``tokenizer.ggml.model`` = ``llama`` for the
score-driven SentencePiece-style merge, ``gpt2`` for byte-level BPE with a merge list), and a byte-level fallback
for synthetic checkpoints that ship no tokenizer.  ``StreamDecoder`` emits text incrementally and never splits a
multi-byte character across events.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence


class ByteTokenizer:
    """ids 0..255 are raw bytes shifted by ``offset``; everything else decodes to nothing."""

    def __init__(self, vocab: int, offset: int = 3, bos: Optional[int] = 1, eos: Optional[int] = 2):
        self.vocab, self.offset, self.bos, self.eos = vocab, offset, bos, eos

    def encode(self, text: str, add_bos: bool = True) -> List[int]:
        ids = [b + self.offset for b in text.encode("utf-8")]
        return ([self.bos] if add_bos and self.bos is not None else []) + ids

    def token_bytes(self, tid: int) -> bytes:
        b = tid - self.offset
        return bytes([b]) if 0 <= b < 256 else b""

    def decode(self, ids: Sequence[int]) -> str:
        return b"".join(self.token_bytes(i) for i in ids).decode("utf-8", errors="replace")

    def vocab_size(self) -> int:
        return self.vocab


class HfTokenizer:
    def __init__(self, path: str):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(path)
        cfg_path = os.path.join(os.path.dirname(path), "tokenizer_config.json")
        self.config = json.load(open(cfg_path)) if os.path.exists(cfg_path) else {}
        self.bos = self._special("bos_token")
        self.eos = self._special("eos_token")

    def _special(self, key: str) -> Optional[int]:
        t = self.config.get(key)
        if isinstance(t, dict):
            t = t.get("content")
        return self.tk.token_to_id(t) if t else None

    def encode(self, text: str, add_bos: bool = True) -> List[int]:
        ids = self.tk.encode(text, add_special_tokens=False).ids
        if add_bos and self.bos is not None and (not ids or ids[0] != self.bos):
            ids = [self.bos] + ids
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=True)

    def token_bytes(self, tid: int) -> bytes:
        return self.tk.decode([tid], skip_special_tokens=False).encode("utf-8")

    def vocab_size(self) -> int:
        return self.tk.get_vocab_size()


class GgufTokenizer:
    """Tokenizer rebuilt from GGUF metadata (``tokenizer.ggml.*``)."""

    def __init__(self, meta: Dict[str, object]):
        self.model = meta.get("tokenizer.ggml.model", "llama")
        self.tokens: List[str] = list(meta["tokenizer.ggml.tokens"])
        self.scores = list(meta.get("tokenizer.ggml.scores", [0.0] * len(self.tokens)))
        self.types = list(meta.get("tokenizer.ggml.token_type", [1] * len(self.tokens)))
        self.index = {t: i for i, t in enumerate(self.tokens)}
        self.bos = meta.get("tokenizer.ggml.bos_token_id")
        self.eos = meta.get("tokenizer.ggml.eos_token_id")
        self.unk = meta.get("tokenizer.ggml.unknown_token_id", 0)
        merges = meta.get("tokenizer.ggml.merges", [])
        self.merge_rank = {tuple(m.split(" ", 1)): r for r, m in enumerate(merges)}
        self._byte_enc = _gpt2_byte_table()
        self._byte_dec = {v: k for k, v in self._byte_enc.items()}

    def vocab_size(self) -> int:
        return len(self.tokens)

    def _merge(self, parts: List[str], rank_of) -> List[str]:
        while len(parts) > 1:
            best, bi = None, -1
            for i in range(len(parts) - 1):
                r = rank_of(parts[i], parts[i + 1])
                if r is not None and (best is None or r < best):
                    best, bi = r, i
            if best is None:
                break
            parts[bi:bi + 2] = [parts[bi] + parts[bi + 1]]
        return parts

    def encode(self, text: str, add_bos: bool = True) -> List[int]:
        ids: List[int] = []
        if self.model == "gpt2":
            import regex
            pat = regex.compile(r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+")
            for piece in pat.findall(text):
                sym = [self._byte_enc[b] for b in piece.encode("utf-8")]
                for p in self._merge(sym, lambda a, b: self.merge_rank.get((a, b))):
                    ids.append(self.index.get(p, self.unk))
        else:
            sym = list(("▁" + text.replace(" ", "▁")) if text else "")

            def rank(a, b):
                i = self.index.get(a + b)
                return None if i is None else -self.scores[i]
            for p in self._merge(sym, rank):
                i = self.index.get(p)
                if i is not None:
                    ids.append(i)
                else:   # byte fallback tokens <0xNN>
                    for byte in p.encode("utf-8"):
                        ids.append(self.index.get(f"<0x{byte:02X}>", self.unk))
        if add_bos and self.bos is not None:
            ids = [int(self.bos)] + ids
        return ids

    def token_bytes(self, tid: int) -> bytes:
        if not 0 <= tid < len(self.tokens) or self.types[tid] in (3, 4):     # control / unused
            return b""
        t = self.tokens[tid]
        if self.model == "gpt2":
            return bytes(self._byte_dec.get(ch, 63) for ch in t)
        if len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
            return bytes([int(t[3:5], 16)])
        return t.replace("▁", " ").encode("utf-8")

    def decode(self, ids: Sequence[int]) -> str:
        s = b"".join(self.token_bytes(i) for i in ids).decode("utf-8", errors="replace")
        return s[1:] if self.model != "gpt2" and s.startswith(" ") else s


def _gpt2_byte_table() -> Dict[int, str]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    cs, n = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


class StreamDecoder:
    """Incremental detokenisation: emits only complete UTF-8 sequences."""

    def __init__(self, tokenizer):
        self.tk, self.pending = tokenizer, b""

    def push(self, tid: int) -> str:
        self.pending += self.tk.token_bytes(tid)
        for cut in range(len(self.pending), max(len(self.pending) - 4, -1), -1):
            try:
                text = self.pending[:cut].decode("utf-8")
            except UnicodeDecodeError:
                continue
            self.pending = self.pending[cut:]
            return text
        return ""

    def flush(self) -> str:
        text, self.pending = self.pending.decode("utf-8", errors="replace"), b""
        return text


def load_tokenizer(handle=None, path: Optional[str] = None, vocab: int = 32000):
    """Tokenizer for a model handle / directory, falling back to bytes."""
    d = path or (handle.tokenizer_dir if handle is not None else None)
    if d and os.path.exists(os.path.join(d, "tokenizer.json")):
        return HfTokenizer(os.path.join(d, "tokenizer.json"))
    if handle is not None and handle.kind == "gguf" and "tokenizer.ggml.tokens" in handle.store.metadata:
        return GgufTokenizer(handle.store.metadata)
    return ByteTokenizer(handle.cfg.vocab if handle is not None else vocab)
