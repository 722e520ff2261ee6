"""The RWKV "world" tokenizer: greedy longest-match over a byte-level vocabulary.

The vocabulary file has one token per line, ``<id> <python literal of the token> <byte length>``; a token is a ``str``
(stored as its UTF-8 bytes) or a ``bytes`` literal.  Encoding walks the UTF-8 bytes of the text and always takes the
longest vocabulary entry that matches at the current position (rwkv7_hf/tokenization_rwkv7.py:45-141).  The trie here
is three flat NumPy arrays (child table ``[nodes, 256]`` int32, token id per node, -1 = none) instead of linked nodes:
building it is one pass over the vocabulary, and a lookup step is two array reads.
"""
from __future__ import annotations

from ast import literal_eval

import numpy as np


def parse_vocab_line(line: str):
    """``(id, token bytes)`` of one vocabulary line; the trailing length field must agree with the token."""
    first, last = line.index(" "), line.rindex(" ")
    idx = int(line[:first])
    obj = literal_eval(line[first + 1:last])
    token = obj.encode("utf-8") if isinstance(obj, str) else obj
    if not isinstance(token, bytes):
        raise TypeError(f"Invalid token type at id={idx}: {type(token)}")
    if len(token) != int(line[last + 1:]):
        raise ValueError(f"Length mismatch at id={idx}: got {len(token)} expected {int(line[last + 1:])}")
    return idx, token


class RWKVWorldTokenizer:
    def __init__(self, vocab_file: str | None = None, *, tokens=None, pad_token_id: int = 0):
        """From a vocabulary file, or from ``tokens``: a mapping ``id -> bytes``."""
        if (vocab_file is None) == (tokens is None):
            raise ValueError("give either vocab_file or tokens")
        if tokens is None:
            tokens = {}
            with open(vocab_file, "r", encoding="utf-8") as f:
                for line in f:
                    line = line.rstrip("\n")
                    if line:
                        idx, tok = parse_vocab_line(line)
                        tokens[idx] = tok
        self.pad_token_id = int(pad_token_id)
        self.max_id = max(tokens) if tokens else 0
        # ids without an entry (unused embedding rows) decode to nothing
        self.id_to_bytes = [b""] * (self.max_id + 1)
        for idx, tok in tokens.items():
            self.id_to_bytes[idx] = bytes(tok)
        self.bytes_to_id = {bytes(tok): idx for idx, tok in tokens.items()}
        self._build()

    def _build(self):
        total = 1 + sum(len(t) for t in self.bytes_to_id)  # an upper bound on the node count
        child = np.full((total, 256), -1, dtype=np.int32)
        token = np.full((total,), -1, dtype=np.int64)
        n = 1
        for tok, idx in self.bytes_to_id.items():
            node = 0
            for b in tok:
                nxt = child[node, b]
                if nxt < 0:
                    nxt = child[node, b] = n
                    n += 1
                node = nxt
            token[node] = idx
        self._child, self._token = child[:n].copy(), token[:n].copy()

    @property
    def vocab_size(self) -> int:
        return self.max_id + 1

    def encode_bytes(self, src: bytes) -> list[int]:
        child, token = self._child, self._token
        out, pos, n = [], 0, len(src)
        while pos < n:
            node, best, end, p = 0, -1, pos, pos
            while p < n:
                node = child[node, src[p]]
                if node < 0:
                    break
                p += 1
                t = token[node]
                if t >= 0:
                    best, end = int(t), p
            if best < 0:
                raise ValueError(f"RWKV tokenizer cannot encode byte at offset {pos}: {src[pos:pos + 8]!r}")
            out.append(best)
            pos = end
        return out

    def encode(self, text: str) -> list[int]:
        return self.encode_bytes(text.encode("utf-8"))

    def decode_bytes(self, ids) -> bytes:
        table, size = self.id_to_bytes, len(self.id_to_bytes)
        return b"".join(table[i] for i in (int(t) for t in ids) if 0 <= i < size)

    def decode(self, ids, errors: str = "replace") -> str:
        return self.decode_bytes(ids).decode("utf-8", errors=errors)

    def __call__(self, texts, *, padding_side: str = "left", return_tensors: str | None = "pt", device=None):
        """Batch encode: ``{"input_ids", "attention_mask"}`` padded with ``pad_token_id`` (left by default: generation
        continues from the last column, and masked positions leave the recurrent state untouched)."""
        if isinstance(texts, str):
            texts = [texts]
        rows = [self.encode(t) for t in texts]
        width = max((len(r) for r in rows), default=0)
        ids = np.full((len(rows), width), self.pad_token_id, dtype=np.int64)
        mask = np.zeros((len(rows), width), dtype=np.int64)
        for i, r in enumerate(rows):
            sl = slice(width - len(r), width) if padding_side == "left" else slice(0, len(r))
            ids[i, sl] = r
            mask[i, sl] = 1
        if return_tensors == "pt":
            import torch
            return {"input_ids": torch.from_numpy(ids).to(device) if device else torch.from_numpy(ids),
                    "attention_mask": torch.from_numpy(mask).to(device) if device else torch.from_numpy(mask)}
        return {"input_ids": ids, "attention_mask": mask}

    def save_vocabulary(self, path: str) -> str:
        with open(path, "w", encoding="utf-8") as f:
            for idx, tok in enumerate(self.id_to_bytes):
                if not tok:
                    continue
                try:
                    lit = repr(tok.decode("utf-8"))
                    if literal_eval(lit).encode("utf-8") != tok:
                        raise UnicodeDecodeError("utf-8", tok, 0, 1, "round trip")
                except UnicodeDecodeError:
                    lit = repr(tok)
                f.write(f"{idx} {lit} {len(tok)}\n")
        return path
