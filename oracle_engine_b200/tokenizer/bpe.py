"""Byte-level BPE tokenizer, used only when the model folder holds a tokenizer.json.

The algorithm is the reference's (core/tokenizer.cpp): text is cut into words at
whitespace, a space or tab staying attached to the word after it and a line break being a
word of its own (:210-241); each word is mapped byte by byte to the printable alphabet of
GPT-2 (:15-36); pairs are merged by lowest merge rank until none applies (:157-181); a
piece that is no token falls back to `<0xXX>` byte tokens (:183-201); a whole word that is
a special token is taken as that token (:254-261).  The reference reads vocabulary and
merges from GGUF metadata (:41-79); here they come from tokenizer.json (`model.vocab`,
`model.merges`, `added_tokens`).  The file's own split pattern is not used, so ids can
differ from other tools on unusual text; token ids (`--tokens`) are the exact interface.
"""
from __future__ import annotations

import json
from pathlib import Path


def _byte_tables():
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    b2u, n = {}, 0
    for b in range(256):
        if b in keep:
            b2u[b] = chr(b)
        else:
            b2u[b] = chr(256 + n)
            n += 1
    return b2u, {u: b for b, u in b2u.items()}


class Tokenizer:
    def __init__(self, vocab: dict, merges: list, special: dict, bos_id=None):
        self.tok2id = dict(vocab)
        self.tok2id.update(special)
        self.id2tok = {i: t for t, i in self.tok2id.items()}
        self.special = dict(special)
        self.special_ids = set(special.values())
        self.rank = {}
        for r, m in enumerate(merges):
            pair = tuple(m.split(" ")) if isinstance(m, str) else tuple(m)
            if len(pair) == 2:
                self.rank.setdefault(pair, r)
        self.bos_id = bos_id
        self.b2u, self.u2b = _byte_tables()

    @classmethod
    def from_folder(cls, folder, bos_id=None):
        path = Path(folder) / "tokenizer.json"
        if not path.is_file():
            return None
        raw = json.loads(path.read_text(encoding="utf-8"))
        model = raw.get("model", {})
        special = {t["content"]: t["id"] for t in raw.get("added_tokens", []) if t.get("special", True)}
        return cls(model.get("vocab", {}), model.get("merges", []), special, bos_id)

    # ------------------------------------------------------------------ encode
    @staticmethod
    def _words(text: str):
        words, cur = [], ""
        for ch in text:
            if ch in " \t":
                if cur:
                    words.append(cur)
                cur = ch
            elif ch in "\n\r":
                if cur:
                    words.append(cur)
                words.append(ch)
                cur = ""
            else:
                cur += ch
        if cur:
            words.append(cur)
        return words

    def _bpe(self, word: str):
        pieces = [self.b2u[b] for b in word.encode("utf-8")]
        while len(pieces) > 1:
            best, at = None, -1
            for i in range(len(pieces) - 1):
                r = self.rank.get((pieces[i], pieces[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if at < 0:
                break
            pieces[at:at + 2] = [pieces[at] + pieces[at + 1]]
        ids = []
        for p in pieces:
            if p in self.tok2id:
                ids.append(self.tok2id[p])
            else:
                for ch in p:
                    ids.append(self.tok2id.get("<0x%02X>" % self.u2b[ch], 0))
        return ids

    def encode(self, text: str, add_bos: bool = True):
        ids = [self.bos_id] if add_bos and self.bos_id is not None else []
        for w in self._words(text):
            if w in self.special:
                ids.append(self.special[w])
            else:
                ids.extend(self._bpe(w))
        return ids

    # ------------------------------------------------------------------ decode
    def decode_bytes(self, token_id: int) -> bytes:
        tok = self.id2tok.get(token_id)
        if tok is None or token_id in self.special_ids:
            return b""                       # special tokens are not shown (core/tokenizer.cpp:284-286)
        if len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">"):
            try:
                return bytes([int(tok[3:5], 16)])
            except ValueError:
                pass
        return bytes(self.u2b[ch] for ch in tok if ch in self.u2b)

    def decode(self, ids) -> str:
        return b"".join(self.decode_bytes(i) for i in ids).decode("utf-8", errors="replace")
