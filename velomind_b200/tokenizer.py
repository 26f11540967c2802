"""Byte-level BPE tokenizer read from a Hugging Face `tokenizer.json` (optional: generation works on token
ids without it).

Behaviour follows the reference's tokenizer (examples/smollm2/tokenizer.cpp): fields `model.vocab`,
`model.merges`, `added_tokens` (:77-167); special ids inferred from the token text (:153-166); the GPT-2
byte <-> unicode table; a hand-written pre-tokenizer (contractions, runs of letters with one leading space,
single digits, runs of other symbols, runs of whitespace; :236-368); lowest-rank-first merges (:370-429);
decoding skips the begin/end/pad ids (:466-498).
One deliberate difference: after a space, the reference glues that space to EVERY digit of a number
(" 12" -> " 1", " 2"), which does not decode back to the input; here the space is a piece of its own and
digits stand alone.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional, Sequence, Tuple


def _byte_unicode_table() -> Dict[int, str]:
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


_BYTE_TO_UNI = _byte_unicode_table()
_UNI_TO_BYTE = {v: k for k, v in _BYTE_TO_UNI.items()}
_CONTRACTIONS = ("'s", "'t", "'m", "'d", "'re", "'ve", "'ll")


def pretokenize(text: str) -> List[str]:
    pieces: List[str] = []
    i, n = 0, len(text)
    while i < n:
        hit = next((c for c in _CONTRACTIONS if text.startswith(c, i)), None)
        if hit:
            pieces.append(hit)
            i += len(hit)
            continue
        ch = text[i]
        j = i
        if ch == " " and i + 1 < n and text[i + 1].isalpha():
            j = i + 1
            while j < n and text[j].isalpha():
                j += 1
        elif ch.isalpha():
            while j < n and text[j].isalpha():
                j += 1
        elif ch.isdigit():
            j = i + 1                                    # digits stand alone
        elif not ch.isspace():
            while j < n and not (text[j].isspace() or text[j].isalpha() or text[j].isdigit()):
                j += 1
        else:
            if ch == " " and i + 1 < n and text[i + 1].isdigit():
                j = i + 1                                # the space before a number is its own piece
            else:
                while j < n and text[j].isspace():
                    j += 1
        pieces.append(text[i:j])
        i = j
    return ["".join(_BYTE_TO_UNI[b] for b in p.encode("utf-8")) for p in pieces]


class ByteLevelBPETokenizer:
    def __init__(self, vocab: Dict[str, int], merges: Sequence[Tuple[str, str]], added: Dict[str, int]):
        self.token_to_id = dict(vocab)
        self.token_to_id.update(added)
        size = max(self.token_to_id.values()) + 1
        self.id_to_token: List[str] = [""] * size
        for tok, i in self.token_to_id.items():
            self.id_to_token[i] = tok
        self.rank = {pair: r for r, pair in enumerate(merges)}
        self.bos_id: Optional[int] = None
        self.eos_id: Optional[int] = None
        self.pad_id: Optional[int] = None
        self.unk_id: Optional[int] = None
        for tok, i in added.items():
            if tok in ("<|endoftext|>", "<s>", "<bos>"):
                self.bos_id = i
                if self.eos_id is None:
                    self.eos_id = i
            elif tok in ("<|im_end|>", "</s>", "<eos>"):
                self.eos_id = i
            elif tok in ("<pad>", "<|padding|>"):
                self.pad_id = i
            elif tok == "<unk>":
                self.unk_id = i
        if self.bos_id is None and self.eos_id is not None:
            self.bos_id = self.eos_id

    @classmethod
    def from_file(cls, path: str) -> "ByteLevelBPETokenizer":
        with open(path, "r", encoding="utf-8") as f:
            root = json.load(f)
        model = root.get("model") if isinstance(root, dict) else None
        if not isinstance(model, dict) or not isinstance(model.get("vocab"), dict) or not model["vocab"]:
            raise ValueError(f"{path}: no model.vocab object")
        merges = []
        for m in model.get("merges", []):
            if isinstance(m, str):
                a, _, b = m.partition(" ")
                merges.append((a, b))
            elif isinstance(m, list) and len(m) == 2:
                merges.append((m[0], m[1]))
        added = {t["content"]: int(t["id"]) for t in root.get("added_tokens", [])
                 if isinstance(t, dict) and isinstance(t.get("content"), str) and isinstance(t.get("id"), int)}
        return cls({k: int(v) for k, v in model["vocab"].items()}, merges, added)

    def _bpe(self, word: str) -> List[str]:
        symbols = list(word)
        while len(symbols) > 1:
            best, at = None, -1
            for i in range(len(symbols) - 1):
                r = self.rank.get((symbols[i], symbols[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            symbols[at: at + 2] = [symbols[at] + symbols[at + 1]]
        return symbols

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        for piece in pretokenize(text):
            if piece in self.token_to_id:
                out.append(self.token_to_id[piece])
                continue
            for sym in self._bpe(piece):
                if sym in self.token_to_id:
                    out.append(self.token_to_id[sym])
                elif self.unk_id is not None:
                    out.append(self.unk_id)
        return out

    def decode(self, ids: Sequence[int]) -> str:
        data = bytearray()
        skip = {self.bos_id, self.eos_id, self.pad_id}
        for i in ids:
            if i < 0 or i >= len(self.id_to_token) or i in skip:
                continue
            for ch in self.id_to_token[i]:
                b = _UNI_TO_BYTE.get(ch)
                if b is not None:
                    data.append(b)
                else:
                    data.extend(ch.encode("utf-8"))
        return data.decode("utf-8", errors="replace")
