"""Optional text front end: a thin wrapper over a Hugging Face tokenizer file.

The engine works on token ids; this wrapper exists so that text prompts can be used when
the model folder ships ``tokenizer.json``.  As in the reference
(``engine/tokenizer.py:71-90``) the beginning-of-sequence id is prepended when the
tokenizer does not add it itself.
"""

from __future__ import annotations

import json
import os


class Tokenizer:
    def __init__(self, backend, bos_token_id: int | None, eos_token_id: int | None) -> None:
        self._backend = backend
        self.bos_token_id = bos_token_id
        self.eos_token_id = eos_token_id

    @classmethod
    def from_pretrained(cls, model_dir: str) -> "Tokenizer":
        path = os.path.join(model_dir, "tokenizer.json")
        if not os.path.isfile(path):
            raise FileNotFoundError(f"{model_dir!r} has no tokenizer.json; pass token ids instead")
        try:
            from tokenizers import Tokenizer as _Backend
        except ImportError as e:  # pragma: no cover
            raise RuntimeError("text prompts need the 'tokenizers' package") from e
        backend = _Backend.from_file(path)
        bos = eos = None
        for name in ("generation_config.json", "config.json"):
            p = os.path.join(model_dir, name)
            if os.path.isfile(p):
                with open(p, "r", encoding="utf-8") as f:
                    raw = json.load(f)
                bos = raw.get("bos_token_id") if bos is None else bos
                eos = raw.get("eos_token_id") if eos is None else eos
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        return cls(backend, bos, eos)

    def encode(self, text: str) -> list[int]:
        ids = list(self._backend.encode(text).ids)
        if self.bos_token_id is not None and (not ids or ids[0] != self.bos_token_id):
            ids.insert(0, self.bos_token_id)
        return ids

    def decode(self, ids) -> str:
        return self._backend.decode(list(ids))
