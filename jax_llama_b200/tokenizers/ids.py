"""Token ids as text: a stand-in tokenizer for checkpoints that come without one.

``"3 17 5"`` encodes to ``[bos, 3, 17, 5]`` and decodes back to the same form, so the generation front-end
(`LLaMA.generate_from_str`, the example command line) can drive any registered model from raw token ids.
"""
from __future__ import annotations

from typing import List, Sequence


class IdTokenizer:
    def __init__(self, vocab_size: int, bos_id: int = 1, eos_id: int = 0):
        self.n_words = int(vocab_size)
        self.bos_id, self.eos_id, self.pad_id = int(bos_id), int(eos_id), int(eos_id)

    def encode(self, s: str, bos: bool = True, eos: bool = False) -> List[int]:
        ids = [int(t) for t in s.split()]
        bad = [t for t in ids if not 0 <= t < self.n_words]
        if bad:
            raise ValueError(f"token ids {bad[:4]} outside the vocabulary of {self.n_words}")
        return ([self.bos_id] if bos else []) + ids + ([self.eos_id] if eos else [])

    def decode(self, ids: Sequence[int]) -> str:
        return " ".join(str(int(i)) for i in ids)
