"""Replay of given token ids through the engine (the library side of ``bin/trace_run``).

It keeps only the map from a request's id to its cache slot; every token goes through
``Engine.step``.
"""
from __future__ import annotations

import numpy as np

from ..core import RuntimeFault
from .model import Model
from .step import Engine, StepEntry


SPARE_BLOCKS = 64  # beyond ``max_tokens``: every live request may hold one cache block that is not full


class Replayer:
    def __init__(self, model_folder: str, dtype: str, max_tokens: int, device: str = "cuda:0", model=None):
        """``max_tokens``: the most tokens that live requests hold at any time.  The cache is made of blocks of
        64 positions and a request's last block is rarely full, so room for ``SPARE_BLOCKS`` more blocks (and
        at least that many live requests) is added."""
        from ..cache import BLOCK_TOKENS
        self.model = model if model is not None else Model.load(model_folder, dtype=dtype, device=device)
        self.engine = Engine(self.model, max(1, int(max_tokens)) + SPARE_BLOCKS * BLOCK_TOKENS)
        self.slots: dict[str, int] = {}

    def run_step(self, record: dict):
        """Runs one step record; returns the wanted logits as a float32 array [wanted, vocab], or
        None if nothing was wanted."""
        entries = []
        for item in record.get("entries", []):
            rid = str(item["id"])
            if rid not in self.slots:
                self.slots[rid] = self.engine.open_slot()
            entries.append(StepEntry(self.slots[rid], list(item["tokens"]), list(item.get("want", []))))
        logits = self.engine.step(entries) if entries else None
        for rid in record.get("end", []):
            rid = str(rid)
            if rid not in self.slots:
                raise RuntimeFault(f"step {record.get('step')}: request {rid!r} ends but was never seen")
            self.engine.close_slot(self.slots.pop(rid))
        self.engine.check_errors()
        if logits is None:
            return None
        return logits.float().cpu().numpy().astype(np.float32)
