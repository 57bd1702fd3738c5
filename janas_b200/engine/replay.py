"""Trace replay over an engine: given token ids, step by step, logits out.

A step is a dictionary {"step": k, "entries": [{"id", "tokens", "want"}, ...],
"end": [ids]}.  Requests get a slot when they first appear and give it back when
they are named in ``end``.  Nothing is sampled.  ``bin/trace_run`` is this class
behind a command line.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import numpy as np

from .engine import Engine, StepEntry


class Replayer:
    def __init__(self, engine: Engine):
        self.engine = engine
        self.slots: Dict[object, int] = {}

    def run_step(self, req: Mapping) -> Optional[np.ndarray]:
        """Runs one step; returns float32 [wanted, vocab] or None."""
        entries = []
        fresh = []
        for e in req.get("entries", []):
            rid = e["id"]
            if rid not in self.slots:
                self.slots[rid] = self.engine.new_sequence()
                fresh.append(rid)
            entries.append(StepEntry(self.slots[rid], e["tokens"], e.get("want", [])))
        out = None
        if entries:
            try:
                out = self.engine.step_numpy(entries)
            except Exception:
                for rid in fresh:      # a refused step leaves no new request behind
                    self.engine.free_sequence(self.slots.pop(rid))
                raise
        for rid in req.get("end", []):
            if rid in self.slots:
                self.engine.free_sequence(self.slots.pop(rid))
        return out
