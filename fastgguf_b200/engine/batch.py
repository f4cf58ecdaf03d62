"""One entry of a step: a slot, its next tokens, and the places among them whose logits are wanted.

A step is a list of such entries: every sequence brings one or more next tokens (all prompts of a batch in
the first step, one token each afterwards - but any mix is legal).  Rows are laid out sequence after
sequence; the host packs the step's integers and copies them to the device in one piece
(``DecoderModel::build_batch`` in ``csrc/host/model.cpp``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()
