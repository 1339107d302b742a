"""Per-sequence state that does not grow with the sequence: a recurrence's state, a convolution's last inputs, the previous
token.  It sits beside the block manager (worker/block_manager.py), which hands out cache rows per token: here every sequence
owns ONE row - its block-table row - of each state tensor for as long as it lives, so a batch addresses state and cache rows
with the same `seq_ids`.

Rows are used again without being cleared: the kernels that read a state take the zero state for a segment that starts at
position 0 (csrc/recurrent.cu, csrc/scan_ops.cu, csrc/stream_ops.cu), so a new sequence never sees what the row's previous owner left, and
freeing a sequence costs nothing here."""
from __future__ import annotations

import torch


class SequenceStateManager:
    def __init__(self, max_seqs: int, layout: dict, device):
        """layout: name -> (shape of one sequence's state, dtype)."""
        self.max_seqs = max_seqs
        self.tensors = {name: torch.zeros((max_seqs,) + tuple(shape), dtype=dtype, device=device)
                        for name, (shape, dtype) in layout.items()}

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.tensors[name]

    def bytes_per_seq(self) -> int:
        return sum(t[0].numel() * t.element_size() for t in self.tensors.values())

    def scratch(self, rows: int) -> "SequenceStateManager":
        """A second set of state tensors with `rows` rows (warm-up runs that must not touch live sequences)."""
        other = SequenceStateManager.__new__(SequenceStateManager)
        other.max_seqs = rows
        other.tensors = {n: torch.zeros((rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device) for n, t in self.tensors.items()}
        return other
