"""Replace the label of specified samples (reference: ``ffcv/transforms/replace_label.py``)."""
from dataclasses import replace
from typing import Callable, Optional, Tuple

import numpy as np

from ..pipeline.allocation_query import AllocationQuery
from ..pipeline.operation import Operation
from ..pipeline.state import State


class ReplaceLabel(Operation):
    """Replace label of specified images.

    Parameters
    ----------
    indices : Sequence[int]
        The indices of images to relabel.
    new_label : int
        The new label to assign.
    """

    def __init__(self, indices, new_label: int):
        super().__init__()
        self.indices = np.sort(indices)
        self.new_label = new_label

    def generate_code(self) -> Callable:
        to_change = self.indices
        new_label = self.new_label

        def replace_label(labels, temp_array, indices):
            indices = np.asarray(indices)
            position = np.searchsorted(to_change, indices)
            inside = position < len(to_change)
            hit = np.zeros(len(indices), dtype=bool)
            hit[inside] = to_change[position[inside]] == indices[inside]
            labels[hit] = new_label
            return labels
        replace_label.with_indices = True
        return replace_label

    def declare_state_and_memory(self, previous_state: State) -> Tuple[State, Optional[AllocationQuery]]:
        return (replace(previous_state, jit_mode=True), None)
