"""CPU restatement of the reference's CircularTensor::update (core/data/circular_tensor.h:111-161).

TEST INFRASTRUCTURE ONLY.  The reference runs one divergent launch over BATCH planes; this model walks the same
planes one by one with the reference's index arithmetic:

* which planes run the caller's chain: SequenceSelectorType::at (circular_tensor.h:26-35) - sequence 1 (the update) for
  plane 0 when the order is NewestFirst, for plane BATCH-1 when it is OldestFirst; sequence 2 (the copy) elsewhere;
* the update stores its result in the hidden tensor through CircularTensorWrite<Ascendent> at plane (z + first) mod
  BATCH (core/execution_model/memory_operations.h:436-446, 566-590) and in the visible tensor at plane z;
* a copy reads the hidden tensor through CircularTensorRead<Descendent> (NewestFirst: plane first - z) or <Ascendent>
  (OldestFirst: plane z + first), both mod BATCH (:436-446, 531-563), and stores at visible plane z;
* first advances by one, mod BATCH (circular_tensor.h:158).

The reference has no host launcher for its divergent kernel, so update() itself cannot be built from its headers and
this model cannot be checked against the reference on the CPU.  On a GPU the library's updates are compared with the
reference's divergent kernel itself (oracle/ref/fklref_circular.cpp launches it with the sequences update() builds);
this model covers the layouts, orders and batch sizes that unit is not built for.
The hidden tensor starts as zeros here (the reference leaves it as allocated).
"""
from __future__ import annotations

import numpy as np

NEWEST_FIRST, OLDEST_FIRST = 0, 1


def circular_index(direction_ascendent: bool, z: int, first: int, batch: int) -> int:
    """computeCircularThreadIdx (memory_operations.h:436-446)."""
    if direction_ascendent:
        zz = z + first
        return zz - batch if zz >= batch else zz
    zz = first - z
    return batch + zz if zz < 0 else zz


def selected_sequence(order: int, z: int, batch: int) -> int:
    """SequenceSelectorType::at (circular_tensor.h:26-35): 1 = the update chain, 2 = the copy."""
    if order == NEWEST_FIRST:
        return 2 if z > 0 else 1
    return 2 if z != batch - 1 else 1


class CircularTensorModel:
    def __init__(self, batch: int, order: int, plane_shape, dtype):
        self.batch, self.order, self.first = batch, order, 0
        self.hidden = np.zeros((batch, *plane_shape), dtype)
        self.visible = np.zeros((batch, *plane_shape), dtype)

    def update(self, result: np.ndarray) -> np.ndarray:
        """`result` is what the caller's chain produces for the new image (one plane)."""
        hidden_before = self.hidden.copy()   # all planes of the launch read the tensor as it was, except the one written
        for z in range(self.batch):
            if selected_sequence(self.order, z, self.batch) == 1:
                self.hidden[circular_index(True, z, self.first, self.batch)] = result
                self.visible[z] = result
            else:
                self.visible[z] = hidden_before[circular_index(self.order == OLDEST_FIRST, z, self.first, self.batch)]
        self.first = (self.first + 1) % self.batch
        return self.visible
