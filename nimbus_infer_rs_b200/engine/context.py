"""What a part sees of the step it runs in."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .batch import BatchLayout
from .model import Runtime


@dataclass
class StepContext:
    rt: Runtime
    ops: Any                 # kernel backend (csrc.ops.CudaBackend)
    layout: BatchLayout
    position: Any            # the model's position-encoding part
    cache: Any               # SequenceCache
    # storage of the schedule entry that is running (set by the model before each layer)
    kv: Any = None           # LayerKV or None
    state: Any = None        # fp32 [n_slots, n_elements] or None
    kv_extra: Any = ()       # LayerKV of the mixer's further stores, in the order it asked
    writes_cache: bool = True
    # what a layer's mixer leaves for the feed-forward beside it: (fp32 rows, first column)
    shared_projection: Any = None
    # buffers that a part keeps for the rest of the step (keyed by the part)
    scratch: dict = field(default_factory=dict)
    # the first norm of the schedule entry that runs next, if that entry's arrangement takes its
    # normed rows from the arrangement before it (which then computes them in its last pass over
    # the stream and leaves them in ``normed``)
    next_norm: Any = None
    normed: Any = None
