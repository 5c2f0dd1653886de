"""Host-side mirror of the reference's graph types for the hot path.

`Node`, `Graph` and the attribute map follow oxionnx-core/src/graph.rs:696-733 (Attributes)
and :851 (Node): an operator name, input/output value names ("" marks an omitted optional
input) and typed attributes.  Tensors are numpy float32 arrays: the reference's f32-lane
convention (oxionnx-core/src/tensor/types.rs:355), where quantised values are integers
carried in f32 lanes.
"""
from dataclasses import dataclass, field
from typing import Dict, List

import numpy as np


@dataclass
class Node:
    op: str
    name: str
    inputs: List[str]
    outputs: List[str]
    attrs: Dict[str, object] = field(default_factory=dict)


@dataclass
class Graph:
    nodes: List[Node]
    input_names: List[str]
    output_names: List[str]


def tensor(data, shape=None) -> np.ndarray:
    """f32-lane tensor (Tensor::new)."""
    a = np.asarray(data, dtype=np.float32)
    if shape is not None:
        a = a.reshape(shape)
    return np.ascontiguousarray(a)
