"""Assembles the dictionaries that `_make_compiler` takes (the same five arguments the reference's
`refactor_graph/onnx.py:make_compiler` passes: topology, nodes, edges, inputs, outputs)."""
from __future__ import annotations

import numpy as np

from . import python_ffi as ffi

# reference DataType codes
F32, I32, I64, BOOL, FP16, BF16 = 1, 6, 7, 9, 10, 16
NP_CODE = {np.dtype(np.float32): F32, np.dtype(np.float16): FP16, np.dtype(np.int64): I64, np.dtype(np.int32): I32,
           np.dtype(np.bool_): BOOL}


class GraphBuilder:
    def __init__(self):
        self.topology, self.nodes, self.edges = {}, {}, {}
        self.inputs, self.outputs = [], []
        self._n = 0

    def input(self, name: str, dtype: int, shape) -> str:
        """A global input edge: fed by executor.set_input / set_input_blob (weights, caches, per-step state)."""
        self.edges[name] = ffi._make_tensor(dtype, list(shape))
        self.inputs.append(name)
        return name

    def constant(self, name: str, array: np.ndarray, dtype: int = 0) -> str:
        """An edge with host data, uploaded once at compile time like an ONNX initializer."""
        self.edges[name] = ffi._make_data(np.ascontiguousarray(array), dtype)
        return name

    def op(self, op_type: str, inputs, n_out: int = 1, name: str | None = None, **attrs):
        self._n += 1
        name = name or f"{self._n:05d}_{op_type.split('::')[-1]}"
        outs = [f"{name}:{i}" for i in range(n_out)]
        self.topology[name] = (list(inputs), outs)
        self.nodes[name] = ffi._make_operator({}, op_type, attrs)
        return outs[0] if n_out == 1 else (outs or None)

    def output(self, edge: str) -> int:
        self.outputs.append(edge)
        return len(self.outputs) - 1

    def compiler(self):
        return ffi._make_compiler(self.topology, self.nodes, self.edges, self.inputs, self.outputs)
