"""Graph nodes and the reverse sweep.

Same contract as the reference's `basic_operator.py` / `autodiff.py` (an `Op` has
`compute(*arrays)` and `gradient(out_grad, node)`; a `Value` caches its data and is realised
eagerly; `backward` walks the graph in reverse topological order, sums the partial adjoints of
each node and stores the sum in `node.grad`), written independently: the ordering is an
explicit-stack depth-first search, so deep graphs do not need a raised recursion limit.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple


class Op:
    """An operator: `compute` maps raw arrays to a raw array, `gradient` maps the upstream
    adjoint (a node) to the adjoints of the inputs (nodes)."""

    def __call__(self, *args):
        raise NotImplementedError

    def compute(self, *arrays):
        raise NotImplementedError

    def gradient(self, out_grad, node):
        raise NotImplementedError

    def gradient_as_tuple(self, out_grad, node) -> Tuple:
        g = self.gradient(out_grad, node)
        return tuple(g) if isinstance(g, (tuple, list)) else (g,)


class Value:
    """A node of the computation graph."""

    op: Optional[Op]
    inputs: Sequence["Value"]
    cached_data: object
    requires_grad: bool

    def _init(self, op, inputs, *, cached_data=None, requires_grad=None, num_outputs=1):
        if requires_grad is None:
            requires_grad = any(x.requires_grad for x in inputs)
        self.op, self.inputs = op, list(inputs)
        self.cached_data, self.requires_grad, self.num_outputs = cached_data, requires_grad, num_outputs

    def is_leaf(self) -> bool:
        return self.op is None

    def realize_cached_data(self):
        if self.cached_data is None:
            self.cached_data = self.op.compute(*[x.realize_cached_data() for x in self.inputs])
        return self.cached_data

    @classmethod
    def make_const(cls, data, *, requires_grad=False):
        node = cls.__new__(cls)
        node._init(None, [], cached_data=data, requires_grad=requires_grad)
        return node

    @classmethod
    def make_from_op(cls, op: Op, inputs: Sequence["Value"]):
        node = cls.__new__(cls)
        node._init(op, inputs)
        if not node.requires_grad:
            return node.detach()
        node.realize_cached_data()
        return node


def topological_order(outputs: Sequence[Value]) -> List[Value]:
    """Inputs before the nodes that use them (post-order depth-first search, explicit stack)."""
    order: List[Value] = []
    seen = set()
    for root in outputs:
        if id(root) in seen:
            continue
        stack = [(root, iter(root.inputs))]
        seen.add(id(root))
        while stack:
            node, children = stack[-1]
            advanced = False
            for child in children:
                if id(child) not in seen:
                    seen.add(id(child))
                    stack.append((child, iter(child.inputs)))
                    advanced = True
                    break
            if not advanced:
                order.append(node)
                stack.pop()
    return order


def backward_pass(output: Value, out_grad: Value) -> None:
    """Reverse sweep from `output` seeded with `out_grad`; leaves `node.grad` on every node."""
    pending: Dict[int, list] = {id(output): [out_grad]}
    for node in reversed(topological_order([output])):
        parts = pending.pop(id(node), None)
        if not parts:
            continue
        total = parts[0]
        for extra in parts[1:]:
            total = total + extra
        node.grad = total
        if node.op is None:
            continue
        for inp, g in zip(node.inputs, node.op.gradient_as_tuple(total, node)):
            pending.setdefault(id(inp), []).append(g)
