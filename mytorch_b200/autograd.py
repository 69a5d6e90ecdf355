"""Tape-based reverse-mode differentiation.

Observable behaviour follows the reference's ``mytorch/autograd.py``: operators call
``add_node(name, input_args, output_tensors, helper_tensors)`` (``:33-54``); ``backward``
(``:120-179``) accepts only a one-element tensor, seeds its gradient with 1, calls each
operator's registered backward as ``f(*output_grads, *helpers, *input_args)``, zips the returned
list with ``input_args`` and accumulates into every input that requires a gradient (first
contribution assigned, later ones added), then forgets the visited graph — a second
``backward`` through the same graph raises "Make sure you don't backward a tensor twice".
``no_grad()`` (``:181-196``) is re-entrant.

The implementation differs: every node carries a creation sequence number, so the nodes
upstream of the loss sorted by descending sequence are already a valid reverse topological
order — no degree counting, no dictionary keyed by tensors.
"""
from __future__ import annotations


class _Node:
    __slots__ = ("name", "inputs", "outputs", "helpers", "seq")

    def __init__(self, name, inputs, outputs, helpers, seq):
        self.name, self.inputs, self.outputs, self.helpers, self.seq = name, inputs, outputs, helpers, seq


class DAGTracker:
    _instance = None

    @classmethod
    def instance(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def __init__(self):
        self._backward_funcs = {}
        self._seq = 0
        self.no_grad = False
        # optional callback(tensor): a leaf tensor has received its last gradient contribution of
        # the running backward pass (used to start gradient all-reduces while backward continues)
        self.leaf_grad_final_hook = None
        # optional callback(): a backend that ran gradient kernels beside the main chain (weight gradients
        # on a second CUDA stream) makes them visible to it; called before a gradient is read or handed
        # out during the pass, and when the pass ends
        self.join_hook = None
        # operators whose backward may be told ``defer_weight_gradient=True``: the returned parameter
        # gradient then becomes valid at the next join_hook() call, not when the backward returns
        self.deferrable = set()
        # operator name -> index of the input whose already accumulated gradient the operator's
        # backward can add itself (keyword ``accumulate_dx``); the tape then stores the returned
        # gradient instead of launching an add
        self.fused_accumulate = {}

    def register_backward_function(self, op_name):
        def decorator(func):
            self._backward_funcs[op_name] = func
            return func

        return decorator

    def add_node(self, name, input_args, output_tensors, helper_tensors=None):
        self._seq += 1
        node = _Node(name, list(input_args), list(output_tensors), list(helper_tensors or []), self._seq)
        for t in output_tensors:
            t._grad_node = node

    def _upstream(self, root):
        from mytorch_b200.tensor import Tensor

        seen, stack, nodes = set(), [root], []
        while stack:
            node = stack.pop()
            if id(node) in seen:
                continue
            seen.add(id(node))
            nodes.append(node)
            for arg in node.inputs:
                if isinstance(arg, Tensor) and arg._grad_node is not None:
                    stack.append(arg._grad_node)
        nodes.sort(key=lambda n: -n.seq)
        return nodes

    def backward(self, tensor):
        from mytorch_b200.tensor import MismatchShapesError, Tensor, shape_size

        if tensor._grad_node is None:
            raise RuntimeError("Make sure you don't backward a tensor twice")
        if shape_size(tensor.shape) != 1:
            raise RuntimeError("Backward tensor must be a scalar")
        order = self._upstream(tensor._grad_node)
        seed = Tensor(shape=tensor.shape, dtype=tensor.dtype, device=tensor.device)
        seed.fill_(1)
        tensor.grad = seed

        hook = self.leaf_grad_final_hook
        pending = {}
        if hook is not None:  # how many contributions every leaf will receive
            for node in order:
                for arg in node.inputs:
                    if isinstance(arg, Tensor) and arg.requires_grad and arg._grad_node is None:
                        pending[id(arg)] = pending.get(id(arg), 0) + 1

        for node in order:
            func = self._backward_funcs[node.name]
            fused = None  # the input whose gradient so far is handed to the operator
            slot = self.fused_accumulate.get(node.name)
            if slot is not None:
                cand = node.inputs[slot]
                if isinstance(cand, Tensor) and cand.requires_grad and cand.grad is not None:
                    fused = cand
            extra = {}
            if fused is not None:
                extra["accumulate_dx"] = fused.grad
            if node.name in self.deferrable and self.join_hook is not None:
                extra["defer_weight_gradient"] = True
            grads = list(func(*[t.grad for t in node.outputs], *node.helpers, *node.inputs, **extra))
            grads += [None] * (len(node.inputs) - len(grads))
            for arg, grad in zip(node.inputs, grads):
                if arg is None or not isinstance(arg, Tensor) or not arg.requires_grad:
                    continue
                if grad is not None:
                    if arg.grad is None or (arg is fused and grad is grads[slot]):
                        arg.grad = grad
                    else:
                        if arg.grad.shape != grad.shape:
                            raise MismatchShapesError([arg.grad.shape, grad.shape])
                        if self.join_hook is not None and arg._grad_node is None:  # a leaf: its gradient may come from there
                            self.join_hook()
                        arg.grad = arg.grad + grad
                if hook is not None and id(arg) in pending:
                    pending[id(arg)] -= 1
                    if pending[id(arg)] == 0 and arg.grad is not None:
                        hook(arg)  # the gradient may still be in flight on the backend's side stream: the hook orders itself after it

        if self.join_hook is not None:
            self.join_hook()

        for node in order:
            for t in node.outputs:
                t._grad_node = None
            node.inputs = node.outputs = node.helpers = ()


class NoGrad:
    _depth = 0

    def __enter__(self):
        NoGrad._depth += 1
        DAGTracker.instance().no_grad = True

    def __exit__(self, exc_type, exc_value, traceback):
        NoGrad._depth -= 1
        if NoGrad._depth == 0:
            DAGTracker.instance().no_grad = False


def no_grad():
    return NoGrad()
