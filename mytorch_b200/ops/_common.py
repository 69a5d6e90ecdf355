"""Shared front-end plumbing: look up the backend function, mark the result, record the node."""
from mytorch_b200.autograd import DAGTracker
from mytorch_b200.backends.backend_dispatcher import BackendDispatcher

tracker = DAGTracker.instance()


def dispatch(device, name):
    return BackendDispatcher.instance().dispatch(device.type, name)


def grad_enabled(*tensors):
    return any(t is not None and t.requires_grad for t in tensors) and not tracker.no_grad


def record(name, inputs, output, helpers=None):
    if output.requires_grad:
        tracker.add_node(name, inputs, [output], helpers)
    return output
