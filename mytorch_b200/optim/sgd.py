"""SGD (``mytorch/optim/sgd.py:6-56``): same constructor, same per-parameter
``state[param]["momentum_buffer"]``.  When every parameter of a group lives on one CUDA device
the whole group is updated by one multi-tensor launch; otherwise (and through the registry's
``sgd`` entry) one launch per parameter, as in the reference."""
from mytorch_b200.backends.backend_dispatcher import BackendDispatcher
from mytorch_b200.optim.optimizer import Optimizer
from mytorch_b200.tensor import Tensor


class SGD(Optimizer):
    def __init__(self, params, lr=0.001, momentum=0, dampening=0, weight_decay=0, nesterov=False, maximize=False):
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov, maximize=maximize))
        self.grad_scale = 1.0  # set to 1/world_size by the data-parallel wrapper

    def step(self):
        dispatcher = BackendDispatcher.instance()
        for group in self.param_groups:
            entries = []
            for param in group["params"]:
                if param.shape != param.grad.shape:
                    raise RuntimeError(f"Mismatched shape between param and param.grad: {param}, {param.grad}")
                state = self.state.setdefault(param, {})
                first = state.get("momentum_buffer") is None
                if first:
                    state["momentum_buffer"] = Tensor(shape=param.shape, device=param.device, dtype=param.dtype)
                entries.append((param, state["momentum_buffer"], first))
            hyper = (group["lr"], group["weight_decay"], group["momentum"], group["dampening"], group["nesterov"], group["maximize"])
            devices = {(p.device.type, p.device.index) for p, _, _ in entries}
            if len(devices) == 1 and next(iter(devices))[0] == "cuda":
                dispatcher.dispatch("cuda", "sgd_multi")(entries, *hyper, self.grad_scale)
            else:
                for param, buf, first in entries:
                    dispatcher.dispatch(param.device.type, "sgd")(param, buf, first, *hyper)
