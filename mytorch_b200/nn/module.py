"""Module base class: parameter / buffer / sub-module registration, ``train``/``eval``, ``to``
(in place, returns None), ``state_dict`` / ``load_state_dict`` with dotted keys — the behaviour
of ``mytorch/nn/module.py:7-211``."""
import logging

from mytorch_b200.nn.parameter import Parameter
from mytorch_b200.tensor import Tensor

_log = logging.getLogger("mytorch_b200")


class Module:
    def __init__(self):
        object.__setattr__(self, "_parameters", {})
        object.__setattr__(self, "_buffers", {})
        object.__setattr__(self, "_modules", {})
        object.__setattr__(self, "training", True)

    # registration ---------------------------------------------------------
    def register_parameter(self, name, parameter):
        if parameter is not None:
            self._parameters[name] = parameter
        object.__setattr__(self, name, parameter)

    def register_buffer(self, name, buffer):
        if buffer is not None:
            self._buffers[name] = buffer
        object.__setattr__(self, name, buffer)

    def register_module(self, name, module):
        if module is not None:
            self._modules[name] = module
        object.__setattr__(self, name, module)

    def __setattr__(self, name, value):
        if isinstance(value, Module):
            self.register_module(name, value)
        elif isinstance(value, Parameter):
            self.register_parameter(name, value)
        elif isinstance(value, Tensor):
            self.register_buffer(name, value)
        else:
            object.__setattr__(self, name, value)

    # modes / movement -----------------------------------------------------
    def train(self, mode=True):
        self.training = mode
        for child in self.children():
            child.train(mode)
        return self

    def eval(self):
        return self.train(False)

    def to(self, device):
        for key in list(self._parameters):
            self.register_parameter(key, self._parameters[key].to(device))
        for key in list(self._buffers):
            self.register_buffer(key, self._buffers[key].to(device))
        for module in self._modules.values():
            module.to(device)

    # traversal ------------------------------------------------------------
    def named_modules(self, memo=None, prefix="", remove_duplicate=True):
        memo = set() if memo is None else memo
        if id(self) in memo:
            return
        if remove_duplicate:
            memo.add(id(self))
        yield prefix, self
        for name, module in self._modules.items():
            if module is not None:
                yield from module.named_modules(memo, f"{prefix}.{name}" if prefix else name, remove_duplicate)

    def _named_members(self, getter, prefix, recurse, remove_duplicate=True):
        seen = set()
        owners = self.named_modules(prefix=prefix, remove_duplicate=remove_duplicate) if recurse else [(prefix, self)]
        for mod_prefix, module in owners:
            for key, value in getter(module).items():
                if value is None or id(value) in seen:
                    continue
                if remove_duplicate:
                    seen.add(id(value))
                yield (f"{mod_prefix}.{key}" if mod_prefix else key), value

    def named_parameters(self, prefix="", recurse=True, remove_duplicate=True):
        yield from self._named_members(lambda m: m._parameters, prefix, recurse, remove_duplicate)

    def named_buffers(self, prefix="", recurse=True, remove_duplicate=True):
        yield from self._named_members(lambda m: m._buffers, prefix, recurse, remove_duplicate)

    def named_children(self):
        seen = set()
        for name, module in self._modules.items():
            if module is not None and id(module) not in seen:
                seen.add(id(module))
                yield name, module

    def parameters(self, recurse=True):
        for _, p in self.named_parameters(recurse=recurse):
            yield p

    def buffers(self, recurse=True):
        for _, b in self.named_buffers(recurse=recurse):
            yield b

    def children(self):
        for _, m in self.named_children():
            yield m

    # checkpoints ----------------------------------------------------------
    def state_dict(self, destination=None, prefix="", keep_vars=False):
        destination = {} if destination is None else destination
        for name, p in self._parameters.items():
            destination[prefix + name] = p if keep_vars else p.detach()
        for name, b in self._buffers.items():
            destination[prefix + name] = b if keep_vars else b.detach()
        for name, module in self._modules.items():
            module.state_dict(destination, prefix + name + ".", keep_vars)
        return destination

    def load_state_dict(self, state_dict):
        own = {}
        for k, v in self.named_parameters(remove_duplicate=False):
            own[k] = v
        for k, v in self.named_buffers(remove_duplicate=False):
            own[k] = v
        missing = [k for k in own if k not in state_dict]
        unexpected = [k for k in state_dict if k not in own]
        for k, v in state_dict.items():
            if k in own:
                own[k].copy_(v)
        if missing:
            _log.warning(f"Missing keys in module: {missing}")
        if unexpected:
            _log.warning(f"Unexpected keys in state_dict: {unexpected}")

    def forward(self, *args, **kwargs):
        raise NotImplementedError()

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)
