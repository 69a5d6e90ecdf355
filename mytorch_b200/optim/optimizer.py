"""Parameter groups, ``zero_grad`` (drops the gradient tensors), ``state_dict`` /
``load_state_dict`` keyed by parameter identity and re-mapped by position
(``mytorch/optim/optimizer.py:6-82``)."""
from mytorch_b200.tensor import Tensor


class Optimizer:
    def __init__(self, params, defaults):
        self.param_groups = []
        self.defaults = defaults
        self.state = {}
        groups = list(params)
        if not isinstance(groups[0], dict):
            groups = [{"params": groups}]
        for g in groups:
            self._add_param_group(g)

    def _add_param_group(self, group):
        group["params"] = list(group["params"])
        for k, v in self.defaults.items():
            group.setdefault(k, v)
        for p in group["params"]:
            if not isinstance(p, Tensor):
                raise RuntimeError(f"There's a non-tensor value in params: {p}")
        existing = {id(p) for g in self.param_groups for p in g["params"]}
        if existing & {id(p) for p in group["params"]}:
            raise RuntimeError("Param groups have overlap")
        self.param_groups.append(group)

    def zero_grad(self):
        for g in self.param_groups:
            for p in g["params"]:
                p.grad = None

    def state_dict(self):
        groups = []
        for g in self.param_groups:
            ng = {k: v for k, v in g.items() if k != "params"}
            ng["params"] = [id(p) for p in g["params"]]
            groups.append(ng)
        return {"state": {id(p): s for p, s in self.state.items()}, "param_groups": groups}

    def load_state_dict(self, state_dict):
        state, groups = state_dict["state"], state_dict["param_groups"]
        if len(groups) != len(self.param_groups):
            raise RuntimeError("Optimizer state_dict has a different param group length from the loaded one")
        for mine, theirs in zip(self.param_groups, groups):
            if len(mine["params"]) != len(theirs["params"]):
                raise RuntimeError("Optimizer state_dict is different from the loaded one")
        for mine, theirs in zip(self.param_groups, groups):
            for p, key in zip(mine["params"], theirs["params"]):
                if state.get(key) is not None:
                    self.state[p] = state[key]
