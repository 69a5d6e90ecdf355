"""``save`` / ``load``: pickle in which every Tensor is stored by ``persistent_id`` as
``("MyTorchTensor", device string, NumPy array in logical layout)`` — the file format of the
reference's ``mytorch/serialization.py:6-38``, so checkpoints move between the two."""
import pickle


class _Pickler(pickle.Pickler):
    def persistent_id(self, obj):
        from mytorch_b200.tensor import Tensor

        if isinstance(obj, Tensor):
            return ("MyTorchTensor", repr(obj.device), obj._host_array())
        return None


class _Unpickler(pickle.Unpickler):
    def __init__(self, file, map_location=None):
        super().__init__(file)
        self.map_location = map_location

    def persistent_load(self, pid):
        from mytorch_b200.tensor import Tensor

        tag, device, array = pid
        if tag != "MyTorchTensor":
            raise pickle.UnpicklingError(f"unsupported persistent object {tag}")
        return Tensor(cpu_array=array, device=self.map_location or device)

    def find_class(self, module, name):
        if module == "mytorch" or module.startswith("mytorch."):
            module = "mytorch_b200" + module[len("mytorch"):]
        return super().find_class(module, name)


def save(obj, path):
    with open(path, "wb") as f:
        _Pickler(f).dump(obj)


def load(path, map_location=None):
    with open(path, "rb") as f:
        return _Unpickler(f, map_location).load()
