"""String-keyed operator registry: ``(backend, op_name) -> callable``.

Same contract as ``mytorch/backends/backend_dispatcher.py:22-39``: registration by decorator,
duplicate registration raises, dispatch of an unknown pair raises ``RuntimeError``.  The CUDA
entries call the sm_100a kernel library; the ``cpu`` entries cover host-side storage only
(allocation, fill, random init, copy, cast, reshape) — there is no CPU compute backend.
"""


class BackendDispatcher:
    _instance = None

    @classmethod
    def instance(cls):
        if cls._instance is None:
            cls._instance = cls()
            cls._instance._load_backends()
        return cls._instance

    def __init__(self):
        self._impls = {}

    def _load_backends(self):
        import mytorch_b200.backends.cpu  # noqa: F401
        import mytorch_b200.backends.cuda  # noqa: F401

    def register_backend_function(self, backend, op_name):
        def decorator(func):
            table = self._impls.setdefault(backend, {})
            if op_name in table:
                raise RuntimeError(f"There's already a function registered for {op_name} on {backend} backend")
            table[op_name] = func
            return func

        return decorator

    def dispatch(self, backend, op_name):
        try:
            return self._impls[backend][op_name]
        except KeyError:
            raise RuntimeError(f"There's no function registered for {op_name} on {backend} backend") from None
