from . import env  # noqa: F401  (registers allocate_memory / transfer_memory)
from . import ops  # noqa: F401  (registers every CUDA operator)
