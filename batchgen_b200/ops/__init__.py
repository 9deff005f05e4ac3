"""Hot operators.  ``ref`` holds the fp32 torch references; the other modules dispatch CUDA
tensors to the hand-written sm_100a kernels and CPU tensors to the references."""
from . import ref  # noqa: F401
