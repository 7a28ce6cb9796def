"""The torch-tensor wrappers of the C ABI live in the package (refactorgraph_b200/torch_ops.py); tests import them under
their old name."""
from refactorgraph_b200.torch_ops import *  # noqa: F401,F403
from refactorgraph_b200.torch_ops import DT, _bstrides, _pad4  # noqa: F401
