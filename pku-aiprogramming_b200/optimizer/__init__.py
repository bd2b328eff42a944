"""Python autograd layer in the reference's shape: `Tensor` nodes holding NumPy data, `TensorOp`
subclasses with `compute`/`gradient`, reverse-mode `backward`, and the `Attention` op that
runs on the B200 kernels through the `myTensor`/`myLayer` modules."""
from .engine import Op, Value, backward_pass, topological_order  # noqa: F401
from .operators import *  # noqa: F401,F403
