"""B200-native dense-layer path: fused GEMM + bias + activation forward, its backward and the
strided-batched form, behind the reference's operator interface.

`ops_gemm` mirrors graph_executor_v2/python/graph_executor_v2/ops/gemm.py (forward, backward, forward_into,
backward_into), `ops_conv2d` mirrors ops/conv2d.py on the same kernels, and `Dense` mirrors layers/dense_gemm.py;
all call the CUDA library through its C ABI.
There is no CPU fallback: importing works anywhere, computing needs the built library and a CUDA device.
"""
from . import _lib  # noqa: F401
from . import ops_gemm  # noqa: F401
from . import ops_conv2d  # noqa: F401
from . import ops_sdpa  # noqa: F401
from .dense import Dense  # noqa: F401
from . import train  # noqa: F401
from . import data_parallel  # noqa: F401
from .train import DenseStackTrainer, MlpPlan, softmax_ce_fused, sgd_update  # noqa: F401
from ._lib import load_library, library_path  # noqa: F401

__all__ = ["ops_gemm", "ops_conv2d", "ops_sdpa", "Dense", "train", "data_parallel", "DenseStackTrainer", "MlpPlan", "softmax_ce_fused", "sgd_update", "load_library",
           "library_path"]
