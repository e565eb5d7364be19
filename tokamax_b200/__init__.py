"""B200-native `ragged_dot` with the API of openxla/tokamax (tokamax/__init__.py:18-41).

The compute path is a C-ABI shared library of hand-written sm_100a CUDA kernels
(`tokamax_b200/csrc`, declared in `include/tokamax_b200.h`); this package is the host
side: argument handling, configs, autotuning and benchmarking.
"""

from tokamax_b200 import config
from tokamax_b200.autotuning import AutotuningResult, autotune
from tokamax_b200.benchmarking import BenchmarkData, benchmark, standardize_function
from tokamax_b200.op import BoundArguments, Op
from tokamax_b200.quantization import AsQArray, QArray, quantize_per_channel
from tokamax_b200.ragged_dot import (
    GroupSizes as RaggedDotGroupSizes,
    generate_group_sizes as generate_ragged_dot_group_sizes,
    HostRaggedDot,
    ragged_dot,
    ragged_dot_general,
    ragged_dot_host,
)

__all__ = [
    "AsQArray", "AutotuningResult", "BenchmarkData", "BoundArguments", "HostRaggedDot", "Op", "QArray",
    "RaggedDotGroupSizes", "autotune", "benchmark", "config",
    "generate_ragged_dot_group_sizes", "quantize_per_channel", "ragged_dot",
    "ragged_dot_general", "ragged_dot_host", "standardize_function",
]
