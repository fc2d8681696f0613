"""litetorch_b200: a Blackwell-native (sm_100a) LLM training and serving engine with the LiteTorch API.

    import litetorch_b200 as lt
    x = lt.Tensor.from_vector([...], [2, 3], lt.auto_device(), requires_grad=True)
    y = lt.Ops.gelu(lt.nn.Linear(3, 4).forward(x))

Sub-modules mirror the reference binding (src/bindings/python_bindings.cpp): `Ops, nn, optim, amp,
quantization, distributed, jit, data, cuda`; `models` and `Trainer` hold the Llama / GPT / MoE engines
that the benchmark configurations run.
"""
__version__ = "0.1.0"

from .core import (DataType, Device, DeviceType, NoGradGuard, Tensor, auto_device, checkpoint, get_backend_name,
                   is_gpu_available, is_tpu_available, manual_seed)
from .ops import Ops
from . import amp, config, cuda, custom_ops, data, jit, memory, nn, optim, quantization
from . import parallel as distributed
from .serialization import (load, load_optimizer_state, load_parameters, save, save_optimizer_state, save_parameters)

# dtype / device constants at module level, as in the reference
CPU, GPU, META, TPU = DeviceType.CPU, DeviceType.GPU, DeviceType.META, DeviceType.TPU
FP64, FP32, FP16, BF16 = DataType.FP64, DataType.FP32, DataType.FP16, DataType.BF16
INT16, INT8, INT4, NF4 = DataType.INT16, DataType.INT8, DataType.INT4, DataType.NF4
FP8_E4M3, FP8_E5M2, FP4_E2M1, FP4 = DataType.FP8_E4M3, DataType.FP8_E5M2, DataType.FP4_E2M1, DataType.FP4_E2M1

_cpu_cache_limit = [128 * 1024 * 1024]


def empty_cache() -> None:
    cuda.empty_cache()


def set_max_cpu_cache_size(nbytes: int) -> None:
    _cpu_cache_limit[0] = int(nbytes)


def get_cached_cpu_bytes() -> int:
    return 0


def get_cached_gpu_bytes() -> int:
    import torch
    if not torch.cuda.is_available():
        return 0
    return max(torch.cuda.memory_reserved() - torch.cuda.memory_allocated(), 0)


def get_gpu_memory_used() -> int:
    return cuda.memory_allocated()
