"""Helpers shared by the GPU parity tests."""
import importlib

import numpy as np
import torch


def mod(name):
    return importlib.import_module(f"mfu-fp4-training_b200.{name}")


def to_dev_bf16(x_f32: np.ndarray) -> torch.Tensor:
    """bf16-exact float32 numpy -> CUDA bfloat16 tensor with identical bits."""
    return torch.from_numpy(np.ascontiguousarray(x_f32)).to(torch.bfloat16).cuda()


def u8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).cpu().numpy()


def assert_status_ok():
    st = mod("_lib").device_status()
    assert st == 0, f"device status word = {st} (a kernel gave up a bounded wait)"
