"""SM-count knob (same API as the reference's tile_kernels/config.py:1-29).

Only the clamp-counting variant of the fused SwiGLU cast sizes its grid from it."""
import functools

import torch

_num_sms = 0


@functools.lru_cache(maxsize=None)
def get_device_num_sms() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


def set_num_sms(num_sms: int) -> None:
    global _num_sms
    assert 0 < num_sms <= get_device_num_sms()
    _num_sms = num_sms


def get_num_sms() -> int:
    return _num_sms if _num_sms else get_device_num_sms()


@functools.lru_cache(maxsize=None)
def get_max_smem_per_sm() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).shared_memory_per_multiprocessor
