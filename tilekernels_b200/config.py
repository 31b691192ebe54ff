"""SM-count knob with the API of the reference's tile_kernels/config.py:1-29 (get_num_sms, set_num_sms,
get_device_num_sms, get_max_smem_per_sm).

Only the clamp-counting variant of the fused SwiGLU cast sizes its grid from it; every other kernel asks the
C library, which queries the device itself."""
import torch

_limit = None        # SM count set by the caller, None = whole device
_properties = {}     # device index -> torch device properties, filled on first use


def _device_properties():
    index = torch.cuda.current_device()
    if index not in _properties:
        _properties[index] = torch.cuda.get_device_properties(index)
    return _properties[index]


def get_device_num_sms() -> int:
    """Streaming multiprocessors of the current device."""
    return _device_properties().multi_processor_count


def get_max_smem_per_sm() -> int:
    """Bytes of shared memory of one SM of the current device."""
    return _device_properties().shared_memory_per_multiprocessor


def set_num_sms(num_sms: int) -> None:
    """Limit the grids that honour the knob to `num_sms` SMs (1 .. device SM count)."""
    global _limit
    available = get_device_num_sms()
    assert 1 <= num_sms <= available, f'num_sms must be in 1..{available}'
    _limit = int(num_sms)


def get_num_sms() -> int:
    """The limit set by set_num_sms, or the device's SM count when none was set."""
    return get_device_num_sms() if _limit is None else _limit
