"""SM-count knob with the API of the reference's tile_kernels/config.py:1-29 (get_num_sms, set_num_sms,
get_device_num_sms, get_max_smem_per_sm).

Only the clamp-counting variant of the fused SwiGLU cast sizes its grid from it; every other kernel asks the
C library, which queries the device itself.

One knob has no counterpart in the reference: set_exact_swiglu_codes (see there)."""
import torch

_limit = None        # SM count set by the caller, None = whole device
_exact_swiglu_codes = False
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


def set_exact_swiglu_codes(exact: bool) -> None:
    """Choose how swiglu_forward_and_per_token_cast evaluates the activation.

    False (default): scales are exact; the FP8 codes come from hardware-approximate exp and reciprocal, so
    about one code in a million lies one step from the exactly evaluated one.
    True: every activation goes through the exact routine (bit-identical to the CPU checker), at roughly half
    the speed."""
    global _exact_swiglu_codes
    _exact_swiglu_codes = bool(exact)


def get_exact_swiglu_codes() -> bool:
    return _exact_swiglu_codes
