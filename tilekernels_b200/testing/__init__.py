"""Comparison helpers and input generators for the quant tests (counterpart of the
reference's tile_kernels/testing package, restricted to what the quant casts use)."""
from .generator import generate_e5m6_inputs, generate_hidden_sizes, generate_num_tokens, make_config_input  # noqa: F401
from .numeric import assert_equal, calc_diff, check_bias, count_bytes  # noqa: F401
from .quant import clear_unused_sf  # noqa: F401
