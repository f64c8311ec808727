"""Helpers shared across the package: JSON/config utilities, profiling groups, memory and printing."""
from .config_utils import array2str, num2str, read_json_config, str2array, write_json_config  # noqa: F401
from .runtime_utils import (average_losses_across_data_parallel_group, get_batch_on_this_cp_rank,  # noqa: F401
                            get_batch_on_this_tp_rank, get_layernorm_offset, get_torch_version, is_torch_min_version,
                            log_single_rank, print_rank_0, rgetattr, rhasattr, rsetattr)
