"""Helpers shared across the package: JSON/config utilities, profiling groups, memory and printing."""
from .config_utils import array2str, num2str, read_json_config, str2array, write_json_config  # noqa: F401
