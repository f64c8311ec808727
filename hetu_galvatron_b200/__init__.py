"""Blackwell-native automatic hybrid-parallel training (profiler -> strategy search -> runtime).

Sub-packages: ``config`` (YAML + dotted overrides -> Pydantic), ``search`` (strategy enumeration,
cost models, dynamic-programming search), ``profiler`` (hardware / model / runtime profilers),
``parallel`` (process groups, TP/SP mappings, ZeRO manager, pipeline schedules, resharding),
``models`` (generic decoder stack, MoE), ``ops`` (sm_100a kernels + autograd), ``runtime``
(initialisation, optimizer, data, checkpoints, rerun state machine), ``cli`` (entry points).
"""
__version__ = "0.1.0"
