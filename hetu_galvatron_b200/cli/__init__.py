"""Command-line entry points: ``python -m hetu_galvatron_b200.cli.<name> <config.yaml> [dotted.key=value ...]``."""
