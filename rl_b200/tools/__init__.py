"""Command-line utilities: ``python -m rl_b200.tools.<name>``."""
