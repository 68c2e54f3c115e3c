"""Typed configuration schema of the recipes (``schema.py``)."""

from .schema import ConfigError, Field, Report, validate, validate_master_config  # noqa: F401
