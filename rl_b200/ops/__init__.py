"""Operators: native sm_100a kernels behind tensor-level functions with PyTorch restatements for CPU."""

from . import functional  # noqa: F401

try:  # installs the native attention behind functional.attention_varlen when the library is present
    from . import attention  # noqa: F401
except Exception:  # the library is absent (pure-CPU checkout): the PyTorch restatement stays in place
    pass
