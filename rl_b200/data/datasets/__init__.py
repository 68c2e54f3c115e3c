"""Dataset registry: ``data.train.dataset_name`` -> dataset builder."""

from .synthetic import RandomTokenPromptDataset  # noqa: F401
