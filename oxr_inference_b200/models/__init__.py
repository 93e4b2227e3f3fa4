"""Architectures this package knows; importing the package registers them."""

from oxr_inference_b200.models import qwen3  # noqa: F401
