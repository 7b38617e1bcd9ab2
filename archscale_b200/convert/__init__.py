"""Checkpoint converters between the lit layout of this package and Hugging Face Llama-style layouts."""
from .hf import hf_config_from_lit, hf_to_lit, lit_to_hf  # noqa: F401
