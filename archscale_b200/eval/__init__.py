"""Evaluation: checkpoint loading by path convention, greedy/sampled generation, lm-eval adapter,
sliding-window perplexity (ProofPile) and the Phonebook retrieval probe."""
from .common import ModelWrapper, config_from_checkpoint_path, load_model  # noqa: F401
