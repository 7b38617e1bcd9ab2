"""archscale_b200 — a Blackwell-native (sm_100a) LLM pretraining framework with the model
registry, flags, optimizers and checkpoint layout of microsoft/ArchScale."""
from archscale_b200.config import Config, get_parameters_count, name_to_config  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    if name == "GPT":
        from archscale_b200.models.gpt import GPT
        return GPT
    raise AttributeError(name)
