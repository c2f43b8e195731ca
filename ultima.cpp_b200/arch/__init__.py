"""Architectures: each turns its typed configuration into a model description (data) and is
entered in the registry under the name its config.json carries."""
from ..config.base import find_architecture
from . import qwen3  # registers Qwen3ForCausalLM


def model_spec_for(config):
    """The ModelSpec of whatever architecture ``config`` belongs to."""
    return find_architecture(config.architecture).build_spec(config)


__all__ = ["model_spec_for"]
