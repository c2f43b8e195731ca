"""Architectures: each turns its typed configuration into a model description (data) and is
entered in the registry under the name its config.json carries.

An architecture that lives outside this package enters the same way: a module that calls
``register_architecture`` when it is imported.  For the command-line programs, which are processes of
their own, the variable ``ULTIMA_ARCH_MODULES`` names such modules (comma-separated, importable from
``sys.path``); they are imported here, after the package's own."""
import importlib
import os

from ..config.base import find_architecture
from . import qwen3  # registers Qwen3ForCausalLM

for _name in filter(None, (m.strip() for m in os.environ.get("ULTIMA_ARCH_MODULES", "").split(","))):
    importlib.import_module(_name)


def model_spec_for(config):
    """The ModelSpec of whatever architecture ``config`` belongs to."""
    return find_architecture(config.architecture).build_spec(config)


__all__ = ["model_spec_for"]
