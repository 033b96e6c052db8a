from . import gpt2  # registers GPT2LMHeadModel
from . import lebedra  # registers Lebedra
from . import porovik  # registers Porovik
from . import fikevik  # registers Fikevik
from . import soporax  # registers Soporax
from .model import Layer, Model, named_params_of_spec

__all__ = ["Layer", "Model", "named_params_of_spec", "gpt2", "lebedra", "porovik", "fikevik", "soporax"]
