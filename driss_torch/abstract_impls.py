"""The fake-tensor registrations under the reference's module name (driss_torch/abstract_impls.py)."""
from driss_torch_b200.abstract_impls import *  # noqa: F401,F403
