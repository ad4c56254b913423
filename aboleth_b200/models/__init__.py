"""Model families served on the framework."""
from .mixtral import MixtralConfig, MixtralEP
