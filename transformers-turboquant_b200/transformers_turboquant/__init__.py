"""Import-name compatibility: `from transformers_turboquant import apply_turboquant`
resolves to the B200 implementation when this directory is on sys.path."""
from turboquant_b200 import apply_turboquant, families  # noqa: F401

__version__ = "0.1.0"
__all__ = ["apply_turboquant"]
