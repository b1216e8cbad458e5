"""Import-name compatibility: `transformers_turboquant.cli` (reference src/transformers_turboquant/cli.py)."""
from turboquant_b200.cli import app, validate  # noqa: F401

if __name__ == "__main__":
    app()
