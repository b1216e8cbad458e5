"""Import-name compatibility: `turboquant_pytorch.validate` (reference src/turboquant_pytorch/validate.py)."""
from turboquant_b200.validate import main, run_validation  # noqa: F401

if __name__ == "__main__":
    main()
