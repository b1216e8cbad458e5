from turboquant_b200.plugin import apply_turboquant  # noqa: F401
