from turboquant_b200.plugin import TurboQuantAttentionBase  # noqa: F401
