from turboquant_b200.plugin import (_REGISTRY, UnsupportedModelError, get_attention_class,  # noqa: F401
                                    register_family)
