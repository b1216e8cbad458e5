from turboquant_b200.families import deepseek, gpt2, llama, qwen2  # noqa: F401
