"""Importing this package registers every family adapter."""
from . import deepseek, gpt2, llama, qwen2  # noqa: F401
