from .llama import LlamaConfig, LlamaDecoder  # noqa: F401
