from . import fuvozen, qwen2  # noqa: F401  (register Fuvozen and Qwen2ForCausalLM)
