from . import fuvozen, fuvuvik, qwen2  # noqa: F401  (register Fuvozen, Fuvuvik and Qwen2ForCausalLM)
