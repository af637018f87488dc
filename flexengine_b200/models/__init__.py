from . import fedutar, fuvozen, fuvuvik, qwen2  # noqa: F401  (register Fedutar, Fuvozen, Fuvuvik and Qwen2ForCausalLM)
