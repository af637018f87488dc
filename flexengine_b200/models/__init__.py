from . import fedutar, fuvozen, fuvuvik, qwen2, rikolix  # noqa: F401  (register Fedutar, Fuvozen, Fuvuvik, Rikolix and Qwen2ForCausalLM)
