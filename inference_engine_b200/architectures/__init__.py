from . import llama, rugedra  # noqa: F401 (register LlamaForCausalLM and Rugedra)
