from . import llama, ravapel, rugedra  # noqa: F401 (register LlamaForCausalLM, Ravapel and Rugedra)
