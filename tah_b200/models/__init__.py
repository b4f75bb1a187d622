"""Backbone model families (Qwen3 0.6B / 1.7B / 4B shapes and the tiny test model)."""
from tah_b200.models.qwen3 import (PRESETS, LoRASpec, Qwen3Config, Qwen3ForCausalLM, attach_lora,
                                   export_hf_state_dict, from_hf_model, import_hf_state_dict, preset)

__all__ = ["PRESETS", "LoRASpec", "Qwen3Config", "Qwen3ForCausalLM", "attach_lora", "export_hf_state_dict",
           "from_hf_model", "import_hf_state_dict", "preset"]
