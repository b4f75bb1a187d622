"""tah_b200: a Blackwell-native Think-at-Hard framework.

Top-level names mirror the reference package (reference ``tah/__init__.py:12-21``).
"""
from tah_b200.model import (IterDeciderLoss, IterLabelDecider, MLPIterDecider, NextTokenPredLoss, TaHCache,
                            TaHCausalLMOutputWithPast, TaHConfig, TaHForCausalLM)

__version__ = "0.1.0"
__all__ = ["TaHForCausalLM", "TaHConfig", "TaHCache", "TaHCausalLMOutputWithPast", "IterLabelDecider",
           "MLPIterDecider", "NextTokenPredLoss", "IterDeciderLoss"]
