"""Core TaH model layer (same public names as the reference ``tah.model`` package)."""
from tah_b200.model.causal_cache import TaHCache
from tah_b200.model.iter_decider import (ITER_DECIDER_BY_NAME, BernoulliIterDecider, IterDecider,
                                         IterLabelDecider, MLPIterDecider, SimpleMLPIterDecider,
                                         get_iter_decider_class, load_iter_decider, save_iter_decider)
from tah_b200.model.loss import (LOSS_BY_NAME, CombinedLoss, IterDeciderLoss, LossFunc, NextTokenPredLoss,
                                 get_loss_func_class)
from tah_b200.model.tah_config import TaHConfig
from tah_b200.model.tah_model import (TaHCausalLMOutputWithPast, TaHForCausalLM, additive_logits_update,
                                      gather_active, scatter_back, topk_softmax_input_update)

__all__ = [
    "TaHCache", "ITER_DECIDER_BY_NAME", "IterDecider", "IterLabelDecider", "MLPIterDecider",
    "SimpleMLPIterDecider", "BernoulliIterDecider", "get_iter_decider_class", "load_iter_decider",
    "save_iter_decider", "LOSS_BY_NAME", "LossFunc", "NextTokenPredLoss", "IterDeciderLoss", "CombinedLoss",
    "get_loss_func_class", "TaHConfig", "TaHForCausalLM", "TaHCausalLMOutputWithPast",
    "topk_softmax_input_update", "additive_logits_update", "gather_active", "scatter_back",
]
