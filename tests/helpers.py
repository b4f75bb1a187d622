"""Shared builders for the tests."""
import torch

from tah_b200 import TaHConfig, TaHForCausalLM
from tah_b200.models import Qwen3ForCausalLM, export_hf_state_dict, preset


def tiny_tah(max_iter=2, r=8, decider="IterLabelDecider", decider_kwargs=None, train_loss="NextTokenPredLoss",
             train_loss_kwargs=None, seed=0, dtype=torch.float32, randomize_lora_b=True, device=None, **cfg_over):
    torch.manual_seed(seed)
    cfg = preset("tiny", torch_dtype=str(dtype).replace("torch.", ""), **cfg_over)
    base = Qwen3ForCausalLM(cfg, device=device)
    tc = TaHConfig(max_iter=max_iter, iter_decider=decider, iter_decider_kwargs=decider_kwargs or {},
                   adapter_kwargs=dict(r=r, lora_alpha=2 * r, lora_dropout=0.0, target_modules="all-linear"),
                   train_loss=train_loss, train_loss_kwargs=train_loss_kwargs or {},
                   input_updater_kwargs={"topk": 100})
    model = TaHForCausalLM(base, tc)
    if randomize_lora_b:
        # LoRA B starts at zero (adapter = no-op); give it values so that pass >= 1 differs from pass 0
        with torch.no_grad():
            for n, p in model.named_parameters():
                if "lora_B" in n:
                    p.normal_(std=0.05)
    if device is not None:
        model = model.to(device)
    return model


def oracle_weights(model):
    from tests.oracle.tah_oracle import OracleWeights
    base, lora = export_hf_state_dict(model.simple_base_model)
    spec = model.simple_base_model.lora
    return OracleWeights(base, lora, model.config, spec.r, spec.lora_alpha)
