"""Training glue (same public names as the reference ``tah.train`` package)."""
from tah_b200.model.loss import fixed_cross_entropy
from tah_b200.train.data_collator import CustomTaHDataCollator
from tah_b200.train.trainer import (CustomTaHTrainer, LoggerCallback, TaHTrainingArguments, TrainerCallback,
                                    TrainerState)

__all__ = ["CustomTaHDataCollator", "CustomTaHTrainer", "LoggerCallback", "fixed_cross_entropy",
           "TaHTrainingArguments", "TrainerCallback", "TrainerState"]
