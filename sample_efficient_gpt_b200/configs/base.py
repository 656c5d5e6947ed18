"""All-defaults config (configs/base.py of the reference)."""

from sample_efficient_gpt_b200.config_schema import Config, DataConfig, ModelConfig, OptimConfig, TrainerConfig

cfg = Config(DataConfig(), ModelConfig(), OptimConfig(), TrainerConfig())
