"""~70M ablation model; also the ``base:`` of the IMU-1 YAML files (configs/gpt_small_faster.py:5-32)."""

from sample_efficient_gpt_b200.config_schema import Config, DataConfig, ModelConfig, OptimConfig, TrainerConfig

cfg = Config(
    data=DataConfig(batch_size=96, val_batch_size=192, context_length=384, seed=42),
    model=ModelConfig(
        vocab_size=32000,
        d_model=768,
        d_ff=2048,
        n_layers=8,
        n_heads=12,
        attn_qknorm=True,
        attn_val_residual=True,
        layernorm_scaling=True,
    ),
    optim=OptimConfig(
        lr=7e-3, lr_min_coeff=1e-2, wd=0.0, betas=(0.95, 0.99), use_muon=True, muon_lr=1.5e-2, muon_wd=1e-4
    ),
    trainer=TrainerConfig(
        dtype="bfloat16", max_steps=24000, gradient_accumulation_steps=2, log_every=50, save_every=4000, val_every=3000
    ),
)
