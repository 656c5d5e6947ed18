"""126M GQA model (configs/gpt_126m.py:5-42 of the reference)."""

from sample_efficient_gpt_b200.config_schema import Config, DataConfig, ModelConfig, OptimConfig, TrainerConfig

cfg = Config(
    data=DataConfig(batch_size=24, val_batch_size=48, context_length=512, seed=42),
    model=ModelConfig(
        vocab_size=32000,
        d_model=1024,
        d_ff=2304,
        n_layers=12,
        n_heads=16,
        n_kv_heads=8,
        attn_qknorm=True,
        attn_val_residual=True,
        layernorm_scaling=True,
    ),
    optim=OptimConfig(
        lr=5.25e-3,
        lr_min_coeff=5e-2,
        wd=0.0,
        betas=(0.95, 0.99),
        use_muon=True,
        muon_lr=1.125e-2,
        muon_wd=1.5e-3,
        muon_wd_min=1.5e-4,
    ),
    trainer=TrainerConfig(
        dtype="bfloat16", max_steps=24000, gradient_accumulation_steps=8, log_every=50, save_every=4000, val_every=3000
    ),
)
