from sample_efficient_gpt_b200.optim.adamw import AdamW, SGD  # noqa: F401
from sample_efficient_gpt_b200.optim.muon import Muon, NorMuon, NorMuonCWD  # noqa: F401
from sample_efficient_gpt_b200.optim.schedules import (  # noqa: F401
    get_cosine_lr,
    get_wsd_lr,
    get_seesaw_lr,
    muon_momentum_warmup,
)
from sample_efficient_gpt_b200.optim.clip import clip_grad_norm_, grad_norm  # noqa: F401
from sample_efficient_gpt_b200.optim.newton_schulz import newton_schulz, POLAR_EXPRESS_COEFFS  # noqa: F401
from sample_efficient_gpt_b200.optim.ema import WeightEMA  # noqa: F401
