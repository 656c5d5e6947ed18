from sample_efficient_gpt_b200.training.data import MemoryMappedDataset  # noqa: F401
from sample_efficient_gpt_b200.training.checkpoint import save_checkpoint, load_model, load_optimizer  # noqa: F401
from sample_efficient_gpt_b200.training.loss import cross_entropy, efficient_cross_entropy  # noqa: F401
