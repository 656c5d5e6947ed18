from sample_efficient_gpt_b200.models.transformer import Transformer, Block, build_model  # noqa: F401
from sample_efficient_gpt_b200.models.attention import KVCache, MultiHeadSelfAttention  # noqa: F401
