from sample_efficient_gpt_b200.parallel.ddp import DDP, NaiveDDP, assign_buckets  # noqa: F401
from sample_efficient_gpt_b200.parallel.sharded_optimizer import ShardedOptimizer  # noqa: F401
