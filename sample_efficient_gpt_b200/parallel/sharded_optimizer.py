"""ZeRO-1 style optimizer wrapper: each rank steps a contiguous share of the parameters and the
updated values are broadcast from their owners.

Counterpart of training/distributed/sharded_optimizer.py:6-102 of the reference (unused there).
The Muon family has its own, finer sharding (``optim.muon`` with ``shard=True``); this wrapper is
for element-wise optimizers such as AdamW.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class ShardedOptimizer(torch.optim.Optimizer):
    def __init__(self, params, optimizer_cls, **kwargs):
        params = list(params)
        assert dist.is_initialized()
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.all_params = params
        per = -(-len(params) // self.world)
        self.owner = [min(i // per, self.world - 1) for i in range(len(params))]
        mine = [p for p, o in zip(params, self.owner) if o == self.rank]
        self.inner = optimizer_cls(mine, **kwargs) if mine else None
        super().__init__(params, kwargs)

    @torch.no_grad()
    def step(self, closure=None):
        out = None
        if self.inner is not None:
            for g_outer in self.param_groups:  # propagate schedule changes
                for g in self.inner.param_groups:
                    for k, v in g_outer.items():
                        if k != "params":
                            g[k] = v
            out = self.inner.step(closure)
        works = [dist.broadcast(p.data, src=o, async_op=True) for p, o in zip(self.all_params, self.owner)]
        for w in works:
            w.wait()
        return out

    def state_dict(self):
        """Full (unsharded) state, identical on every rank; a collective call."""
        local = self.inner.state_dict() if self.inner is not None else {"state": {}, "param_groups": []}
        gathered = [None] * self.world
        dist.all_gather_object(gathered, local["state"])
        merged, idx = {}, 0
        counts = [self.owner.count(r) for r in range(self.world)]
        for r, st in enumerate(gathered):
            for k in range(counts[r]):
                if k in st:
                    merged[idx + k] = st[k]
            idx += counts[r]
        groups = [{**{k: v for k, v in g.items() if k != "params"}, "params": list(range(len(self.all_params)))} for g in self.param_groups]
        return {"state": merged, "param_groups": groups}
