"""Checkpoints of expert-parallel runs in the layout of a single-process run.

Under ``trainer.dist_mode=ddp_ep`` a rank holds ``E / world`` experts per block and a third optimizer that steps them.
A file written from rank 0's objects alone would contain only that rank's experts.  ``gather_full_state`` collects every
rank's experts and their NorMuon state on rank 0 and lays them out exactly as a process holding all experts would:
model keys ``...experts.up.{g}`` / ``...experts.down.{g}`` for all global ids ``g``, two optimizers (AdamW, then one
Muon-family optimizer over every matrix including the experts, one parameter group per shape).  ``split_muon_state`` is
the way back: from such a file, the state of the shared matrices and of this rank's experts in the layout of the two
Muon-family optimizers of an expert-parallel trainer - for any world size that divides E.

The reference has no mixture of experts; the file layout it defines (training/checkpoint.py:22-88) is kept.
"""

from __future__ import annotations

import re

import torch
import torch.distributed as dist

_EXPERT = re.compile(r"^(.*\.experts\.(?:up|down)\.)(\d+)$")
_ADAM_NAMES = ("embedding", "lm_head", ".router.")


def full_matrix_names(local_named: list[tuple[str, torch.Size]], n_local: int, world: int) -> list[tuple[str, int | None, str]]:
    """The Muon-family parameters of the full model, in the order ``named_parameters()`` of a process that holds all experts
    lists them: ``(global name, owner rank or None for replicated matrices, the owner's local name)``.

    ``local_named``: (name, shape) of this rank's ``named_parameters()`` - every rank has the same block structure with its
    own ``n_local`` experts named ``0 .. n_local-1``."""
    out: list[tuple[str, int | None, str]] = []
    for name, shape in local_named:
        if len(shape) < 2 or any(k in name for k in _ADAM_NAMES):
            continue
        m = _EXPERT.match(name)
        if m is None:
            out.append((name, None, name))
        elif int(m.group(2)) == 0:  # first local expert of this kind: all global experts of the kind go here
            for g in range(n_local * world):
                out.append((f"{m.group(1)}{g}", g // n_local, f"{m.group(1)}{g % n_local}"))
    return out


def _shape_groups(shapes: list[torch.Size]) -> list[list[int]]:
    """Indices grouped the way the Muon family builds its parameter groups: one group per distinct shape, groups in the
    iteration order of the set of shapes (optim/muon.py, ``Muon.__init__``)."""
    order = {s for s in shapes}
    return [[i for i, s in enumerate(shapes) if s == size] for size in order]


def _muon_param_state(opt, p) -> dict:
    st = opt.state.get(p, {})
    return {k: (v.detach().cpu().clone() if torch.is_tensor(v) else v) for k, v in st.items()}


def gather_experts(state: dict, model, ep_group) -> dict | None:
    """Collective.  ``state``: a state dict of this rank's model layout (global expert keys, as ``model.state_dict()`` and the
    weight average produce them); returns it completed with every other rank's expert entries on rank 0, None elsewhere."""
    world, rank = dist.get_world_size(ep_group), dist.get_rank(ep_group)
    mine = {k: v.detach().cpu() for k, v in state.items() if _EXPERT.match(k)}
    gathered: list | None = [None] * world if rank == 0 else None
    dist.gather_object(mine, gathered, dst=_group_root(ep_group), group=ep_group)
    if rank != 0:
        return None
    out = {k: v.detach().cpu() for k, v in state.items()}
    for part in gathered:
        out.update(part)
    return out


def _group_root(ep_group) -> int:
    return 0 if ep_group is dist.group.WORLD else dist.get_global_rank(ep_group, 0)


def gather_full_state(model, optimizers, ep_group) -> tuple[dict, list[dict]] | None:
    """Collective over ``ep_group``.  Returns ``(model_state_dict, [adamw_sd, muon_sd])`` for the full model on rank 0 of the
    group and None elsewhere.  ``optimizers`` = [AdamW, shared Muon-family, local-expert Muon-family]."""
    world, rank = dist.get_world_size(ep_group), dist.get_rank(ep_group)
    adam, shared_opt, local_opt = optimizers
    named = list(model.named_parameters())
    first = next(m for m in model.modules() if hasattr(m, "first_global_id"))
    n_local = len(first.up)
    mine: dict[str, tuple[torch.Tensor, dict]] = {}
    for name, p in named:
        m = _EXPERT.match(name)
        if m is not None:
            g = rank * n_local + int(m.group(2))
            mine[f"{m.group(1)}{g}"] = (p.detach().cpu().clone(), _muon_param_state(local_opt, p))
    gathered: list | None = [None] * world if rank == 0 else None
    dist.gather_object(mine, gathered, dst=_group_root(ep_group), group=ep_group)
    if rank != 0:
        return None
    experts: dict[str, tuple[torch.Tensor, dict]] = {}
    for part in gathered:
        experts.update(part)
    model_sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    for gname, (tensor, _) in experts.items():
        model_sd[gname] = tensor
    # the Muon-family optimizer of a process that holds everything
    by_name = dict(named)
    names = full_matrix_names([(n, p.shape) for n, p in named], n_local, world)
    shapes = [experts[g][0].shape if owner is not None else by_name[g].shape for g, owner, _ in names]
    groups = _shape_groups(shapes)
    hyper = {k: v for k, v in shared_opt.param_groups[0].items() if k != "params"}
    state, param_groups, next_id = {}, [], 0
    for members in groups:
        ids = []
        for i in members:
            gname, owner, _ = names[i]
            st = experts[gname][1] if owner is not None else _muon_param_state(shared_opt, by_name[gname])
            if st:
                state[next_id] = st
            ids.append(next_id)
            next_id += 1
        param_groups.append({**hyper, "params": ids})
    return model_sd, [adam.state_dict(), {"state": state, "param_groups": param_groups}]


def split_muon_state(saved: dict, model, shared_opt, local_opt, ep_group) -> tuple[dict, dict]:
    """From the Muon-family state of a full-model file, the state dicts that ``shared_opt`` (replicated matrices) and
    ``local_opt`` (this rank's experts) load."""
    world, rank = dist.get_world_size(ep_group), dist.get_rank(ep_group)
    named = list(model.named_parameters())
    first = next(m for m in model.modules() if hasattr(m, "first_global_id"))
    n_local = len(first.up)
    names = full_matrix_names([(n, p.shape) for n, p in named], n_local, world)
    by_name = dict(named)
    shapes = [by_name[local].shape for _, _, local in names]
    flat_ids = [pid for g in saved["param_groups"] for pid in g["params"]]
    order = [i for members in _shape_groups(shapes) for i in members]
    if len(flat_ids) != len(order):
        raise ValueError(f"optimizer state covers {len(flat_ids)} matrices, the full model has {len(order)}")
    saved_id_of = {names[i][0]: pid for i, pid in zip(order, flat_ids)}
    name_of_param = {p: n for n, p in named}

    def build(opt, to_global):
        cur = opt.state_dict()
        out_state = {}
        for g_cur, g_obj in zip(cur["param_groups"], opt.param_groups):
            for pid, p in zip(g_cur["params"], g_obj["params"]):
                st = saved["state"].get(saved_id_of[to_global(name_of_param[p])])
                if st:
                    out_state[pid] = st
        return {"state": out_state, "param_groups": cur["param_groups"]}

    def expert_global(name):
        m = _EXPERT.match(name)
        return f"{m.group(1)}{rank * n_local + int(m.group(2))}"

    return build(shared_opt, lambda n: n), build(local_opt, expert_global)
