"""Training orchestration.

Public surface of the reference ``Trainer`` (training/trainer.py:54-678): ``Trainer(cfg, load_from,
load_components, compile, wandb, **overrides)``, ``train()``, ``train_step()``, ``validate()``,
``generate()``, ``save_state()``, ``load_state()``.  Behaviour that shapes the loss curve is kept:
seeds ``42 + rank``; fp32 master weights; loss coefficient ``1/GA * local_bs/global_bs`` with
SUM-reduced gradients; AdamW for every tensor with fewer than two dimensions plus embedding and head,
(Nor)Muon for the other matrices; WSD / cosine / seesaw schedules per iteration; Muon momentum warm-up
over 300 iterations; gradient clipping that only reports the norm unless ``trainer.clip_fix``; optimizer
step every ``gradient_accumulation_steps`` iterations; checkpoints at ``save_every`` (including
iteration 0) and at the end; validation on the logging rank.

What is different: on a GPU (and on CPU for dense models) the step runs through the hand-scheduled
``FusedEngine`` instead of autograd + a tracing compiler; step time is measured with CUDA events;
training works on CPU and with the gloo backend; there are an in-training weight EMA, optional sharding of
the Muon step, a JSONL metrics sink, a step watchdog and a non-finite-loss guard.
"""

from __future__ import annotations

import math
import os
import random
import time
from contextlib import nullcontext
from pathlib import Path
from typing import Any

import numpy as np
import torch
import torch.distributed as dist
from torch import Tensor

from sample_efficient_gpt_b200.config_schema import Config
from sample_efficient_gpt_b200.models import build_model
from sample_efficient_gpt_b200.optim import (
    AdamW,
    Muon,
    NorMuon,
    NorMuonCWD,
    WeightEMA,
    clip_grad_norm_,
    get_cosine_lr,
    get_seesaw_lr,
    get_wsd_lr,
    grad_norm,
    muon_momentum_warmup,
)
from sample_efficient_gpt_b200.parallel.ddp import DDP
from sample_efficient_gpt_b200.training.checkpoint import load_model, load_optimizer, save_checkpoint
from sample_efficient_gpt_b200.training.data import MemoryMappedDataset
from sample_efficient_gpt_b200.training.engine import FusedEngine, engine_supports
from sample_efficient_gpt_b200.training.loss import efficient_cross_entropy, fused_linear_cross_entropy
from sample_efficient_gpt_b200.utils import metrics as M
from sample_efficient_gpt_b200.utils.config_tools import apply_overrides, load_config
from sample_efficient_gpt_b200.utils.fault import NonFiniteGuard, StepWatchdog
from sample_efficient_gpt_b200.utils.logger import logger
from sample_efficient_gpt_b200.utils.profiling import mem


def _load_tokenizer(path: str):
    if not path:
        return None
    try:
        from transformers import PreTrainedTokenizerFast

        return PreTrainedTokenizerFast.from_pretrained(path)
    except Exception as e:  # offline box without the files
        logger.warning(f"tokenizer {path!r} unavailable ({type(e).__name__}); bits-per-byte is not reported")
        return None


class Trainer:
    def __init__(
        self,
        cfg: Config | None = None,
        load_from: str | None = None,
        load_components: str = "all",
        compile: bool = False,
        wandb: Any | None = None,
        **cfg_overrides,
    ):
        self.is_distributed = dist.is_available() and dist.is_initialized()
        self.world_size = dist.get_world_size() if self.is_distributed else 1
        self.rank = dist.get_rank() if self.is_distributed else 0
        self.target_log_rank = 0

        seed = 42 + self.rank
        random.seed(seed)
        np.random.seed(seed)
        torch.manual_seed(seed)

        if cfg is None:
            assert load_from is not None, "you must load from checkpoint if cfg is None"
            cfg = load_config(torch.load(load_from, map_location="cpu", weights_only=False)["config"])
            cfg = apply_overrides(cfg, cfg_overrides)
            logger.info(f"Loading from the checkpoint, device={cfg.trainer.device}")
        elif cfg_overrides:
            cfg = apply_overrides(cfg, cfg_overrides)
        self.cfg = cfg
        tc = cfg.trainer
        if tc.use_fp8:
            logger.warning("use_fp8 only changes the MFU denominator (as in the reference); compute stays bf16")
        if cfg.data.mode == "sft":
            raise NotImplementedError("data.mode='sft' has no dataset implementation (the reference's is absent too)")
        self.device = torch.device(tc.device)
        if self.device.type == "cuda":
            torch.cuda.manual_seed_all(seed)
            if self.device.index is None:
                self.device = torch.device("cuda", torch.cuda.current_device())
        self.act_dtype = torch.bfloat16 if tc.dtype == "bfloat16" else torch.float32
        self.iteration = 0
        self.run_id = None
        self.engine: FusedEngine | None = None
        self.optimizers = None
        self.wandb = wandb
        if wandb is None and tc.metrics_jsonl and self.rank == self.target_log_rank:
            self.wandb = M.JsonlSink(tc.metrics_jsonl)

        # fp32 master weights are created on the CPU and moved, so that init does not depend on the device
        self.ep_group = None
        if self.is_distributed and tc.dist_mode == "ddp_ep" and getattr(cfg.model, "n_experts", 0):
            self.ep_group = dist.group.WORLD
            # experts are split over the ranks: every rank draws the same stream and keeps its own experts
            with torch.random.fork_rng(devices=[]):
                torch.manual_seed(42)
                self.model = build_model(cfg.model, device="cpu", dtype=torch.float32, ep_group=self.ep_group)
        else:
            self.model = build_model(cfg.model, device="cpu", dtype=torch.float32)
        self.model.to(self.device)
        load_from = load_from or tc.load_from
        if load_from is not None:
            self.load_state(load_from, model_only=True)

        self.ddp: DDP | None = None
        if self.is_distributed and load_components == "all":
            if tc.dist_mode not in ("ddp", "ddp_ep"):
                raise ValueError(f"Unsupported dist_mode={tc.dist_mode!r}; expected 'ddp' or 'ddp_ep'.")
            comm = self._make_comm()
            local = (lambda n: ".experts." in n) if self.ep_group is not None else None
            self.ddp = DDP(self.model, bucket_size_mb=tc.bucket_size_mb, comm=comm, is_local=local)
        self.total_params = M.non_embedding_params(cfg.model)
        if self.wandb is not None and self.rank_zero_only:
            self.wandb.log(
                {
                    "total/params": self.total_params,
                    "total/tokens": tc.max_steps * cfg.data.batch_size * cfg.data.context_length,
                },
                step=self.iteration,
            )

        self.tokenizer = _load_tokenizer(str(cfg.data.tokenizer_path))
        self.id2byte_len: Tensor | None = None
        if self.tokenizer is not None:
            V = cfg.model.vocab_size
            lens = [len(self.tokenizer.decode([i], clean_up_tokenization_spaces=False).encode("utf-8")) for i in range(V)]
            self.id2byte_len = torch.tensor(lens, device=self.device, dtype=torch.float32)
            specials = [x for x in self.tokenizer.added_tokens_decoder if x < V]
            if specials:
                self.id2byte_len[torch.tensor(specials, device=self.device)] = 0

        self.use_engine = engine_supports(self.model) and os.environ.get("SEGPT_ENGINE", "1") == "1"
        self.ema: WeightEMA | None = None
        if load_components == "all":
            self._init_optimizers()
            if self.use_engine:
                self.engine = FusedEngine(self.model, self.act_dtype, moe_exchange=self._make_moe_exchange())
                self.engine.ensure_grads()
                self.engine.register_with(self.optimizers)
                if self.ddp is not None:
                    self.engine.grad_ready = self.ddp.grads_ready
            if load_from is not None:
                self.load_state(load_from, model_only=False, optimizers_only=True)
            if tc.ema_every > 0:
                self.ema = WeightEMA(self.model, decay=tc.ema_decay, every=tc.ema_every)
            logger.info(f"Model is created with hparams {cfg.model}")
            self.train_dataset = (
                MemoryMappedDataset(
                    cfg.data.train_path, cfg.data.context_length, self.device, cfg.data.seed + self.rank,
                    world_size=self.world_size, rank=self.rank,
                )
                if cfg.data.train_path
                else None
            )
            self.val_dataset = (
                MemoryMappedDataset(cfg.data.validation_path, cfg.data.context_length, self.device, cfg.data.seed + self.rank)
                if cfg.data.validation_path
                else None
            )
            self.save_dir = Path(tc.save_dir)
            if self.rank_zero_only:
                self.save_dir.mkdir(exist_ok=True, parents=True)
        else:
            self.model.eval()
            if self.use_engine and self.device.type == "cuda":
                self.engine = FusedEngine(self.model, self.act_dtype)

        if cfg.optim.scheduler == "wsd" and cfg.optim.wsd_phase == "decay":
            self.start_decay_step = int(cfg.optim.wsd_decay_step or self.iteration)
            self.decay_steps = tc.max_steps - self.start_decay_step
        else:
            self.decay_steps, self.start_decay_step = 0, 0
        if compile and not self.use_engine:
            self.model.compile()

        tp = str(cfg.data.tokenizer_path)
        self.train_loss_multiplier = 0.7985 if "superbpe" in tp else 1
        self.val_loss_multiplier = 0.8013 if "superbpe" in tp else 1
        self._watchdog = StepWatchdog(tc.watchdog_seconds) if tc.watchdog_seconds > 0 else None
        self._nan_guard = NonFiniteGuard(tc.nan_abort_after)
        self._micro_in_window = 0
        self.last_step_ms = 0.0
        self.status_probes: list[tuple[str, Any]] = []
        if self.device.type == "cuda":
            from sample_efficient_gpt_b200 import ops

            if ops.has_kernel("gemm_status"):
                self.status_probes.append(("a GEMM / attention kernel", lambda: ops.ext().gemm_status(self.device.index)))
        logger.info(
            f"Init [rank={self.rank}]: max_steps={tc.max_steps}, start_iter={self.iteration}, "
            f"val_every={tc.val_every}, save_every={tc.save_every}, world_size={self.world_size}, "
            f"grad_accum={tc.gradient_accumulation_steps}, batch_size={cfg.data.batch_size}, engine={self.use_engine}"
        )

    # ------------------------------------------------------------------ construction helpers
    def _make_comm(self):
        backend = self.cfg.trainer.comm_backend
        if backend in ("p2p", "nvls") or (backend == "auto" and self.device.type == "cuda"):
            try:
                from sample_efficient_gpt_b200.parallel.symm import SymmComm

                blocks = int(os.environ.get("SEGPT_COMM_BLOCKS", "32"))  # CTAs per bucket kernel (they share the GPU with the backward pass)
                return SymmComm.create(self.device, use_multimem=(backend == "nvls"), blocks=blocks)
            except Exception as e:
                if backend != "auto":
                    raise
                logger.warning(f"NVLink kernels unavailable ({type(e).__name__}: {e}); using torch.distributed collectives")
        return None

    def _make_moe_exchange(self):
        """Expert-parallel token exchange: NVLink push/pull kernels on symmetric memory when the communicator exists,
        ``all_to_all_single`` otherwise; None (local buffers) without expert parallelism."""
        if self.ep_group is None:
            return None
        from sample_efficient_gpt_b200.ops import moe as moe_ops

        comm = self.ddp.comm if self.ddp is not None else None
        if comm is not None and self.act_dtype == torch.bfloat16:
            return moe_ops.PeerExchange(self.cfg.model.n_experts, comm)
        return moe_ops.TorchExchange(self.cfg.model.n_experts, self.ep_group)

    @property
    def rank_zero_only(self) -> bool:
        return not self.is_distributed or self.rank == self.target_log_rank

    @property
    def raw_model(self):
        return self.model

    def _init_optimizers(self):
        oc = self.cfg.optim
        if oc.use_lion:
            raise NotImplementedError("use_lion: the reference has no Lion implementation either")
        named = list(self.model.named_parameters())
        kw = dict(lr=float(oc.lr), betas=tuple(oc.betas), weight_decay=oc.wd)
        if not oc.use_muon:
            self.optimizer = AdamW([p for _, p in named], **kw)
            self.optimizers = [self.optimizer]
            return
        adam_names = ("embedding", "lm_head", ".router.")
        one_d = [p for n, p in named if p.ndim < 2 or any(k in n for k in adam_names)]
        two_d = [p for n, p in named if p.ndim >= 2 and not any(k in n for k in adam_names)]
        local_2d = []
        if self.ep_group is not None:  # this rank's experts: never sharded, every rank steps its own
            local_2d = [p for n, p in named if ".experts." in n]
            two_d = [p for n, p in named if p.ndim >= 2 and not any(k in n for k in adam_names) and ".experts." not in n]
        for n, p in named:  # set as in the reference; only the Muon family reads lr_mul, whose params all get 1.0
            p.lr_mul = self.cfg.model.d_model**0.5 if "embedding" in n else (0.5 if "lm_head" in n else 1.0)
        self.optimizer1 = AdamW(one_d, **kw)
        muon_lr = float(oc.lr if oc.muon_lr is None else oc.muon_lr)
        muon_wd = oc.wd if oc.muon_wd is None else oc.muon_wd
        cls = (NorMuonCWD if oc.normuon_cautious_wd else NorMuon) if oc.muon_enable_normuon else Muon
        self.optimizer2 = cls(two_d, lr=muon_lr, momentum=oc.betas[0], weight_decay=muon_wd, shard=oc.shard_muon)
        if self.ddp is not None and self.ddp.comm is not None:
            self.optimizer2.comm = self.ddp.comm
        self.optimizers = [self.optimizer1, self.optimizer2]
        if local_2d:
            self.optimizer3 = cls(local_2d, lr=muon_lr, momentum=oc.betas[0], weight_decay=muon_wd, shard=False)
            self.optimizers.append(self.optimizer3)

    @property
    def tokens_processed(self) -> int:
        return self.iteration * self.cfg.data.batch_size * self.cfg.data.context_length

    # ------------------------------------------------------------------ state
    def load_state(self, path, model_only=True, optimizers_only=False):
        logger.info(f"Loading {model_only=} state from {str(path)}")
        if optimizers_only:
            if self.ep_group is not None and len(self.optimizers) == 3:
                return self._load_optimizers_expert_parallel(path)
            return load_optimizer(path, self.cfg, self.model, self.optimizers)
        self.iteration, self.run_id = load_model(path, self.cfg, self.model)
        if self.engine is not None:
            self.engine.refresh_shadows()
        logger.info(f"Restored {self.iteration} iteration")
        return self.iteration

    def _load_optimizers_expert_parallel(self, path):
        """Files hold the state of a run with all experts in one process (two optimizers); this rank takes the state of the
        replicated matrices and of its own experts out of it."""
        from sample_efficient_gpt_b200.training.ep_checkpoint import split_muon_state

        ckpt = torch.load(path, map_location="cpu", weights_only=False)
        saved = ckpt.get("optimizer")
        if not saved or saved[0] is None or len(saved) < 2:
            logger.info("no optimizers detected in the checkpoint, skipping...")
            return
        shared_sd, local_sd = split_muon_state(saved[1], self.model, self.optimizers[1], self.optimizers[2], self.ep_group)
        for opt, sd in zip(self.optimizers, (saved[0], shared_sd, local_sd)):
            opt.load_state_dict(sd)
            for p_, st in opt.state.items():
                for k, v in list(st.items()):
                    if torch.is_tensor(v):
                        st[k] = v.to(p_.device)
            if hasattr(opt, "_batches"):
                opt.load_state_dict(opt.state_dict())  # rebind the stacked storage on the right device

    def check_kernel_status(self):
        """Raise ``CommTimeout`` if a bounded wait inside one of this package's kernels gave up since the last check (the kernel
        then returned early and what it produced is incomplete).  Reads the status words on the device, which synchronises;
        the training loop calls it where it synchronises anyway (logging steps) and before every checkpoint, so that no file
        is written after a failed step.  ``status_probes`` holds the readers (name, callable returning a code, 0 = fine)."""
        from sample_efficient_gpt_b200.parallel.symm import CommTimeout

        if self.ddp is not None and self.ddp.comm is not None:
            self.ddp.comm.check()
        for name, probe in self.status_probes:
            code = int(probe())
            if code != 0:
                raise CommTimeout(f"a bounded wait inside {name} gave up (status {code}) at iteration {self.iteration}")

    def save_state(self):
        """Collective when the Muon step is sharded (owner-resident momentum is gathered first) or experts are split over
        ranks (every rank's experts and their optimizer state are gathered into the single-process layout)."""
        self.check_kernel_status()
        for opt in self.optimizers or []:
            if hasattr(opt, "consolidate_state"):
                opt.consolidate_state()
        model_sd, opt_sds, ema_sd = None, None, None
        if self.ep_group is not None and len(self.optimizers or []) == 3:
            from sample_efficient_gpt_b200.training.ep_checkpoint import gather_experts, gather_full_state

            full = gather_full_state(self.model, self.optimizers, self.ep_group)
            if self.ema is not None:
                ema_sd = gather_experts(self.ema.state_dict(), self.model, self.ep_group)
            if full is not None:
                model_sd, opt_sds = full
        if not self.rank_zero_only:
            return
        logger.info(f"Saving training state at iter={self.iteration}")
        run_id = getattr(self.wandb, "id", None) if self.wandb is not None else self.run_id
        fpath = self.save_dir / f"{self.iteration}.pt"
        if model_sd is not None:
            save_checkpoint(fpath, self.cfg, model_sd, None, self.iteration, run_id, extra={"optimizer": opt_sds})
        else:
            save_checkpoint(fpath, self.cfg, self.model, self.optimizers, self.iteration, run_id)
        if self.ema is not None:
            save_checkpoint(self.save_dir / f"{self.iteration}_ema.pt", self.cfg, ema_sd if ema_sd is not None else self.ema.state_dict(),
                            None, self.iteration, run_id)

    def log(self, data, rank_zero=True):
        if (not rank_zero) or self.rank_zero_only:
            for k, v in data.items():
                if "log" not in k:
                    logger.info(f"{k}: {v}")
            if self.wandb is not None:
                self.wandb.log(data, step=self.iteration)

    # ------------------------------------------------------------------ inference
    def generate(self, prompt: str, eos_token_id: int, top_p=1.0, temperature=0.0, max_steps=256, eos_prob_multiplier=1.0):
        assert self.tokenizer is not None, "generate() needs a tokenizer"
        ids = torch.tensor(self.tokenizer.encode(prompt)).unsqueeze(0).to(self.device)
        ctx = torch.autocast(self.device.type, dtype=torch.bfloat16) if self.act_dtype == torch.bfloat16 else nullcontext()
        with ctx:
            out, eos_probs = self.model.generate(
                ids, eos_token_id, top_p=top_p, temperature=temperature, max_steps=max_steps, eos_prob_multiplier=eos_prob_multiplier
            )
        return self.tokenizer.decode(out[0].cpu().tolist()), eos_probs

    @torch.no_grad()
    def validate(self) -> dict:
        logger.info(mem("before validation"))
        self.model.eval()
        n = 0
        loss_sum = torch.zeros((), device=self.device)
        bpb_sum = torch.zeros((), device=self.device)
        for inputs, targets in self.val_dataset.get_iterator(self.cfg.data.val_batch_size):
            inputs, targets = inputs.to(self.device), targets.to(self.device)
            loss, _, bpb = self._eval_loss(inputs, targets)
            loss_sum += loss.float() * self.val_loss_multiplier
            if bpb is not None:
                bpb_sum += bpb.float()
            n += 1
        self.model.train()
        n = max(n, 1)
        val_loss = (loss_sum / n).item()
        return {"val_loss": val_loss, "val_loss_bpb": (bpb_sum / n).item(), "val_perplexity": math.exp(min(val_loss, 80.0))}

    def _eval_loss(self, inputs, targets):
        if self.engine is not None:
            out = self.engine.forward_loss(inputs, targets, self.id2byte_len)
            return out.loss, out.z_loss, out.loss_bpb
        ctx = torch.autocast(self.device.type, dtype=torch.bfloat16) if self.act_dtype == torch.bfloat16 else nullcontext()
        with ctx:
            logits, _ = self.model(inputs)
            return efficient_cross_entropy(logits, targets.long(), per_token_byte_lengths=self.id2byte_len)

    # ------------------------------------------------------------------ schedules
    def _get_lr(self, lr: float, lr_min: float) -> float:
        oc = self.cfg.optim
        if oc.scheduler == "cosine":
            return get_cosine_lr(self.iteration, lr, lr_min, oc.warmup_steps, oc.cosine_steps)
        if oc.scheduler == "wsd":
            return get_wsd_lr(
                self.iteration, lr, lr_min, oc.zero_lr_steps, oc.warmup_steps, self.decay_steps,
                self.start_decay_step, oc.wsd_need_warmup, oc.wsd_phase,
            )
        if oc.scheduler == "seesaw":
            it_lr = get_seesaw_lr(self.iteration, lr, oc.warmup_steps, oc.seesaw_steps)
            return it_lr
        raise ValueError("unrecognized optim scheduler")

    def _set_lr(self):
        oc = self.cfg.optim
        if oc.scheduler == "seesaw" and self.iteration in tuple(oc.seesaw_steps):
            self.cfg.trainer.gradient_accumulation_steps *= 2
            logger.info(f"Global batch size is changed to {self.cfg.data.batch_size * self.cfg.trainer.gradient_accumulation_steps}")
        lr = float(oc.lr)
        iter_lr = self._get_lr(lr, lr * oc.lr_min_coeff)
        for pg in self.optimizers[0].param_groups:
            pg["lr"] = iter_lr
        if oc.use_muon:
            mlr = float(oc.lr if oc.muon_lr is None else oc.muon_lr)
            iter_lr = self._get_lr(mlr, mlr * oc.lr_min_coeff)
            for opt in self.optimizers[1:]:  # the Muon family: shared matrices and, with expert parallelism, local experts
                for pg in opt.param_groups:
                    if self.iteration < 300:
                        pg["momentum"] = muon_momentum_warmup(self.iteration, oc.betas[0])
                    pg["lr"] = iter_lr
        return iter_lr, oc.muon_wd

    # ------------------------------------------------------------------ the step
    def _loss_coef(self) -> float:
        ga = max(1, int(self.cfg.trainer.gradient_accumulation_steps))
        coef = 1.0 / ga
        if self.is_distributed and self.train_dataset is not None and self.train_dataset.local_batch_size:
            coef *= self.train_dataset.local_batch_size / self.cfg.data.batch_size
        elif self.is_distributed:
            coef /= self.world_size
        return coef

    def _expert_parallel_grad_norm(self, params, max_norm: float | None, ga: int) -> Tensor:
        """Global gradient norm when experts are split over ranks: the replicated parameters' (already reduced) gradients
        count once, every rank's own experts are added through one scalar all-reduce, so that all ranks see the same norm
        and - with clipping on - scale by the same factor (replicated weights then stay identical)."""
        named = list(self.model.named_parameters())
        expert_grads = [p.grad for n, p in named if p.grad is not None and ".experts." in n]
        shared_grads = [p.grad for n, p in named if p.grad is not None and ".experts." not in n]
        sq_local = torch.stack([n.float() ** 2 for n in torch._foreach_norm(expert_grads)]).sum() if expert_grads else torch.zeros((), device=self.device)
        dist.all_reduce(sq_local, group=self.ep_group)
        sq_shared = None
        if self.ddp is not None and self.ddp.comm is not None and ga == 1:
            in_buckets = [p.grad for n, p in named if p.grad is not None and ".experts." not in n and p not in self.ddp.param_bucket]
            sq_shared = self.ddp.reduced_grad_norm(in_buckets)
            sq_shared = None if sq_shared is None else sq_shared.float() ** 2
        if sq_shared is None:
            sq_shared = torch.stack([n.float() ** 2 for n in torch._foreach_norm(shared_grads)]).sum()
        norm = (sq_shared + sq_local).sqrt()
        if max_norm is not None:
            factor = (max_norm / (norm + 1e-8)).clamp(max=1.0)
            factor = torch.where(norm >= max_norm, factor, torch.ones_like(factor))
            torch._foreach_mul_([p.grad for p in params], factor)
        return norm

    def _zero_grads(self):
        if self.ddp is not None:
            self.ddp.zero_grad()
        elif self.engine is None:
            for p in self.model.parameters():
                if p.grad is not None:
                    p.grad.zero_()

    def train_step(self, inputs: Tensor, targets: Tensor) -> dict:
        self.model.train()
        iter_lr, iter_wd = self._set_lr()
        tc = self.cfg.trainer
        ga = max(1, int(tc.gradient_accumulation_steps))
        boundary = ((self.iteration + 1) % ga) == 0
        first_micro = self._micro_in_window == 0
        coef = self._loss_coef()
        sync_ctx = self.ddp.no_sync() if (self.ddp is not None and not boundary) else nullcontext()

        aux = None
        if self.engine is not None:
            with sync_ctx:
                out = self.engine.forward_backward(inputs, targets, coef, self.id2byte_len, first_micro_step=first_micro)
            loss, z_loss, loss_bpb, kurt = out.loss, out.z_loss, out.loss_bpb, out.kurtosis
            aux = out.aux_loss
        else:
            if first_micro:
                self._zero_grads()
            ctx = torch.autocast(self.device.type, dtype=torch.bfloat16) if self.act_dtype == torch.bfloat16 else nullcontext()
            with ctx:
                if tc.fused_linear_ce:
                    hidden, kurt = self.model.hidden_states(inputs)
                    loss, z_loss, loss_bpb = fused_linear_cross_entropy(
                        hidden, self.model.lm_head.linear.weight, targets.long(), self.id2byte_len, self.model.output_mult
                    )
                else:
                    logits, kurt = self.model(inputs)
                    loss, z_loss, loss_bpb = efficient_cross_entropy(logits, targets.long(), per_token_byte_lengths=self.id2byte_len)
                total = loss + tc.z_loss_weight * z_loss
                aux = self.model.aux_loss()
                if aux is not None:
                    total = total + aux
            with sync_ctx:
                (total * coef).backward()
        self._micro_in_window = 0 if boundary else self._micro_in_window + 1

        time_comm = 0.0
        if boundary:
            if self.ddp is not None:
                time_comm = self.ddp.finish_gradient_synchronization()
            params = [p for p in self.model.parameters() if p.grad is not None]
            if self.ep_group is not None:
                gnorm = self._expert_parallel_grad_norm(params, tc.max_grad_norm if tc.clip_fix else None, ga)
            elif tc.clip_fix:
                gnorm = clip_grad_norm_(params, tc.max_grad_norm)
            else:  # norm only: the reference's clipping never scales
                gnorm = None
                if self.ddp is not None and ga == 1:
                    local = [p.grad for n, p in self.model.named_parameters() if p.grad is not None and p not in self.ddp.param_bucket]
                    gnorm = self.ddp.reduced_grad_norm(local)  # partial sums from inside the reduction kernels
                if gnorm is None and self.engine is not None and self.ddp is None:
                    gnorm = self.engine.flat_grad_norm()  # one reduction over the engine's flat gradient buffer
                if gnorm is None:
                    gnorm = grad_norm([p.grad for p in params])
            update_ratios = [opt.step() for opt in self.optimizers]
            if self.ema is not None:
                self.ema.maybe_update()
        else:
            gnorm = torch.tensor(0.0)
            update_ratios = [torch.tensor(0.0) for _ in self.optimizers]

        need_log = self.rank_zero_only and (self.iteration % tc.log_every == 0)
        pnorms = {}
        if need_log:
            named = [(k, p) for k, p in self.model.named_parameters() if "attn" in k or "ffn" in k]
            norms = torch._foreach_norm([p.detach() for _, p in named])
            pnorms = {k: n for (k, _), n in zip(named, norms)}
        log = {
            "train_loss": loss.detach() * self.train_loss_multiplier,
            "train_loss_bpb": loss_bpb,
            "z_loss": z_loss.detach() * self.train_loss_multiplier,
            "grad_norm": gnorm,
            "learning_rate": iter_lr,
            "avg_kurtosis": kurt,
            "parameter_norms": pnorms,
            "time_comm": time_comm,
            f"rank_{self.rank}_fwd_bwd": 0,
        }
        if iter_wd is not None:
            log["wd"] = iter_wd
        if aux is not None:
            log["moe_aux_loss"] = aux.detach()
        for i, r in enumerate(update_ratios):
            log[f"opt_{i}_update_ratio"] = r
        return log

    def postprocess_step_stats(self, stats: dict) -> dict:
        cfg = self.cfg
        tps = cfg.data.batch_size * cfg.data.context_length / max(stats["step_time"], 1e-9)
        out = {
            "avg_kurtosis": stats["avg_kurtosis"].float().cpu().tolist(),
            "parameter_norms": {k: v.item() for k, v in stats["parameter_norms"].items()},
            "mfu": M.mfu(cfg.model, cfg.data.context_length, tps, self.world_size, cfg.trainer.use_fp8),
            "tokens_per_s": tps,
        }
        for k, v in stats.items():
            if k not in out:
                out[k] = v.item() if torch.is_tensor(v) else v
        return out

    def _check_finite(self, loss: Tensor):
        bad = (~torch.isfinite(loss.detach().float())).float().reshape(1)
        if self.is_distributed:
            bad = bad.to(self.device)
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        self._nan_guard.check(float("nan") if float(bad.item()) > 0 else 0.0)

    def fetch_batch(self) -> tuple[Tensor, Tensor]:
        inputs, targets = self.train_dataset.get_batch(self.cfg.data.batch_size)
        return inputs.to(self.device, non_blocking=True), targets.to(self.device, non_blocking=True)

    def train(self):
        logger.info("Starting training loop")
        tc = self.cfg.trainer
        cuda = self.device.type == "cuda"
        no_val = os.getenv("NO_VAL", "0") == "1"
        while self.iteration < tc.max_steps:
            if self.iteration % tc.save_every == 0:
                self.save_state()
            if self.rank_zero_only and self.val_dataset is not None and not no_val:
                if self.iteration > 0 and self.iteration % tc.val_every == 0:
                    self.log(self.validate())
            if cuda:
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
            t0 = time.monotonic()
            inputs, targets = self.fetch_batch()
            stats = self.train_step(inputs, targets)
            need_log = self.rank_zero_only and (self.iteration % tc.log_every == 0)
            if cuda:
                ev1.record()
            if self.iteration % tc.log_every == 0:
                # every rank takes the same decision at the same iteration: a failed bounded wait or a run of non-finite losses
                # stops all of them here instead of leaving the others to wait for a rank that has raised
                self.check_kernel_status()
                self._check_finite(stats["train_loss"])
            if need_log:
                if cuda:
                    ev1.synchronize()
                    stats["step_time"] = ev0.elapsed_time(ev1) / 1e3
                else:
                    stats["step_time"] = time.monotonic() - t0
                self.last_step_ms = stats["step_time"] * 1e3
                s = self.postprocess_step_stats(stats)
                logger.info(f"Train iteration {self.iteration}")
                self.log(
                    {
                        "train/loss": s["train_loss"],
                        "train/loss_bpb": s["train_loss_bpb"],
                        "train/z_loss": s["z_loss"],
                        "train/grad_norm": s["grad_norm"],
                        "train/learning_rate": s["learning_rate"],
                        **({"train/wd": s["wd"]} if "wd" in s else {}),
                        **{f"train/opt_{i}_update_ratio": s[f"opt_{i}_update_ratio"] for i in range(2) if f"opt_{i}_update_ratio" in s},
                        "train/step": self.iteration,
                        "train/step_time": s["step_time"],
                        "train/step_comm_time": s["time_comm"],
                        "train/tokens_processed": self.tokens_processed,
                        "train/tokens_per_s": s["tokens_per_s"],
                        "train/mfu": s["mfu"],
                        **{f"log/block{i}_kurtosis": v for i, v in enumerate(s["avg_kurtosis"])},
                        **{f"log/{k}_norm": v for k, v in s["parameter_norms"].items()},
                    }
                )
            if self._watchdog is not None:
                self._watchdog.beat()
            self.iteration += 1
        self.save_state()
        if self.rank_zero_only and self.val_dataset is not None and not no_val:
            self.log(self.validate())
        if self._watchdog is not None:
            self._watchdog.stop()
