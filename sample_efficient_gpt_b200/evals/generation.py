"""Batched KV-cache text generation on this package's own model - the serving path behind the chat evaluation and the
web chat server (the reference delegates this to vLLM in evals/chat_eval.py:289-310 and to ``transformers.generate`` in
evals/chat_web.py:89-110).

* ``StaticKVCache``: keys/values in buffers allocated once for ``max_len`` positions and written in place - a decode
  step appends one column instead of re-concatenating the whole cache.
* ``SamplingParams``: n, max_tokens, temperature, top_k, top_p, stop_token_ids (the subset of vLLM's the evaluations use).
* ``GraphDecoder``: the one-token decode step of a dense model as a CUDA graph over static buffers (token, position,
  per-layer K/V caches of ``max_len`` positions, a position mask): the ~12 small kernels per layer of a decode step are
  launch-bound, a graph replay issues them in one call.  The prompt is prefilled eagerly into the same buffers.
* ``EngineDecoder``: the same step on the training engine's fused kernels and bf16 weight shadows (default on a GPU).
* ``ChatEngine``: renders conversations (tokenizer chat template, else the ``<|user_start|>...`` special-token format,
  else a plain-text fallback), runs prompts of equal length as one batch (the model has no padding mask), samples on the
  device, and checks for "all rows finished" every few steps so the decode loop does not synchronise per token.
  ``stream`` yields tokens one by one for a single conversation.
"""

from __future__ import annotations

from contextlib import nullcontext
from dataclasses import dataclass, field
from pathlib import Path

import torch
from torch import Tensor

from sample_efficient_gpt_b200.models.attention import KVCache


class StaticKVCache(KVCache):
    def __init__(self, max_len: int):
        super().__init__()
        self.max_len = max_len
        self._k: Tensor | None = None
        self._v: Tensor | None = None
        self._n = 0

    @property
    def length(self) -> int:
        return self._n

    def append(self, k: Tensor, v: Tensor):
        if self._k is None:
            b, h, _, d = k.shape
            # zero-filled: positions beyond the current length are masked in attention, but 0 x NaN would still poison it
            self._k = k.new_zeros(b, h, self.max_len, d)
            self._v = v.new_zeros(b, h, self.max_len, d)
        s = k.size(2)
        if self._n + s > self.max_len:
            raise ValueError(f"KV cache overflow: {self._n}+{s} > {self.max_len}")
        self._k[:, :, self._n : self._n + s] = k
        self._v[:, :, self._n : self._n + s] = v
        self._n += s
        self.keys, self.values = self._k[:, :, : self._n], self._v[:, :, : self._n]
        return self.keys, self.values


class GraphDecoder:
    """Static-shape decode step ``(token [B,1], position) -> logits [B,V]`` captured in a CUDA graph.

    Same math as models/attention.py with every shape fixed: the new key/value are written at ``pos`` with ``index_copy_``,
    attention runs over all ``max_len`` cached positions under the mask ``arange(max_len) <= pos``.  Dense blocks only.
    """

    def __init__(self, model, batch: int, max_len: int, device, autocast):
        import torch.nn.functional as F

        self.model, self.B, self.max_len, self.device, self.autocast, self.F = model, batch, max_len, torch.device(device), autocast, F
        at = model.blocks[0].attn
        if any(b.is_moe for b in model.blocks) or at.gating not in (False, "per-head"):
            raise ValueError("graph decode supports dense blocks with per-head (or no) gating")
        self.caches = [StaticKVCache(max_len) for _ in range(model.n_layers)]
        self.token = torch.zeros(batch, 1, dtype=torch.long, device=self.device)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.device)
        self.arange = torch.arange(max_len, device=self.device)
        self.logits: Tensor | None = None
        self.graph: torch.cuda.CUDAGraph | None = None

    def reset(self):
        for c in self.caches:
            c._n = 0
            c.keys = c.values = None

    def _step(self) -> Tensor:
        """The caches hold *finished* keys and values (rotated + QK-normalised keys, mixed values): per position these
        transformations do not depend on later tokens, so they are applied once, when a position is written."""
        from sample_efficient_gpt_b200.models.rope import apply_rope

        F, model, pos = self.F, self.model, self.pos
        mask = (self.arange <= pos).view(1, 1, 1, self.max_len)
        x = model.embedding(self.token)
        v1 = None
        for blk, cache in zip(model.blocks, self.caches):
            at = blk.attn
            b, h, hkv, hd = self.B, at.n_heads, at.n_kv_heads, at.head_dim
            n1 = blk.ln1(x)
            q, k, v = at.qkv(n1).split((h * hd, hkv * hd, hkv * hd), dim=-1)
            q = q.view(b, 1, h, hd).transpose(1, 2)
            k = k.view(b, 1, hkv, hd).transpose(1, 2)
            v = v.view(b, 1, hkv, hd).transpose(1, 2)
            cos, sin = at.rope.cos.index_select(0, pos), at.rope.sin.index_select(0, pos)
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
            vm = at.mix_values(v, v if v1 is None else v1)
            if v1 is None:
                v1 = vm
            if at.qknorm:
                q, k = at.sdpa_qknorm.normalize(q, k)
            cache._k.index_copy_(2, pos, k.to(cache._k.dtype))
            cache._v.index_copy_(2, pos, vm.to(cache._v.dtype))
            o = F.scaled_dot_product_attention(q, cache._k.to(q.dtype), cache._v.to(q.dtype), attn_mask=mask, enable_gqa=True).transpose(1, 2)
            if at.gating:
                o = (2.0 * at.attn_gate(n1).sigmoid()).unsqueeze(-1) * o
            y = x + at.out(o.reshape(b, 1, h * hd))
            x = y + blk.ffn(blk.ln2(y))
        logits = model.lm_head(model.final_norm(x))[:, -1, :]
        return logits * model.output_mult if model.output_mult != 1.0 else logits

    @torch.inference_mode()
    def prefill(self, prompt: Tensor) -> Tensor:
        """Eager forward of the prompt [B,S] into the static caches (raw: rotated keys, un-mixed values, as the model's own
        KV cache keeps them), then one pass that finishes them in place; returns the last position's logits."""
        self.reset()
        with self.autocast:
            logits, _ = self.model(prompt, kv_cache=self.caches)
            S = prompt.size(1)
            v1 = None
            for blk, cache in zip(self.model.blocks, self.caches):
                at = blk.attn
                raw_v = cache._v[:, :, :S]
                vm = at.mix_values(raw_v, raw_v if v1 is None else v1)
                if v1 is None:
                    v1 = vm.clone()
                cache._v[:, :, :S] = vm.to(cache._v.dtype)
                if at.qknorm:
                    kk = cache._k[:, :, :S]
                    cache._k[:, :, :S] = at.sdpa_qknorm.normalize(kk, kk)[1].to(cache._k.dtype)
        self.pos.fill_(prompt.size(1))
        return logits[:, -1, :]

    @torch.inference_mode()
    def step(self, tokens: Tensor) -> Tensor:
        """Feed one token per row at the current position; returns logits [B,V] (a static buffer) and advances."""
        self.token.copy_(tokens.view(self.B, 1))
        if self.device.type != "cuda":  # no graphs on the CPU: the same static-shape step, eagerly
            with self.autocast:
                self.logits = self._step()
            self.pos.add_(1)
            return self.logits
        if self.graph is None:
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side), self.autocast:  # warm-up outside the capture (lazy initialisations, autotuning)
                for _ in range(2):
                    self._step()
            torch.cuda.current_stream(self.device).wait_stream(side)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph), self.autocast:
                self.logits = self._step()
        self.graph.replay()
        self.pos.add_(1)
        return self.logits


class EngineDecoder:
    """Decode step on the fused kernels of the training engine (bf16 weight shadows, fused qkv+gate projection, one
    kernel each for add+RMSNorm, RoPE/QK-norm/value-mix at the cache position, gate, SwiGLU) captured in a CUDA graph:
    about a dozen launches per block instead of the several dozen of the module path.  Caches hold finished keys and values
    token-major, ``[B, max_len, Hkv, hd]``; the prompt is prefilled with the engine's forward."""

    def __init__(self, model, batch: int, max_len: int, device, engine=None):
        import torch.nn.functional as F

        from sample_efficient_gpt_b200.training.engine import FusedEngine

        self.F, self.model, self.B, self.max_len, self.device = F, model, batch, max_len, torch.device(device)
        self.eng = engine if engine is not None else FusedEngine(model, torch.bfloat16)  # bf16 copies of the weights
        at = model.blocks[0].attn
        self.H, self.Hkv, self.hd = at.n_heads, at.n_kv_heads, at.head_dim
        mk = lambda: torch.zeros(batch, max_len, self.Hkv, self.hd, dtype=torch.bfloat16, device=self.device)  # noqa: E731
        self.kc, self.vc = [mk() for _ in model.blocks], [mk() for _ in model.blocks]
        self.token = torch.zeros(batch, dtype=torch.long, device=self.device)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.device)
        self.pos32 = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.arange = torch.arange(max_len, device=self.device)
        # host copies of the per-block norm scales: reading a device scalar is not allowed while a graph is captured
        self.scales = [float(b.ln1.position_scale) for b in model.blocks]
        self.final_scale = float(model.final_norm.position_scale)
        self.logits: Tensor | None = None
        self.graph: torch.cuda.CUDAGraph | None = None

    def _final(self, res, delta):
        from sample_efficient_gpt_b200 import ops

        fn = self.model.final_norm
        _, hf, _, _ = ops.add_rmsnorm_fwd(res, delta, fn.gain, self.final_scale, fn.eps, torch.bfloat16, False)
        logits = ops.matmul_nt(hf, self.eng._w(self.model.lm_head.linear.weight)).float()
        return logits * self.model.output_mult if self.model.output_mult != 1.0 else logits

    @torch.inference_mode()
    def prefill(self, prompt: Tensor) -> Tensor:
        eng, model = self.eng, self.model
        B, S = prompt.shape
        res = model.embedding.weight.detach()[prompt.reshape(-1)].float()
        delta, v1 = None, None
        for i in range(model.n_layers):
            res, delta, v, _, saved = eng._layer_fwd(i, res, delta, v1, B, S, want_kurt=False, train=False)
            if v1 is None:
                v1 = v
            self.kc[i][:, :S].copy_(saved[6].view(B, S, self.Hkv, self.hd))  # finished keys / values of the prompt
            self.vc[i][:, :S].copy_(saved[7].view(B, S, self.Hkv, self.hd))
        last = torch.arange(B, device=self.device) * S + (S - 1)
        self.pos.fill_(S)
        self.pos32.fill_(S)
        return self._final(res[last], delta[last])

    def _step(self) -> Tensor:
        from sample_efficient_gpt_b200 import ops

        eng, model, F = self.eng, self.model, self.F
        B, H, Hkv, hd, lp = self.B, self.H, self.Hkv, self.hd, torch.bfloat16
        mask = (self.arange <= self.pos).view(1, 1, 1, self.max_len)
        res = model.embedding.weight.detach()[self.token].float()
        delta, v1 = None, None
        for i, blk in enumerate(model.blocks):
            at = blk.attn
            scale = self.scales[i]
            x, n1, _, _ = ops.add_rmsnorm_fwd(res, delta, blk.ln1.gain, scale, blk.ln1.eps, lp, False)
            if i in eng.qkvz_w:
                n_qkv = at.qkv.linear.weight.size(0)
                qkvz = ops.matmul_nt(n1, eng.qkvz_w[i])
                qkv, z = qkvz[:, :n_qkv], qkvz[:, n_qkv : n_qkv + H].contiguous()
            else:
                qkv = ops.matmul_nt(n1, eng._w(at.qkv.linear.weight))
                z = ops.matmul_nt(n1, eng._w(at.attn_gate.linear.weight)) if at.gating else None
            qgain = at.sdpa_qknorm.gain if at.qknorm else eng._ones
            q, k, v = ops.qkv_post_fwd(qkv, v1, at.rope.cos, at.rope.sin, qgain, at.alpha1, at.alpha2, at.scale, B, 1, H, Hkv, hd, at.qknorm,
                                       pos=self.pos32)
            if v1 is None:
                v1 = v
            self.kc[i].index_copy_(1, self.pos, k)
            self.vc[i].index_copy_(1, self.pos, v)
            o = F.scaled_dot_product_attention(q.transpose(1, 2), self.kc[i].transpose(1, 2), self.vc[i].transpose(1, 2), attn_mask=mask,
                                               enable_gqa=True)
            o = o.transpose(1, 2).reshape(B, H, hd)
            g = ops.gate_fwd(o, z) if at.gating else o.reshape(B, H * hd)
            a = ops.matmul_nt(g, eng._w(at.out.linear.weight))
            y, n2, _, _ = ops.add_rmsnorm_fwd(x, a, blk.ln2.gain, scale, blk.ln2.eps, lp, False)
            _, f = ops.up_swiglu(n2, eng._w(blk.ffn.up.linear.weight))
            m = ops.matmul_nt(f, eng._w(blk.ffn.down.linear.weight))
            res, delta = y, m
        return self._final(res, delta)

    @torch.inference_mode()
    def step(self, tokens: Tensor) -> Tensor:
        self.token.copy_(tokens.view(self.B))
        if self.graph is None:
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._step()
            torch.cuda.current_stream(self.device).wait_stream(side)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.logits = self._step()
        self.graph.replay()
        self.pos.add_(1)
        self.pos32.add_(1)
        return self.logits


@dataclass
class SamplingParams:
    n: int = 1
    max_tokens: int = 512
    temperature: float = 0.0
    top_k: int | None = 50
    top_p: float = 1.0
    stop_token_ids: list[int] = field(default_factory=list)
    seed: int | None = None


def sample_next(logits: Tensor, p: SamplingParams, gen: torch.Generator | None = None) -> Tensor:
    """logits [B,V] -> token ids [B]."""
    if p.temperature <= 0:
        return logits.argmax(-1)
    logits = logits.float() / p.temperature
    if p.top_k and p.top_k < logits.size(-1):
        kth = logits.topk(p.top_k, dim=-1).values[:, -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    probs = logits.softmax(-1)
    if p.top_p < 1.0:
        sp, si = probs.sort(-1, descending=True)
        keep = sp.cumsum(-1) - sp < p.top_p  # always keeps the most likely token
        probs = torch.zeros_like(probs).scatter_(-1, si, sp * keep)
        probs = probs / probs.sum(-1, keepdim=True)
    return torch.multinomial(probs, 1, generator=gen).squeeze(-1)


SPECIAL_FORMAT = ("<|bos|>", "<|user_start|>", "<|user_end|>", "<|assistant_start|>", "<|assistant_end|>")


def _message_text(content) -> str:
    if isinstance(content, str):
        return content
    return "".join(part.get("text", "") for part in content)


class ChatEngine:
    def __init__(self, model, tokenizer, device="cpu", max_model_len: int = 2048, chat_template: str | None = None,
                 dtype: torch.dtype | None = None, sync_every: int = 16, cuda_graphs: bool | None = None, cast_weights: bool = False,
                 fused_decode: bool | None = None):
        self.model, self.tokenizer, self.device = model.to(device).eval(), tokenizer, torch.device(device)
        self.max_model_len, self.chat_template, self.sync_every = max_model_len, chat_template, sync_every
        self.autocast = (torch.autocast("cuda", dtype=dtype or torch.bfloat16) if self.device.type == "cuda" else nullcontext())
        if cast_weights and self.device.type == "cuda" and (dtype or torch.bfloat16) != torch.float32:
            # serving: keep the weights in the compute dtype instead of re-casting fp32 masters on every decode step
            for prm in self.model.parameters():  # matrices only: gains, scalars, rotary tables and norm scales stay fp32
                if prm.ndim >= 2:
                    prm.data = prm.data.to(dtype or torch.bfloat16)
        vocab = tokenizer.get_vocab() if hasattr(tokenizer, "get_vocab") else {}
        self._special = {t: vocab[t] for t in SPECIAL_FORMAT if t in vocab}
        dense = not any(b.is_moe for b in self.model.blocks) and self.model.blocks[0].attn.gating in (False, "per-head")
        self.cuda_graphs = (self.device.type == "cuda" and dense) if cuda_graphs is None else (cuda_graphs and self.device.type == "cuda")
        self._decoders: dict = {}  # batch size -> decoder (caches for max_model_len positions)
        # decode on the engine's fused kernels when they are built and apply (bf16, dense, per-head or no gate)
        from sample_efficient_gpt_b200 import ops as _ops

        can_fuse = (self.cuda_graphs and (dtype or torch.bfloat16) == torch.bfloat16 and _ops.ext() is not None
                    and self.model.blocks[0].attn.head_dim % 16 == 0)
        self.fused_decode = can_fuse if fused_decode is None else (fused_decode and can_fuse)

    # ---- prompt rendering -------------------------------------------------------------------------------------------
    def render(self, messages: list[dict]) -> list[int]:
        tok = self.tokenizer
        template = self.chat_template or getattr(tok, "chat_template", None)
        if template:
            out = tok.apply_chat_template(messages, chat_template=template, add_generation_prompt=True, tokenize=True)
            return list(out["input_ids"] if hasattr(out, "keys") else out)
        enc = lambda s: list(tok.encode(s, add_special_tokens=False))
        if len(self._special) == len(SPECIAL_FORMAT):
            sp = self._special
            ids = [sp["<|bos|>"]]
            for m in messages:
                role = "user" if m["role"] in ("user", "system") else "assistant"
                ids += [sp[f"<|{role}_start|>"]] + enc(_message_text(m["content"])) + [sp[f"<|{role}_end|>"]]
            return ids + [sp["<|assistant_start|>"]]
        text = "".join(f"{m['role'].capitalize()}: {_message_text(m['content'])}\n" for m in messages) + "Assistant:"
        return enc(text)

    def default_stop_ids(self) -> list[int]:
        vocab = self.tokenizer.get_vocab() if hasattr(self.tokenizer, "get_vocab") else {}
        ids = [vocab[t] for t in ("<|endoftext|>", "<|assistant_end|>") if t in vocab]
        eos = getattr(self.tokenizer, "eos_token_id", None)
        return ids + ([eos] if eos is not None and eos not in ids else [])

    # ---- decoding ---------------------------------------------------------------------------------------------------
    @torch.inference_mode()
    def _decode_batch(self, prompt: Tensor, p: SamplingParams, gen=None, on_token=None) -> list[list[int]]:
        """prompt [B,S] (same length for every row) -> new token ids per row (stop token excluded)."""
        B, S = prompt.shape
        budget = min(p.max_tokens, self.max_model_len - S)
        if budget <= 0:
            return [[] for _ in range(B)]
        stop = torch.tensor(sorted(set(p.stop_token_ids)), device=self.device, dtype=torch.long)
        out = torch.zeros(B, budget, dtype=torch.long, device=self.device)
        done = torch.zeros(B, dtype=torch.bool, device=self.device)
        step_in, steps = prompt, 0
        decoder = None
        if self.cuda_graphs:
            decoder = self._decoders.get(B)
            if decoder is None:
                if self.fused_decode:
                    shared = next((d.eng for d in self._decoders.values() if isinstance(d, EngineDecoder)), None)
                    decoder = self._decoders[B] = EngineDecoder(self.model, B, self.max_model_len, self.device, shared)
                else:
                    decoder = self._decoders[B] = GraphDecoder(self.model, B, self.max_model_len, self.device, self.autocast)
        else:
            caches = [StaticKVCache(S + budget) for _ in range(self.model.n_layers)]
        with self.autocast:
            for t in range(budget):
                if decoder is not None:
                    last = decoder.prefill(prompt) if t == 0 else decoder.step(step_in)
                else:
                    last = self.model(step_in, kv_cache=caches)[0][:, -1, :]
                nxt = sample_next(last, p, gen)
                if stop.numel():
                    done = done | torch.isin(nxt, stop)
                out[:, t] = torch.where(done, torch.full_like(nxt, -1), nxt)
                step_in, steps = nxt[:, None], t + 1
                if on_token is not None:
                    if bool(done[0]):
                        break
                    on_token(int(nxt[0]))
                elif (t + 1) % self.sync_every == 0 and bool(done.all()):
                    break
        rows = out[:, :steps].cpu().tolist()
        return [row[: row.index(-1)] if -1 in row else row for row in rows]

    def generate_ids(self, prompts: list[list[int]], p: SamplingParams) -> list[list[list[int]]]:
        """For each prompt, ``p.n`` continuations (token ids)."""
        gen = None
        if p.seed is not None:
            gen = torch.Generator(device=self.device).manual_seed(p.seed)
        results: list[list[list[int]] | None] = [None] * len(prompts)
        by_len: dict[int, list[int]] = {}
        for i, ids in enumerate(prompts):
            ids = ids[-(self.max_model_len - 1):]
            prompts[i] = ids
            by_len.setdefault(len(ids), []).append(i)
        for _, members in sorted(by_len.items()):
            batch = torch.tensor([prompts[i] for i in members for _ in range(p.n)], dtype=torch.long, device=self.device)
            rows = self._decode_batch(batch, p, gen)
            for j, i in enumerate(members):
                results[i] = rows[j * p.n : (j + 1) * p.n]
        return results  # type: ignore[return-value]

    def chat(self, conversations: list[list[dict]], p: SamplingParams) -> list[list[str]]:
        ids = self.generate_ids([self.render(c) for c in conversations], p)
        return [[self.tokenizer.decode(r, skip_special_tokens=True) for r in rows] for rows in ids]

    def stream(self, messages: list[dict], p: SamplingParams):
        """Generator of text pieces for one conversation (decodes the growing id list so multi-byte characters that span
        tokens come out whole)."""
        import queue
        import threading

        q: queue.Queue = queue.Queue()
        prompt = torch.tensor([self.render(messages)[-(self.max_model_len - 1):]], dtype=torch.long, device=self.device)

        def run():
            try:
                self._decode_batch(prompt, p, None, on_token=q.put)
            finally:
                q.put(None)

        threading.Thread(target=run, daemon=True).start()
        ids: list[int] = []
        shown = ""
        while (tok := q.get()) is not None:
            ids.append(tok)
            text = self.tokenizer.decode(ids, skip_special_tokens=True)
            if text.endswith("�"):
                continue
            if len(text) > len(shown):
                yield text[len(shown):]
                shown = text


def load_chat_template(tokenizer_dir) -> str | None:
    """The tokenizer's own template, else a ``chat_template.jinja`` beside it (evals/chat_eval.py:25-34 of the reference)."""
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(str(tokenizer_dir), local_files_only=True, trust_remote_code=False)
    if getattr(tok, "chat_template", None):
        return tok.chat_template
    f = Path(tokenizer_dir) / "chat_template.jinja"
    return f.read_text() if f.is_file() else None


def load_engine(checkpoint: str, device="cuda", dtype: str = "bfloat16", max_model_len: int = 2048) -> ChatEngine:
    """``checkpoint`` is a converted HF directory (config.json + weights + tokenizer) or a native ``.pt`` file."""
    path = Path(checkpoint)
    if path.is_dir():
        from transformers import AutoTokenizer

        from sample_efficient_gpt_b200.scripts.hf.run_imu1_hf import load_native_from_hf

        model, _ = load_native_from_hf(path)
        tokenizer = AutoTokenizer.from_pretrained(str(path), local_files_only=True, trust_remote_code=False)
        template = load_chat_template(path)
    else:
        from sample_efficient_gpt_b200.training.trainer import Trainer

        tr = Trainer(load_from=str(path), load_components="infer", **{"trainer.device": str(device)})
        model, tokenizer, template = tr.model, tr.tokenizer, None
    torch_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, "auto": None}[dtype]
    return ChatEngine(model, tokenizer, device, max_model_len, template, torch_dtype, cast_weights=True)
