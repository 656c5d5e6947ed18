"""Batched KV-cache text generation on this package's own model - the serving path behind the chat evaluation and the
web chat server (the reference delegates this to vLLM in evals/chat_eval.py:289-310 and to ``transformers.generate`` in
evals/chat_web.py:89-110).

* ``StaticKVCache``: keys/values in buffers allocated once for ``max_len`` positions and written in place - a decode
  step appends one column instead of re-concatenating the whole cache.
* ``SamplingParams``: n, max_tokens, temperature, top_k, top_p, stop_token_ids (the subset of vLLM's the evaluations use).
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
            self._k = k.new_empty(b, h, self.max_len, d)
            self._v = v.new_empty(b, h, self.max_len, d)
        s = k.size(2)
        if self._n + s > self.max_len:
            raise ValueError(f"KV cache overflow: {self._n}+{s} > {self.max_len}")
        self._k[:, :, self._n : self._n + s] = k
        self._v[:, :, self._n : self._n + s] = v
        self._n += s
        self.keys, self.values = self._k[:, :, : self._n], self._v[:, :, : self._n]
        return self.keys, self.values


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
                 dtype: torch.dtype | None = None, sync_every: int = 16):
        self.model, self.tokenizer, self.device = model.to(device).eval(), tokenizer, torch.device(device)
        self.max_model_len, self.chat_template, self.sync_every = max_model_len, chat_template, sync_every
        self.autocast = (torch.autocast("cuda", dtype=dtype or torch.bfloat16) if self.device.type == "cuda" else nullcontext())
        vocab = tokenizer.get_vocab() if hasattr(tokenizer, "get_vocab") else {}
        self._special = {t: vocab[t] for t in SPECIAL_FORMAT if t in vocab}

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
        caches = [StaticKVCache(S + budget) for _ in range(self.model.n_layers)]
        stop = torch.tensor(sorted(set(p.stop_token_ids)), device=self.device, dtype=torch.long)
        out = torch.zeros(B, budget, dtype=torch.long, device=self.device)
        done = torch.zeros(B, dtype=torch.bool, device=self.device)
        step_in, steps = prompt, 0
        with self.autocast:
            for t in range(budget):
                logits, _ = self.model(step_in, kv_cache=caches)
                nxt = sample_next(logits[:, -1, :], p, gen)
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
    return ChatEngine(model, tokenizer, device, max_model_len, template, torch_dtype)
