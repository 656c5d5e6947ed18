"""``Tokenizer``: the native incremental BPE trainer (same API as the reference's ``rustbpe`` extension)."""

from sample_efficient_gpt_b200.tokenizer.fastsplit import _mod

Tokenizer = _mod.Tokenizer
