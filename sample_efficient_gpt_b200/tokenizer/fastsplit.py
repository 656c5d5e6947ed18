"""``Splitter``: the native pre-tokeniser (same API as the reference's ``fastsplit`` extension), built on first use."""

from __future__ import annotations


def _load():
    try:
        from sample_efficient_gpt_b200.tokenizer import _segtok
    except ImportError:
        from sample_efficient_gpt_b200.tokenizer.build import build

        build()
        from sample_efficient_gpt_b200.tokenizer import _segtok
    return _segtok


_mod = _load()
Splitter = _mod.Splitter
