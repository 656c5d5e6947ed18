"""Export the pickled BPE vocabulary / merges as a HuggingFace fast tokenizer
(tokenizer/convert_tokenizer_to_hf.py:28-151 of the reference): GPT-2 byte <-> unicode table, ``tokenizers.BPE`` model,
``Split(regex)`` + ``ByteLevel`` pre-tokenizer, special tokens appended after the merges, and a spot check that
both tokenizers cut a few sentences identically."""

from __future__ import annotations

import pickle
import tempfile
from argparse import ArgumentParser
from pathlib import Path

from sample_efficient_gpt_b200.tokenizer.train_bpe import PAT_STR

SUPERBPE_BOUNDARY = r"""
(?<=\p{L})(?=['’](?i:(?:s|d|m|t|ll|ve|re)))
| (?<=['’](?i:(?:s|d|m|t|ll|ve|re)))
| (?<=-)(?=\|) | (?<=\|)(?=-)
| (?<=\d)(?=(?:\d{3})+(?!\d))
"""


def bytes_to_unicode() -> dict[int, str]:
    """The GPT-2 reversible byte -> printable unicode character table."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    chars, extra = keep[:], 0
    for b in range(256):
        if b not in keep:
            keep.append(b)
            chars.append(256 + extra)
            extra += 1
    return dict(zip(keep, map(chr, chars)))


def to_unicode(b: bytes, table: dict[int, str]) -> str:
    return "".join(table[x] for x in b)


def build_tokenizer(vocab: dict[int, bytes], merges: list[tuple[bytes, bytes]], specials: list[str], superbpe: bool = False,
                    add_prefix_space: bool = False):
    from tokenizers import AddedToken, Regex, Tokenizer
    from tokenizers.decoders import ByteLevel as ByteLevelDec
    from tokenizers.models import BPE
    from tokenizers.pre_tokenizers import ByteLevel as ByteLevelPre
    from tokenizers.pre_tokenizers import Sequence, Split
    from tokenizers.processors import ByteLevel as ByteLevelProc

    table = bytes_to_unicode()
    special_bytes = {s.encode() for s in specials}
    base = sorted((i, b) for i, b in vocab.items() if b not in special_bytes)
    str_vocab = {to_unicode(b, table): new for new, (_, b) in enumerate(base)}
    str_merges = [(to_unicode(l, table), to_unicode(r, table)) for l, r in merges]
    tok = Tokenizer(BPE(vocab=str_vocab, merges=str_merges, fuse_unk=False, byte_fallback=False))
    tok.pre_tokenizer = Sequence([
        Split(Regex(SUPERBPE_BOUNDARY if superbpe else PAT_STR), behavior="isolated", invert=False),
        ByteLevelPre(add_prefix_space=add_prefix_space, use_regex=False),
    ])
    tok.decoder = ByteLevelDec()
    tok.post_processor = ByteLevelProc(trim_offsets=False)
    tok.add_special_tokens([AddedToken(s, special=True, normalized=False) for s in specials])
    return tok


def main():
    p = ArgumentParser()
    p.add_argument("--tokenizer-path", required=True, help="folder with vocab.pickle and merges.pickle")
    p.add_argument("--superbpe-transition-idx", default=-1, type=int)
    p.add_argument("--save-path", required=True)
    a = p.parse_args()
    from transformers import PreTrainedTokenizerFast

    from sample_efficient_gpt_b200.tokenizer.tokenizer import Tokenizer as OwnTokenizer

    src = Path(a.tokenizer_path)
    vocab = pickle.loads((src / "vocab.pickle").read_bytes())
    merges = pickle.loads((src / "merges.pickle").read_bytes())
    superbpe = a.superbpe_transition_idx != -1
    specials = ["<|endoftext|>"] + [f"<|reserved_{i}|>" for i in range(20)]
    tok = build_tokenizer(vocab, merges, specials, superbpe=superbpe)
    own = OwnTokenizer(vocab, merges, ["<|endoftext|>"], a.superbpe_transition_idx if superbpe else None)
    with tempfile.NamedTemporaryFile(suffix=".json") as f:
        tok.save(f.name)
        hf = PreTrainedTokenizerFast(tokenizer_file=f.name)
    for text in ["Big cat sat on a mat", "I earn 1234567 dollars", "class NaturalHistory(nn.Module)",
                 "def function_a(arg1: int, arg2: str) -> str:", "am i on a right track here? help plz"]:
        ours = [own.decode([x]) for x in own.encode(text)]
        theirs = [hf.decode([x]) for x in hf(text).input_ids]
        if ours != theirs:
            print(f"mismatch: {ours=} {theirs=}")
    hf.save_pretrained(a.save_path)


if __name__ == "__main__":
    main()
