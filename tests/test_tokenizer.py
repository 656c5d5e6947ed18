import pickle
import random

import numpy as np
import pytest
import regex

from sample_efficient_gpt_b200.tokenizer.cppbpe import Tokenizer as NativeBPE
from sample_efficient_gpt_b200.tokenizer.fastsplit import Splitter
from sample_efficient_gpt_b200.tokenizer.pretokenization import find_chunk_boundaries, pre_tokenize
from sample_efficient_gpt_b200.tokenizer.tokenizer import Tokenizer
from sample_efficient_gpt_b200.tokenizer.train_bpe import BPE, PAT

CORPUS = (
    "The quick brown fox jumps over the lazy dog. It's 12345 o'clock; they'll see!\n\n"
    "def f(x):\n    return x + 1  # héllo wörld 漢字 ٣٤\r\n<|endoftext|>"
    "Lower lowest newer newest wider widest low low low new new.\t tab\n \n  end  "
)


def oracle_pretokens(text, special="<|endoftext|>"):
    out = []
    for seg in text.split(special):
        out += PAT.findall(seg)
    return out


def test_native_scanner_matches_the_regex_on_random_text():
    sp = Splitter("<|endoftext|>")
    rnd = random.Random(0)
    alphabet = list("abcXYZ 019\t\n\r'.,!?-_()[]é漢字ßſ٣२  '") + ["'s", "'LL", "'Re", "  ", "\n\n", " \n ", "<|endoftext|>"]
    for _ in range(1500):
        text = "".join(rnd.choice(alphabet) for _ in range(rnd.randint(0, 40)))
        assert sp.pretokens(text) == oracle_pretokens(text), repr(text)
    assert sp.pretokens(CORPUS) == oracle_pretokens(CORPUS)


def test_split_counts_bytes_str_and_file_ranges(tmp_path):
    sp = Splitter("<|endoftext|>")
    want = {}
    for t in oracle_pretokens(CORPUS):
        want[t] = want.get(t, 0) + 1
    assert sp.split(CORPUS) == want and sp.split(CORPUS.encode()) == want
    raw = b"abc \xff\xfe def \xe2\x82"
    assert sp.split(raw) == sp.split(raw.decode("utf-8", "replace"))
    with pytest.raises(TypeError):
        sp.split(3)
    f = tmp_path / "c.txt"
    f.write_bytes((CORPUS * 50).encode())
    n = f.stat().st_size
    whole = sp.seek_and_split(str(f), 0, n)
    with f.open("rb") as fh:
        bounds = find_chunk_boundaries(fh, 7, b"<|endoftext|>")
    assert bounds[0] == 0 and bounds[-1] == n and bounds == sorted(set(bounds))
    for nproc in (1, 3):
        assert pre_tokenize(sp, str(f), num_processes=nproc) == whole
    with pytest.raises(ValueError):
        sp.seek_and_split(str(f), 5, 1)


def test_native_bpe_equals_python_trainer(tmp_path):
    text = CORPUS * 20 + " ".join(f"w{i % 17}x{i % 5}" for i in range(400))
    counts = Splitter("<|endoftext|>").split(text)
    specials = ["<|endoftext|>", "<|reserved_0|>"]
    a = BPE(specials, vocab_size=340, save_dir=tmp_path / "native")
    b = BPE(specials, vocab_size=340, save_dir=tmp_path / "python")
    va, ma = a.train_from_counts(counts, use_native=True)
    vb, mb = b.train_from_counts(counts, use_native=False)
    assert ma == mb and va == vb and len(ma) == 340 - 256 - 2
    assert va[256] == b"<|endoftext|>" and va[258] == ma[0][0] + ma[0][1]
    assert pickle.loads((tmp_path / "native" / "vocab.pickle").read_bytes()) == va
    nt = NativeBPE()
    nt.train_from_pretokens([(k.encode(), v) for k, v in counts.items()], 300)
    assert [tuple(m) for m in nt.export_merges_bytes()] == ma[:44]
    assert dict(nt.get_mergeable_ranks())[b"a"] == 97 and len(nt.export_vocab_bytes()) == 300
    ids = nt.encode("the lowest fox")
    assert b"".join(dict(nt.export_vocab_bytes())[i] for i in ids) == b"the lowest fox"


def test_tokenizer_roundtrip_specials_superbpe_and_tools(tmp_path):
    text = CORPUS * 20
    bpe = BPE(["<|endoftext|>"], vocab_size=420, save_dir=tmp_path / "tok")
    bpe.train_from_counts(Splitter("<|endoftext|>").split(text))
    tok = Tokenizer.from_files(tmp_path / "tok" / "vocab.pickle", tmp_path / "tok" / "merges.pickle", ["<|endoftext|>"])
    ids = tok.encode(CORPUS)
    assert tok.decode(ids) == CORPUS and ids.count(256) == 1 and max(ids) < 420
    assert len(ids) < len(CORPUS.encode()) * 0.7
    # lowest-rank-first merging agrees with replaying the merges in order on every pre-token
    for pre in set(oracle_pretokens(CORPUS)):
        seq = [bytes([x]) for x in pre.encode()]
        for l, r in bpe.merges_tuples:
            i, out = 0, []
            while i < len(seq):
                if i + 1 < len(seq) and seq[i] == l and seq[i + 1] == r:
                    out.append(l + r); i += 2
                else:
                    out.append(seq[i]); i += 1
            seq = out
        assert [tok.vocab[i] for i in tok.encode(pre)] == seq, pre
    first_stage = len(bpe.merges_tuples)
    docs = [tok.encode(d) for d in (CORPUS * 3).split("<|endoftext|>")]
    bpe.resume_train(docs, vocab_size=440, superbpe=True)
    tok2 = Tokenizer(bpe.vocab, bpe.merges_tuples, ["<|endoftext|>"], superbpe_transition_idx=first_stage)
    ids2 = tok2.encode(CORPUS)
    assert tok2.decode(ids2) == CORPUS and len(ids2) < len(ids)
    f = tmp_path / "t.txt"
    f.write_text(CORPUS * 5)
    assert tok.decode(tok.encode_file(f, chunk_size=64)) == CORPUS * 5
    from sample_efficient_gpt_b200.tokenizer.split_val import split_validation

    d = tmp_path / "data"; d.mkdir()
    np.save(d / "a.npy", np.arange(100, dtype=np.uint16))
    np.save(d / "offsets_a.npy", np.array([0, 10, 35, 60, 100]))
    cut = split_validation(d, tmp_path / "val", "val.npy", val_tokens=40)
    assert cut == 35 and np.load(tmp_path / "val" / "val.npy").tolist() == list(range(35))
    assert np.load(d / "a.npy")[0] == 35 and np.load(d / "offsets_a.npy").tolist() == [0, 25, 65]


def test_hf_export_matches_own_tokenizer(tmp_path):
    pytest.importorskip("tokenizers")
    from sample_efficient_gpt_b200.tokenizer.convert_tokenizer_to_hf import build_tokenizer

    bpe = BPE(["<|endoftext|>"], vocab_size=400, save_dir=tmp_path / "tok")
    bpe.train_from_counts(Splitter("<|endoftext|>").split(CORPUS * 20))
    own = Tokenizer(bpe.vocab, bpe.merges_tuples, ["<|endoftext|>"])
    hf = build_tokenizer(bpe.vocab, bpe.merges_tuples, ["<|endoftext|>"])
    for text in ["The quick brown fox", "It's 12345 o'clock", "def f(x):\n    return x + 1"]:
        assert [own.decode([i]) for i in own.encode(text)] == [hf.decode([i]) for i in hf.encode(text).ids]


def _word_tokenizer():
    from tokenizers import Tokenizer as HFTok, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    words = ["<|endoftext|>", "<unk>", "<|bos|>", "a", "b", "c", "d"]
    tok = HFTok(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    return PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", eos_token="<|endoftext|>",
                                   additional_special_tokens=["<|bos|>"])


def test_dataset_tokeniser_parquet_jsonl_txt(tmp_path, monkeypatch):
    import gzip
    import json

    import numpy as np
    import pyarrow as pa
    import pyarrow.parquet as pq

    from sample_efficient_gpt_b200.tokenizer import tokenize_with_fast_tokenizer as T

    monkeypatch.setenv("STAGE", "1")
    proc = T.TokenizerProcessor(_word_tokenizer())
    src = tmp_path / "finemath_x"
    src.mkdir()
    rows = [{"text": "a b", "score": 4.0}, {"text": "c", "score": 1.0}, {"text": "d d d", "score": 3.8}]
    pq.write_table(pa.Table.from_pylist(rows), src / "part.0.parquet")
    out = tmp_path / "tok"
    n = proc.encode_hf(src, out)
    tokens, offsets = np.load(out / "part0.npy"), np.load(out / "offsets_part.0.npy")
    assert tokens.dtype == np.uint16 and offsets.dtype == np.int64 and n == 7
    assert tokens.tolist() == [3, 4, 0, 6, 6, 6, 0] and offsets.tolist() == [0, 3, 7]  # score 1.0 <= 3.7 dropped, EOT appended
    assert proc.encode_hf(src, out, limit=100) == 7  # finished shard is skipped but counted
    assert T.threshold("finemath", 2) == 4.1 and T.threshold("pleias_synth", 3) == 2.1

    js = tmp_path / "plain"
    js.mkdir()
    with gzip.open(js / "x.jsonl.gz", "wt") as f:
        for t in ("a", "b c"):
            f.write(json.dumps({"text": t}) + "\n")
    proc.encode_hf(js, out)
    assert np.load(out / "0.npy").tolist() == [3, 0, 4, 5, 0] and np.load(out / "offsets_0.npy").tolist() == [0, 2, 5]

    monkeypatch.setenv("STAGE", "3")
    assert proc.preprocess_text("q\n<think>r") == "<|bos|><|user_start|>q<|user_end|><|assistant_start|>\n<think>r<|assistant_end|><|endoftext|>"
    assert proc.preprocess_text("x") == "<|bos|>x<|endoftext|>"
    assert not proc.keep_row({"text": "short"}, "anything") and proc.keep_row({"text": "x" * 4001}, "anything")
    monkeypatch.setenv("STAGE", "1")

    txt = tmp_path / "txt"
    txt.mkdir()
    (txt / "c_train.txt").write_text("a b<|endoftext|>c d<|endoftext|>")
    (txt / "c_val.txt").write_text("a a a a<|endoftext|>")
    proc.encode_hf_txt(txt, out)
    assert np.load(out / "c_train.npy").tolist() == [3, 4, 0, 5, 6, 0]
    ratios = proc.compression_ratios(txt)
    assert ratios["c_val.txt"] == pytest.approx(7 / 5)


def test_tokenizer_bench_runs_and_native_trainer_matches_python(tmp_path):
    """The CPU benchmark of the native tools on a 1 MB synthetic corpus: both BPE trainers must learn the same merges."""
    import json
    import subprocess
    import sys

    r = subprocess.run([sys.executable, "-m", "sample_efficient_gpt_b200.tokenizer.bench_tokenizer", "--mb", "1", "--vocab-size", "320",
                        "--threads", "2", "--python-mb", "1"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["bpe_same_merges"] is True and out["bpe_merges"] == 64 and out["distinct_pretokens"] > 1000
    assert out["encode_same_ids"] is True


def test_native_encoder_matches_the_python_statements(tmp_path):
    """tokenizer/csrc/segtok.cpp::Encoder against ``merge_by_rank`` + cache in Python: one-stage and two-stage (superbpe)
    vocabularies, special tokens in the text, random unicode, and the batch API on several threads."""
    import random

    rnd = random.Random(3)
    alphabet = list("abcdefghij  \n.,'0123456789") + ["é", "ü", "あ", "語", "😀", "it's", " don't", "<|endoftext|>"]
    texts = ["".join(rnd.choice(alphabet) for _ in range(rnd.randint(1, 400))) for _ in range(60)] + [CORPUS, "", " ", "<|endoftext|>"]
    bpe = BPE(["<|endoftext|>"], vocab_size=420, save_dir=tmp_path / "tok")
    bpe.train_from_counts(Splitter("<|endoftext|>").split(CORPUS * 20 + "".join(texts)))
    first = len(bpe.merges_tuples)
    py1 = Tokenizer(bpe.vocab, bpe.merges_tuples, ["<|endoftext|>"], use_native=False)
    na1 = Tokenizer(bpe.vocab, bpe.merges_tuples, ["<|endoftext|>"])
    assert na1._native is not None and py1._native is None
    docs = [py1.encode(d) for d in (CORPUS * 3 + "".join(texts)).split("<|endoftext|>")]
    bpe.resume_train(docs, vocab_size=470, superbpe=True)
    py2 = Tokenizer(bpe.vocab, bpe.merges_tuples, ["<|endoftext|>"], superbpe_transition_idx=first, use_native=False)
    na2 = Tokenizer(bpe.vocab, bpe.merges_tuples, ["<|endoftext|>"], superbpe_transition_idx=first)
    for t in texts:
        assert na1.encode(t) == py1.encode(t), t
        assert na2.encode(t) == py2.encode(t), t
        assert na2.decode(na2.encode(t)) == t
    assert na1.encode_batch(texts, threads=4) == [py1.encode(t) for t in texts]
    assert na2.encode_batch(texts, threads=3) == [py2.encode(t) for t in texts]
    assert py1.encode_batch(texts[:5]) == [py1.encode(t) for t in texts[:5]]
