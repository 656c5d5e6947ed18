"""Evaluation stack on CPU: CORE prompt rendering and scoring, the execution guard, MBPP scoring, chat tasks, the
generation engine (static KV cache == plain forward) and the web API."""

import json
import os

import pytest
import torch

from sample_efficient_gpt_b200.config_schema import ModelConfig
from sample_efficient_gpt_b200.evals import core_eval
from sample_efficient_gpt_b200.evals.execution import execute_code
from sample_efficient_gpt_b200.evals.generation import ChatEngine, SamplingParams, sample_next
from sample_efficient_gpt_b200.models import build_model

WORDS = ["the", "cat", "dog", "sat", "ran", "on", "mat", "far", "Q", "A", "B", "C", "D", "is", "answer", "yes", "no", ":", "?"]


def make_tokenizer(chat_specials=False):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    specials = ["<|endoftext|>", "<unk>"]
    if chat_specials:
        specials += ["<|bos|>", "<|user_start|>", "<|user_end|>", "<|assistant_start|>", "<|assistant_end|>"]
    vocab = {w: i for i, w in enumerate(specials + WORDS)}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    return PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", eos_token="<|endoftext|>",
                                   additional_special_tokens=specials[2:])


def tiny_model(vocab=32, seed=0):
    torch.manual_seed(seed)
    cfg = ModelConfig(d_model=64, d_ff=128, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=vocab, attn_qknorm=True,
                      attn_val_residual=True, attn_gating="per-head", layernorm_scaling=True, weight_tying=False)
    return build_model(cfg).eval()


# ---- CORE ---------------------------------------------------------------------------------------------------------------
def test_render_prompts_golden():
    mc = dict(query="Q ?", choices=["yes", "no"], gold=0)
    shots = [dict(query="the cat ?", choices=["A", "B"], gold=1)]
    assert core_eval.render_prompts_mc(mc, " ") == ["Q ? yes", "Q ? no"]
    assert core_eval.render_prompts_mc(mc, " answer : ", shots) == ["the cat ? answer : B\n\nQ ? answer : yes", "the cat ? answer : B\n\nQ ? answer : no"]
    sc = dict(context_options=["the cat", "the dog"], continuation="sat", gold=1)
    assert core_eval.render_prompts_schema(sc, " ") == ["the cat sat", "the dog sat"]
    lm = dict(context="the cat sat on  ", continuation="the mat")
    assert core_eval.render_prompts_lm(lm, " ") == ["the cat sat on", "the cat sat on the mat"]
    two = core_eval.render_prompts_lm(lm, " ", [dict(context=" the dog ", continuation="ran")])
    assert two == ["the dog ran\n\nthe cat sat on", "the dog ran\n\nthe cat sat on the mat"]


def test_common_length_and_spans():
    assert core_eval.find_common_length([[1, 2, 3], [1, 2, 4]], "left") == 2
    assert core_eval.find_common_length([[9, 2, 3], [1, 2, 3]], "right") == 2
    assert core_eval.find_common_length([[1, 2], [1, 2]], "left") == 2
    toks, s, e = core_eval.answer_spans("multiple_choice", [[0, 5, 6, 7], [0, 5, 8]])
    assert (s, e) == ([2, 2], [4, 3])
    toks, s, e = core_eval.answer_spans("schema", [[0, 5, 9, 9], [0, 6, 7, 9, 9]])
    assert (s, e) == ([2, 3], [4, 5])
    toks, s, e = core_eval.answer_spans("language_modeling", [[0, 5], [0, 5, 6, 7]])
    assert toks == [[0, 5, 6, 7]] and (s, e) == ([2], [4])


class _Oracle(torch.nn.Module):
    """Predicts token (id + 1) % V with certainty: continuation 'follows' iff it counts upwards."""

    max_seq_len = 64

    def __init__(self, V):
        super().__init__()
        self.V = V

    def forward(self, ids):
        logits = torch.full((*ids.shape, self.V), -20.0)
        logits.scatter_(-1, ((ids + 1) % self.V)[..., None], 20.0)
        return logits, None


class _IdTokenizer:
    """'3 4 5' -> [3, 4, 5]; no BOS."""

    pad_token_id = 0
    bos_token_id = None
    eos_token_id = None

    def __call__(self, prompts, add_special_tokens=False):
        return {"input_ids": [[int(t) for t in p.split()] for p in prompts]}


def test_evaluate_example_all_types():
    model, tok = _Oracle(50), _IdTokenizer()
    mc = [dict(query="3 4", choices=["9 9", "5 6", "7"], gold=1), dict(query="1 2", choices=["3", "8"], gold=1)]
    meta = dict(task_type="multiple_choice", num_fewshot=0, continuation_delimiter=" ")
    assert core_eval.evaluate_example(0, model, tok, mc, "cpu", meta) is True
    assert core_eval.evaluate_example(1, model, tok, mc, "cpu", meta) is False
    sc = [dict(context_options=["7 7", "3 4"], continuation="5 6", gold=1)]
    assert core_eval.evaluate_example(0, model, tok, sc, "cpu", dict(meta, task_type="schema")) is True
    lm = [dict(context="10 11", continuation="12 13"), dict(context="10 11", continuation="12 14"), dict(context="1", continuation="2")]
    meta_lm = dict(meta, task_type="language_modeling")
    assert core_eval.evaluate_example(0, model, tok, lm, "cpu", meta_lm) is True
    assert core_eval.evaluate_example(1, model, tok, lm, "cpu", meta_lm) is False
    assert core_eval.evaluate_example(0, model, tok, lm, "cpu", dict(meta_lm, num_fewshot=2)) is True  # few-shot path
    assert core_eval.evaluate_task(model, tok, lm, "cpu", meta_lm) == pytest.approx(2 / 3)


def test_base_eval_bundle(tmp_path):
    from sample_efficient_gpt_b200.evals.base_eval import evaluate_model, write_csv

    bundle = tmp_path / "eval_bundle"
    (bundle / "eval_data").mkdir(parents=True)
    rows = [dict(context="10 11", continuation="12 13"), dict(context="5", continuation="7")]
    (bundle / "eval_data" / "count.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    mc = [dict(query="3 4", choices=["9", "5"], gold=1)] * 3
    (bundle / "eval_data" / "mc.jsonl").write_text("\n".join(json.dumps(r) for r in mc))
    (bundle / "core.yaml").write_text(
        "icl_tasks:\n"
        "- {label: count, dataset_uri: count.jsonl, num_fewshot: [0], icl_task_type: language_modeling}\n"
        "- {label: mc, dataset_uri: mc.jsonl, num_fewshot: [1], icl_task_type: multiple_choice, continuation_delimiter: ' '}\n")
    (bundle / "eval_meta_data.csv").write_text("Eval Task,Task Category,Random baseline\ncount,lm,0\nmc,mc,50\n")
    out = evaluate_model(tmp_path, _Oracle(50), _IdTokenizer(), "cpu")
    assert out["results"] == {"count": 0.5, "mc": 1.0}
    assert out["centered_results"]["mc"] == pytest.approx(1.0) and out["core_metric"] == pytest.approx(0.75)
    with pytest.raises(ValueError):
        evaluate_model(tmp_path, _Oracle(50), _IdTokenizer(), "cpu", task="nope")
    write_csv(tmp_path / "r" / "x.csv", out)
    assert "CORE" in (tmp_path / "r" / "x.csv").read_text()


# ---- execution guard + MBPP -------------------------------------------------------------------------------------------------
def test_execute_code_outcomes():
    ok = execute_code("print('hello world')")
    assert ok.success and ok.stdout == "hello world\n"
    assert execute_code("assert 1 == 2, 'nope'").error == "AssertionError: nope"
    t = execute_code("while True:\n    pass", timeout=0.5)
    assert not t.success and t.timeout
    m = execute_code("x = bytearray(1 << 30)", maximum_memory_bytes=128 << 20)
    assert not m.success and m.memory_exceeded
    blocked = execute_code("import os\nos.system('echo hi')")
    assert not blocked.success and "NoneType" in blocked.error
    assert not execute_code("import sys\nsys.exit(0)").success


def test_mbpp_lite_scoring(tmp_path):
    from sample_efficient_gpt_b200.evals import mbpp_eval, mbpp_lite

    assert len(mbpp_lite.DATA) == 10
    ev = mbpp_eval.SimpleMBPPEvaluator("lite", timeout=5.0)
    by_prompt = {v["prompt"]: v["canonical_solution"] for v in mbpp_lite.DATA.values()}
    ids = ["Mbpp/10001", "Mbpp_10002", "Mbpp/10007"]
    good = ev.evaluate_with_generate(lambda p: by_prompt[p], task_ids=ids)
    assert good["pass_at_k"] == {"base": {"pass@1": 1.0}, "plus": {"pass@1": 1.0}}
    bad = ev.evaluate_with_generate(lambda p: "    return 0\n", task_ids=ids[:2], plus=False)
    assert bad["pass_at_k"] == {"base": {"pass@1": 0.0}}
    assert mbpp_eval.estimate_pass_at_k([10, 10], [3, 0], 1) == pytest.approx(0.15)
    assert mbpp_eval.estimate_pass_at_k([5], [5], 3) == 1.0
    assert mbpp_eval.safe_compare([1.0, (2, 3)], [1.0 + 1e-9, (2, 3)], 1e-6) and not mbpp_eval.safe_compare([1], [1, 2], 0)
    samples = tmp_path / "s.jsonl"
    samples.write_text(json.dumps({"task_id": "Mbpp/10002", "completion": mbpp_lite.DATA["Mbpp/10002"]["canonical_solution"]}) + "\n"
                       + json.dumps({"task_id": "Mbpp/10002", "solution": "def gcd(a, b):\n    return 1\n"}) + "\n")
    out = mbpp_eval.main(["--samples", str(samples), "--k", "1,2"])
    assert out["pass_at_k"]["base"] == {"pass@1": 0.5, "pass@2": 1.0}
    assert (tmp_path / "s.eval_results.json").exists()


# ---- chat tasks -----------------------------------------------------------------------------------------------------------
def _mirror(root, repo, subset, split, rows):
    d = root / repo.replace("/", "__") / (subset or "")
    d.mkdir(parents=True, exist_ok=True)
    (d / f"{split}.jsonl").write_text("\n".join(json.dumps(r) for r in rows))


def test_tasks_from_local_mirror(tmp_path, monkeypatch):
    from sample_efficient_gpt_b200.evals.tasks.arc import ARC
    from sample_efficient_gpt_b200.evals.tasks.common import TaskMixture, TaskSequence, render_mc
    from sample_efficient_gpt_b200.evals.tasks.gsm8k import GSM8K, answer_text, extract_answer
    from sample_efficient_gpt_b200.evals.tasks.humaneval import HumanEval, extract_imports, extract_program
    from sample_efficient_gpt_b200.evals.tasks.mmlu import MMLU
    from sample_efficient_gpt_b200.evals.tasks.smoltalk import SmolTalk

    monkeypatch.setenv("SEGPT_DATASETS_DIR", str(tmp_path))
    arc_rows = [dict(question=f"q{i}", choices=dict(text=["x", "y", "z"], label=["A", "B", "C"]), answerKey="ABC"[i % 3]) for i in range(7)]
    _mirror(tmp_path, "allenai/ai2_arc", "ARC-Easy", "test", arc_rows)
    arc = ARC("ARC-Easy", "test")
    assert len(arc) == 7 and len(ARC("ARC-Easy", "test", start=1, stop=6, step=2)) == 3
    ex = arc[0]
    assert ex["messages"][0]["content"].startswith("Multiple Choice question: q") and "- x=A\n" in ex["messages"][0]["content"]
    assert arc.evaluate(ex, ex["messages"][-1]["content"]) and sorted(e["messages"][0]["content"] for e in arc) != [e["messages"][0]["content"] for e in arc]
    assert render_mc("Q", "AB", ["u", "v"]) == "Multiple Choice question: Q\n- u=A\n- v=B\n\nRespond only with the letter of the correct answer."

    _mirror(tmp_path, "cais/mmlu", "all", "test", [dict(question="q", choices=list("wxyz"), answer=2, subject="s")])
    m = MMLU("all", "test")[0]
    assert m["messages"][-1]["content"] == "C" and m["subject"] == "s"

    gsm = [dict(question=f"q{i}", answer=f"a <<1+{i}={1 + i}>>{1 + i} b\n#### {1 + i}") for i in range(6)]
    _mirror(tmp_path, "openai/gsm8k", "main", "test", gsm)
    _mirror(tmp_path, "openai/gsm8k", "main", "train", gsm)
    g = GSM8K("main", "test", few_shot=True, use_llama_system_prompt=True)
    conv = g[0]
    assert len(conv["messages"]) == 12 and conv["messages"][0]["content"].startswith("Given the following problem")
    gold = extract_answer(conv["messages"][-1]["content"])
    assert g.evaluate(conv, f"so #### {gold}") == 1 and g.evaluate(conv, "#### 999") == 0 and g.reward(conv, "none") == 0.0
    assert extract_answer("#### 1,234") == "1234"
    assert answer_text("a <<1+0=1>>1 b\n#### 1") == "a \n1+0\n1\n1 b\n#### 1"

    he = [dict(prompt="import math\n\ndef add(a, b):\n", canonical_solution="    return a + b\n", entry_point="add",
               test="def check(f):\n    assert f(1, 2) == 3\n")]
    _mirror(tmp_path, "openai/openai_humaneval", None, "test", he)
    h = HumanEval()
    c = h[0]
    assert h.evaluate(c, "```python\ndef add(a, b):\n    return a + b\n```") and not h.evaluate(c, "def add(a, b):\n    return a - b")
    assert extract_imports("# c\nimport os\nfrom x import y\nz = 1\nimport late") == "import os\nfrom x import y"
    assert extract_program("text\n```\ncode()\n```\nmore") == "code()"

    _mirror(tmp_path, "HuggingFaceTB/smol-smoltalk", None, "train", [dict(messages=[dict(role="user", content=str(i))]) for i in range(5)])
    st = SmolTalk("train")
    mix, seq = TaskMixture([st, arc]), TaskSequence([st, arc])
    assert len(mix) == 12 and len(seq) == 12 and seq[5] == arc[0]
    assert sorted(json.dumps(x, sort_keys=True) for x in mix) == sorted(json.dumps(x, sort_keys=True) for x in seq)


# ---- generation engine ------------------------------------------------------------------------------------------------------
def test_static_cache_matches_full_forward():
    model = tiny_model()
    engine = ChatEngine(model, make_tokenizer(), "cpu", max_model_len=48)
    prompt = [[3, 4, 5, 6], [7, 8, 9, 10]]
    out = engine.generate_ids([list(p) for p in prompt], SamplingParams(max_tokens=6, temperature=0.0))
    for p, rows in zip(prompt, out):
        ids = list(p)
        for _ in range(6):  # greedy decoding by re-running the whole sequence
            logits, _ = model(torch.tensor([ids]))
            ids.append(int(logits[0, -1].argmax()))
        assert rows[0] == ids[len(p):]


def test_static_decode_step_matches_full_forward():
    """The fixed-shape decode step (what the CUDA graph captures) against re-running the whole sequence."""
    from contextlib import nullcontext

    from sample_efficient_gpt_b200.evals.generation import GraphDecoder

    model = tiny_model()
    dec = GraphDecoder(model, 2, 24, "cpu", nullcontext())
    prompt = torch.tensor([[3, 4, 5, 6], [7, 8, 9, 10]])
    ids = prompt.clone()
    logits = dec.prefill(prompt)
    for _ in range(5):
        want, _ = model(ids)
        assert torch.allclose(logits, want[:, -1, :], atol=2e-4, rtol=1e-4)
        nxt = logits.argmax(-1, keepdim=True)
        ids = torch.cat([ids, nxt], dim=1)
        logits = dec.step(nxt)
    dec.prefill(prompt[:, :2])  # reuse of the same buffers for a shorter prompt: stale entries are masked
    assert torch.allclose(dec.step(prompt[:, 2:3]), model(prompt[:, :3])[0][:, -1, :], atol=2e-4, rtol=1e-4)


def test_sampling_rules_and_stop_tokens():
    logits = torch.tensor([[0.0, 1.0, 5.0, 2.0]])
    assert int(sample_next(logits, SamplingParams(temperature=0.0))) == 2
    g = torch.Generator().manual_seed(0)
    draws = {int(sample_next(logits, SamplingParams(temperature=1.0, top_k=2), g)) for _ in range(50)}
    assert draws <= {2, 3} and 2 in draws
    assert {int(sample_next(logits, SamplingParams(temperature=1.0, top_k=None, top_p=0.5), g)) for _ in range(20)} == {2}
    model = tiny_model()
    engine = ChatEngine(model, make_tokenizer(), "cpu", max_model_len=32, sync_every=1)
    first = engine.generate_ids([[3, 4, 5]], SamplingParams(max_tokens=5))[0][0]
    cut = engine.generate_ids([[3, 4, 5]], SamplingParams(max_tokens=5, stop_token_ids=[first[2]]))[0][0]
    assert cut == first[: first.index(first[2])]
    many = engine.generate_ids([[3, 4, 5], [6, 7]], SamplingParams(n=3, max_tokens=4, temperature=1.0, seed=1))
    assert [len(r) for r in many] == [3, 3] and all(len(x) == 4 for r in many for x in r)
    assert engine.generate_ids([list(range(3, 31)) + [3, 4, 5, 6]], SamplingParams(max_tokens=50))[0][0].__len__() == 1  # 31-token prompt, room for 1


def test_chat_rendering_and_eval_loop():
    from sample_efficient_gpt_b200.evals.chat_eval import chatcore, pick_letter, run_chat_eval, ALL_TASKS
    from sample_efficient_gpt_b200.evals.tasks.common import Task

    tok = make_tokenizer(chat_specials=True)
    engine = ChatEngine(tiny_model(), tok, "cpu", max_model_len=64)
    v = tok.get_vocab()
    ids = engine.render([{"role": "user", "content": "the cat"}, {"role": "assistant", "content": "sat"}, {"role": "user", "content": "on"}])
    assert ids == [v["<|bos|>"], v["<|user_start|>"], v["the"], v["cat"], v["<|user_end|>"], v["<|assistant_start|>"], v["sat"],
                   v["<|assistant_end|>"], v["<|user_start|>"], v["on"], v["<|user_end|>"], v["<|assistant_start|>"]]
    assert set(engine.default_stop_ids()) == {v["<|endoftext|>"], v["<|assistant_end|>"]}
    plain = ChatEngine(tiny_model(), make_tokenizer(), "cpu")
    assert plain.tokenizer.decode(plain.render([{"role": "user", "content": "the cat"}])).split()[-2:] == ["<unk>", ":"]
    assert pick_letter(" (b) maybe", ["A", "B"]) == "B" and pick_letter("zzz", ["A"]) is None

    class Fixed(Task):
        eval_type = "categorical"

        def num_examples(self):
            return 5

        def get_example(self, i):
            return {"messages": [{"role": "user", "content": "Q ?"}, {"role": "assistant", "content": "A"}], "letters": ["A", "B"]}

        def evaluate(self, conv, reply):
            return reply == "A"

    class Echo:
        def default_stop_ids(self):
            return []

        def chat(self, convs, params):
            assert params.max_tokens == 8 and all(len(c) == 1 for c in convs)
            return [["a) because"] for _ in convs]

    assert run_chat_eval("x", Echo(), 0, 1, "cpu", batch_size=2, task=Fixed(), quiet=True) == 1.0
    assert run_chat_eval("x", Echo(), 1, 2, "cpu", batch_size=2, task=Fixed(), max_problems=3, quiet=True) == 1.0
    assert isinstance(run_chat_eval("x", engine, 0, 1, "cpu", batch_size=4, task=Fixed(), quiet=True), float)
    assert chatcore({"MMLU": 0.5}) is None
    assert chatcore({t: 0.25 if t in ("ARC-Easy", "ARC-Challenge", "MMLU") else 0.0 for t in ALL_TASKS}) == pytest.approx(0.0)


def test_chat_web_api():
    from fastapi.testclient import TestClient

    from sample_efficient_gpt_b200.evals.chat_web import WorkerPool, create_app

    engine = ChatEngine(tiny_model(), make_tokenizer(chat_specials=True), "cpu", max_model_len=64)
    with TestClient(create_app(WorkerPool([engine]), max_tokens=5, temperature=0.0)) as client:
        assert client.get("/health").json() == {"status": "ok", "ready": True, "num_gpus": 1, "available_workers": 1}
        assert "<textarea" in client.get("/").text
        r = client.post("/chat/completions", json={"messages": [{"role": "user", "content": "the cat sat"}], "max_tokens": 6})
        assert r.status_code == 200
        events = [json.loads(line[6:]) for line in r.text.split("\n\n") if line.startswith("data: ")]
        assert events[-1] == {"done": True} and all("token" in e and e["gpu"] == 0 for e in events[:-1])
        text = "".join(e["token"] for e in events[:-1])
        expect = engine.chat([[{"role": "user", "content": "the cat sat"}]], SamplingParams(max_tokens=6, stop_token_ids=engine.default_stop_ids()))[0][0]
        assert text == expect
        assert client.get("/stats").json()["available_workers"] == 1  # released after the stream
        for bad in ({"messages": []}, {"messages": [{"role": "system", "content": "x"}]}, {"messages": [{"role": "user", "content": "x" * 4001}]},
                    {"messages": [{"role": "user", "content": "x"}], "temperature": 3.0}, {"messages": [{"role": "user", "content": "x"}], "top_k": 0}):
            assert client.post("/chat/completions", json=bad).status_code == 400
