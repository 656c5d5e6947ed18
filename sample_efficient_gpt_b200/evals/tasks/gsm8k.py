"""GSM8K (openai/gsm8k) as a generative chat task; evals/tasks/gsm8k.py:23-148 of the reference.

The dataset marks calculator calls as ``<<expr=result>>``; the assistant turn is the solution with every such marker
split into its expression and result on separate lines, and the final line ``#### <number>`` carries the answer.
"""

import re
from copy import deepcopy

from sample_efficient_gpt_b200.evals.tasks.common import Task, load_rows

GSM_RE = re.compile(r"#### (\-?[0-9\.\,]+)")
LLAMA_SYSTEM_PROMPT = (
    "Given the following problem, reason and give a final answer to the problem.\nProblem: {question}\n"
    'Your response should end with "#### [answer]" where [answer] is the response to the problem.\n'
)


def extract_answer(completion: str):
    m = GSM_RE.search(completion)
    return m.group(1).strip().replace(",", "") if m else None


def answer_text(answer: str) -> str:
    lines = []
    for piece in re.split(r"(<<[^>]+>>)", answer):
        if piece.startswith("<<") and piece.endswith(">>"):
            expr, _, result = piece[2:-2].rpartition("=") if "=" in piece else (piece[2:-2], "", "")
            lines += [expr, result]
        else:
            lines.append(piece)
    return "\n".join(lines)


class GSM8K(Task):
    eval_type = "generative"

    def __init__(self, subset, split, few_shot: bool = False, use_llama_system_prompt: bool = False, **kwargs):
        super().__init__(**kwargs)
        assert subset in ["main", "socratic"], "GSM8K subset must be main|socratic"
        assert split in ["train", "test"], "GSM8K split must be train|test"
        self.use_llama_system_prompt = use_llama_system_prompt
        self.ds = load_rows("openai/gsm8k", subset, split)
        self.few_shot_examples = []
        if few_shot:  # the first five training problems, unshuffled
            support = load_rows("openai/gsm8k", subset, "train", seed=None)
            for i in range(min(5, len(support))):
                self.few_shot_examples.append((self._format_question(support[i]["question"]), answer_text(support[i]["answer"])))

    def num_examples(self):
        return len(self.ds)

    def _format_question(self, question):
        return LLAMA_SYSTEM_PROMPT.format(question=question) if self.use_llama_system_prompt else question

    def _build_answer_parts(self, answer: str):
        return answer_text(answer)

    def get_example(self, index):
        row = self.ds[index]
        messages = []
        for q, a in self.few_shot_examples:
            messages += [{"role": "user", "content": q}, {"role": "assistant", "content": deepcopy(a)}]
        messages += [
            {"role": "user", "content": self._format_question(row["question"])},
            {"role": "assistant", "content": answer_text(row["answer"])},
        ]
        return {"messages": messages}

    def evaluate(self, conversation, assistant_response: str):
        assert isinstance(assistant_response, str), "Assuming simple string response for now"
        last = conversation["messages"][-1]
        assert last["role"] == "assistant", "Last message must be from the Assistant"
        return int(extract_answer(assistant_response) == extract_answer(last["content"].split("\n")[-1]))

    def reward(self, conversation, assistant_response):
        return float(self.evaluate(conversation, assistant_response))
