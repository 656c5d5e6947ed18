"""HumanEval (openai/openai_humaneval) as a generative chat task scored by running the tests;
evals/tasks/humaneval.py:13-99 of the reference."""

import re

from sample_efficient_gpt_b200.evals.execution import execute_code
from sample_efficient_gpt_b200.evals.tasks.common import Task, load_rows


def extract_imports(prompt: str) -> str:
    """Leading import lines of a program (comments and blank lines skipped; stops at the first other line)."""
    found = []
    for line in prompt.split("\n"):
        s = line.strip()
        if s.startswith(("import ", "from ")):
            found.append(s)
        elif s and not s.startswith("#"):
            break
    return "\n".join(found)


def extract_program(completion: str) -> str:
    """First fenced code block (```python or ```), else the whole reply."""
    blocks = re.findall(r"```(?:python)?\s*\n(.*?)\n```", completion, re.DOTALL)
    return (blocks[0] if blocks else completion).strip()


class HumanEval(Task):
    eval_type = "generative"

    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self.ds = load_rows("openai/openai_humaneval", None, "test")

    def num_examples(self):
        return len(self.ds)

    def get_example(self, index):
        row = self.ds[index]
        messages = [
            {"role": "user", "content": row["prompt"]},
            {"role": "assistant", "content": f"{row['prompt']}\n{row['canonical_solution']}"},
        ]
        return {"messages": messages, "entry_point": row["entry_point"], "test": row["test"]}

    def evaluate(self, conversation, completion):
        program = "\n\n".join([extract_imports(conversation["messages"][0]["content"]), extract_program(completion), conversation["test"]])
        return execute_code(program + f"\ncheck({conversation['entry_point']})").success
