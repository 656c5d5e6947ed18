"""MMLU (cais/mmlu) as a categorical chat task; evals/tasks/mmlu.py:10-117 of the reference."""

from sample_efficient_gpt_b200.evals.tasks.common import Rows, Task, load_rows, render_mc


class MMLU(Task):
    letters = ("A", "B", "C", "D")
    eval_type = "categorical"

    def __init__(self, subset, split, **kwargs):
        super().__init__(**kwargs)
        assert subset in ["all", "auxiliary_train"], f"subset {subset} must be all|auxiliary_train"
        assert split in ["train", "validation", "dev", "test"], f"split {split} must be train|validation|dev|test"
        assert subset != "auxiliary_train" or split == "train", "auxiliary_train must be split into train"
        self.subset, self.split = subset, split
        self.ds = load_rows("cais/mmlu", subset, split)
        self._unwrap = subset == "auxiliary_train"  # those rows sit inside an extra {'train': row} wrapper

    def num_examples(self):
        return len(self.ds)

    def get_example(self, index):
        row = self.ds[index]
        if self._unwrap and "train" in row:
            row = row["train"]
        assert len(row["choices"]) == 4, "MMLU should have 4 choices"
        user = render_mc(row["question"], self.letters, row["choices"])
        messages = [{"role": "user", "content": user}, {"role": "assistant", "content": self.letters[row["answer"]]}]
        return {"messages": messages, "subject": row.get("subject", ""), "letters": self.letters}

    def evaluate(self, conversation, assistant_response):
        assert assistant_response in self.letters, f"MMLU answer {assistant_response} is expected to be one of {self.letters}"
        return assistant_response.strip() == conversation["messages"][-1]["content"].strip()
