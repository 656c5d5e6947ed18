"""ARC (allenai/ai2_arc) as a categorical chat task; evals/tasks/arc.py:10-47 of the reference."""

from sample_efficient_gpt_b200.evals.tasks.common import Task, load_rows, render_mc


class ARC(Task):
    def __init__(self, subset, split, **kwargs):
        super().__init__(**kwargs)
        assert subset in ["ARC-Easy", "ARC-Challenge"], "ARC subset must be ARC-Easy or ARC-Challenge"
        assert split in ["train", "validation", "test"], "ARC split must be train|validation|test"
        self.ds = load_rows("allenai/ai2_arc", subset, split)

    eval_type = "categorical"

    def num_examples(self):
        return len(self.ds)

    def get_example(self, index):
        row = self.ds[index]
        letters, key = row["choices"]["label"], row["answerKey"]
        assert key in letters, f"ARC answer {key} must be one of {letters}"
        user = render_mc(row["question"], letters, row["choices"]["text"])
        return {"messages": [{"role": "user", "content": user}, {"role": "assistant", "content": key}], "letters": letters}

    def evaluate(self, conversation, assistant_response):
        assert assistant_response in conversation["letters"], f"ARC answer {assistant_response} is expected to be one of {conversation['letters']}"
        return assistant_response == conversation["messages"][-1]["content"]
