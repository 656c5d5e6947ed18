"""Tulu 3 SFT mixture (allenai/tulu-3-sft-mixture) conversations; evals/tasks/tulu3.py:11-54 of the reference."""

from sample_efficient_gpt_b200.evals.tasks.common import ConversationTask, load_rows


class Tulu3(ConversationTask):
    def __init__(self, split, **kwargs):
        assert split in ["train", "test"], "Tulu3 split must be train|test"
        super().__init__(load_rows("allenai/tulu-3-sft-mixture", None, split), **kwargs)
