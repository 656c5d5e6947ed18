"""Nemotron post-training set v2 (math + code + stem + chat splits joined); evals/tasks/nemotron.py:11-55 of the
reference."""

from sample_efficient_gpt_b200.evals.tasks.common import ConversationTask, Rows, load_rows


class Nemotron(ConversationTask):
    SPLITS = ("math", "code", "stem", "chat")

    def __init__(self, **kwargs):
        rows = []
        for split in self.SPLITS:
            rows.extend(load_rows("nvidia/Nemotron-Post-Training-Dataset-v2", None, split, seed=None))
        super().__init__(Rows(rows).shuffle(seed=42), **kwargs)
