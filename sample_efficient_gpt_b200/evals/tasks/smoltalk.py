"""SmolTalk (HuggingFaceTB/smol-smoltalk) conversations; evals/tasks/smoltalk.py:11-51 of the reference."""

from sample_efficient_gpt_b200.evals.tasks.common import ConversationTask, load_rows


class SmolTalk(ConversationTask):
    def __init__(self, split, **kwargs):
        assert split in ["train", "test"], "SmolTalk split must be train|test"
        super().__init__(load_rows("HuggingFaceTB/smol-smoltalk", None, split), **kwargs)
