"""MBPP-lite pass@1 of a checkpoint with this package's own BPE tokenizer files (utils/eval_mbpp.py of the reference).

    python -m sample_efficient_gpt_b200.utils.eval_mbpp --checkpoint run/8000.pt --tokenizer tok_dir

``tok_dir`` holds ``vocab.pickle`` and ``merges.pickle``.  The model's output (prompt + continuation) is scored as a whole
file.
"""

from argparse import ArgumentParser
from pathlib import Path

import torch

from sample_efficient_gpt_b200.utils.logger import logger


def parse_args(argv=None):
    p = ArgumentParser()
    p.add_argument("--checkpoint", required=True)
    p.add_argument("--tokenizer", required=True)
    p.add_argument("--top-p", default=0.4, type=float)
    p.add_argument("--temperature", default=0.7, type=float)
    p.add_argument("--max-steps", default=512, type=int)
    p.add_argument("--device", default="cuda", type=str)
    p.add_argument("--timeout", default=8.0, type=float)
    return p.parse_args(argv)


def main(argv=None) -> dict:
    from sample_efficient_gpt_b200.evals.mbpp_eval import SimpleMBPPEvaluator
    from sample_efficient_gpt_b200.tokenizer.tokenizer import Tokenizer
    from sample_efficient_gpt_b200.training.trainer import Trainer

    a = parse_args(argv)
    trainer = Trainer(load_from=a.checkpoint, load_components="infer", **{"trainer.device": a.device})
    tok = Tokenizer.from_files(Path(a.tokenizer) / "vocab.pickle", Path(a.tokenizer) / "merges.pickle", special_tokens=["<|endoftext|>"])
    eos = tok.encode(tok.special_tokens[0])[0]
    logger.info(f"EOS {eos}")

    def generate(prompt: str) -> str:
        ids = torch.tensor(tok.encode(prompt)).unsqueeze(0).to(trainer.device)
        out, _ = trainer.model.generate(ids, eos, top_p=a.top_p, temperature=a.temperature, max_steps=a.max_steps)
        return tok.decode([t for t in out[0].cpu().tolist() if t != eos])

    metrics = SimpleMBPPEvaluator(dataset="lite", timeout=a.timeout).evaluate_with_generate(generate, num_samples=1, mode="solution")
    print(metrics["pass_at_k"])
    return metrics


if __name__ == "__main__":
    main()
