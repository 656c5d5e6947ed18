"""Sample text from a checkpoint (utils/sample_outputs.py of the reference).

    python -m sample_efficient_gpt_b200.utils.sample_outputs --checkpoint run/8000.pt --tokenizer tok_dir --prompt "Once"
"""

from argparse import ArgumentParser

from sample_efficient_gpt_b200.utils.logger import logger


def parse_args(argv=None):
    p = ArgumentParser()
    p.add_argument("--checkpoint", required=True)
    p.add_argument("--prompt", default="Once")
    p.add_argument("--tokenizer", required=True, help="directory of a fast tokenizer")
    p.add_argument("--eos-prob-multiplier", default=1, type=float)
    p.add_argument("--top-p", default=0.4, type=float)
    p.add_argument("--temperature", default=0.7, type=float)
    p.add_argument("--max-steps", default=512, type=int)
    p.add_argument("--device", default="cuda", type=str)
    return p.parse_args(argv)


def main(argv=None) -> str:
    from sample_efficient_gpt_b200.training.trainer import Trainer

    a = parse_args(argv)
    trainer = Trainer(load_from=a.checkpoint, load_components="infer", **{"trainer.device": a.device, "data.tokenizer_path": a.tokenizer})
    eos_token_id = list(trainer.tokenizer.added_tokens_decoder)[0]
    logger.info(f"EOS {eos_token_id}")
    text, _ = trainer.generate(a.prompt, eos_token_id, top_p=a.top_p, temperature=a.temperature, max_steps=a.max_steps,
                               eos_prob_multiplier=a.eos_prob_multiplier)
    logger.info(text)
    return text


if __name__ == "__main__":
    main()
