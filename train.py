"""``python train.py --config ... --config-key ... --override ...`` (see sample_efficient_gpt_b200/train.py)."""

from sample_efficient_gpt_b200.train import main

if __name__ == "__main__":
    main()
