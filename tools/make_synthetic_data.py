"""Write a seeded uniform-random ``uint16`` token file (the format ``train.py`` reads)."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gpt_from_scratch_b200.data import write_synthetic_tokens  # noqa: E402

if __name__ == "__main__":
    p = argparse.ArgumentParser()
    p.add_argument("--output", required=True)
    p.add_argument("--num-tokens", type=int, default=1 << 24)
    p.add_argument("--vocab-size", type=int, default=50257)
    p.add_argument("--seed", type=int, default=1234)
    a = p.parse_args()
    print(write_synthetic_tokens(a.output, a.num_tokens, a.vocab_size, a.seed))
