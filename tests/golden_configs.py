"""The tiny configurations whose logits from the reference's own kernels are committed under
``tests/golden/``: the three test configurations without frequency scaling (the reference has
none), differing in every size, in tying, theta and eps."""
from helpers import TINY_A, TINY_B, TINY_C, random_tokens

GOLDEN = {
    "A": (dict(TINY_A), 0),
    "B": (dict(TINY_B, rope_scaling=None), 1),
    "C": (dict(TINY_C), 5),
}
LENGTHS = {"A": 40, "B": 33, "C": 47}


def tokens_for(name: str):
    cfg, seed = GOLDEN[name]
    return random_tokens(LENGTHS[name], cfg["vocab_size"], 100 + seed)
