"""Size strings and model-shape solving.

Command-line sizes accept binary suffixes: "2k" = 2048, "100m" = 100 * 2^20, "1g" = 2^30 (reference
train.py:424-434).  A model of dimension d and depth L has about  L (3e + 2f) d^2 + 2 v d  parameters
(e = expansion, f = ff_mult, v = vocabulary); the solvers below invert that estimate the way the reference
does (train.py:319-363, 589-610) so that ``--params 1g`` picks the same shape.
"""
from __future__ import annotations

import math
import re

_SUFFIX = {"k": 1024, "m": 1024 ** 2, "g": 1024 ** 3}


def parse_size_with_suffix(text):
    if not isinstance(text, str):
        return text
    m = re.fullmatch(r"(\d+(?:\.\d+)?)([kmg])?", text.strip().lower())
    if m is None:
        return float(text)
    return float(m.group(1)) * _SUFFIX.get(m.group(2), 1)


def round_to_multiple(n: float, multiple: int = 64) -> int:
    return multiple * round(n / multiple)


def _per_layer_factor(expansion: float, ff_mult: float) -> float:
    return 3 * expansion + 2 * ff_mult


def solve_for_dimension(target_params, depth, vocab_size=256, ff_mult=4, expansion=1.5) -> int:
    a = depth * _per_layer_factor(expansion, ff_mult)
    b = 2 * vocab_size
    disc = b * b + 4 * a * target_params
    if disc < 0:
        raise ValueError("no real dimension satisfies this parameter budget")
    return round_to_multiple((-b + math.sqrt(disc)) / (2 * a))


def solve_for_depth(target_params, dim, vocab_size=256, ff_mult=4, expansion=1.5) -> int:
    per_layer = dim * dim * _per_layer_factor(expansion, ff_mult)
    if per_layer <= 0:
        return 1
    return max(1, round((target_params - 2 * dim * vocab_size) / per_layer))


def calculate_model_size(config: dict) -> int:
    d, L, v = config["dim"], config["depth"], config["num_tokens"]
    return int(2 * d * v + L * d * d * _per_layer_factor(config["expansion"], config["ff_mult"]))


def get_parameter_count_str(config: dict) -> str:
    n = calculate_model_size(config)
    if n >= 1e9:
        return f"{n / 1e9:.2f}B"
    if n >= 1e6:
        return f"{n / 1e6:.1f}M"
    return f"{n / 1e3:.1f}K"


def resolve_model_config(params, dim=None, depth=None, expansion=1.5, ff_mult=4.0, num_tokens=256) -> dict:
    """Shape selection of the reference CLI: both given -> as is; one given -> solve the other; neither ->
    guess a dimension from the budget, solve the depth, then refine the dimension."""
    budget = parse_size_with_suffix(params)
    if dim is not None:
        dim = int(parse_size_with_suffix(dim))
    if dim and depth:
        pass
    elif dim:
        depth = solve_for_depth(budget, dim, num_tokens, ff_mult, expansion)
    elif depth:
        dim = solve_for_dimension(budget, depth, num_tokens, ff_mult, expansion)
    else:
        big = budget >= 1e9
        guess = round_to_multiple((1024 if big else 512) * (budget / (1e9 if big else 100e6)) ** 0.25)
        depth = solve_for_depth(budget, guess, num_tokens, ff_mult, expansion)
        dim = solve_for_dimension(budget, depth, num_tokens, ff_mult, expansion)
    return {"num_tokens": num_tokens, "dim": dim, "depth": depth, "ff_mult": ff_mult, "expansion": expansion,
            "enable_conv": False, "dropout": 0.0}
