"""Planner / dispatch shape list shared by the CPU oracle test and the single-GPU kernel test.

The shapes follow the case list of the reference's planner tests
(tests/test_planning.py:22-204 there): one token, K=1, no padding, padding larger than any
segment, non-power-of-two expert counts, near-degenerate skew, expert counts that exceed one
thread block or one histogram tile, and the four synthetic routings.  ``min_R`` / ``max_R``
bound the group sizes a case makes sense for (or fits one GPU's emulation for).
"""
from dataclasses import dataclass


@dataclass(frozen=True)
class ShapeCase:
    name: str
    S: int
    K: int
    epn: int
    pad: int = 128
    routing: str = "balanced"       # balanced | biased | all_local | all_remote | single_expert | duplicate_topk
    sigma: float = 0.0
    seed: int = 42
    min_R: int = 1
    max_R: int = 8
    H: int = 64


SHAPE_CASES = [
    ShapeCase("balanced_epn16", 256, 8, 16),
    ShapeCase("one_token_k1", 1, 1, 1, pad=8),
    ShapeCase("tiny_biased_slots", 3, 5, 3, pad=32, routing="biased", sigma=1.0, seed=9002, min_R=2),
    ShapeCase("no_padding", 33, 2, 2, pad=1, routing="biased", sigma=1.0, seed=10001),
    ShapeCase("odd_mild_bias", 17, 3, 3, pad=16, routing="biased", sigma=0.5, seed=10501),
    ShapeCase("odd_balanced", 17, 3, 3, pad=16, seed=11001),
    ShapeCase("near_degenerate", 64, 2, 5, routing="biased", sigma=5.0, seed=12001),
    ShapeCase("typical_bias", 32, 4, 4, pad=64, routing="biased", sigma=1.0, seed=13001),
    ShapeCase("heavy_bias", 96, 3, 7, routing="biased", sigma=2.0, seed=14001),
    ShapeCase("many_experts_256", 1024, 1, 256, pad=1),
    ShapeCase("many_experts_320", 2048, 1, 320, pad=1, max_R=4),
    ShapeCase("many_experts_320_tail", 1536, 1, 320, pad=1, min_R=4, max_R=4),
    ShapeCase("experts_beyond_block", 256, 1, 1025, pad=1, max_R=2),
    ShapeCase("all_local", 32, 4, 8, pad=16, routing="all_local"),
    ShapeCase("all_remote", 32, 4, 8, pad=16, routing="all_remote", min_R=2),
    ShapeCase("duplicate_topk", 16, 4, 4, pad=8, routing="duplicate_topk", min_R=2),
    ShapeCase("single_expert_exact_pad", 8, 2, 4, pad=8, routing="single_expert"),
    ShapeCase("single_expert_pad_tail", 9, 2, 4, pad=8, routing="single_expert"),
]

GROUP_SIZES = (1, 2, 4, 8)


def case_params():
    """(case, R) pairs that respect each case's group-size bounds and K <= E."""
    out = []
    for c in SHAPE_CASES:
        for R in GROUP_SIZES:
            if c.min_R <= R <= c.max_R and c.K <= R * c.epn:
                out.append((c, R))
    return out


def case_id(p):
    return f"{p[0].name}-R{p[1]}"
