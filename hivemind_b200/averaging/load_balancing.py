"""How much of the averaged vector each peer should reduce, given the peers' bandwidths.

Model (hivemind/averaging/load_balancing.py:13-105): peer i with bandwidth b_i that reduces a fraction x_i of a vector
spends (sum_j x_j - x_i + (n - 1) x_i) / b_i on communication; minimise the slowest peer's time with a linear
program, drop peers whose share would be smaller than ``min_size`` elements, then round shares to integers by
Hagenbach-Bischoff apportionment. Peers with unknown bandwidth get the mean; if nobody reports one, shares are equal.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import numpy as np
import scipy.optimize

from hivemind_b200.utils.logging import get_logger

logger = get_logger(__name__)
LOAD_BALANCING_LP_DECIMALS = 9


def load_balance_peers(vector_size: int, bandwidths: Sequence[Optional[float]], min_size: int = 0) -> Tuple[int, ...]:
    """Integer number of elements each peer reduces (sums to ``vector_size``); client-mode peers pass bandwidth 0."""
    specified = [item for item in bandwidths if item is not None and item > 0]
    if specified:
        default = float(np.mean(specified))
        bandwidths = [item if item is not None else default for item in bandwidths]
        scores = optimize_parts_lp(vector_size, np.asarray(bandwidths, dtype=np.float64), min_size)
    else:
        assert not all(item == 0 for item in bandwidths), "must have at least one nonzero bandwidth"
        scores = np.asarray([1.0 if item is None else 0.0 for item in bandwidths])
    return tuple(hagenbach_bishoff(vector_size, scores))


def optimize_parts_lp(vector_size: int, bandwidths: np.ndarray, min_size: int = 0) -> np.ndarray:
    """Fractions minimising max_i of peer i's communication time; variables are (x_1..x_n, xi = the max time)."""
    assert np.all(bandwidths >= 0) and np.any(bandwidths > 0)
    bandwidths = np.asarray(bandwidths, dtype=np.float64)
    permutation = np.argsort(-bandwidths)
    bandwidths = bandwidths[permutation]
    bandwidths = bandwidths / bandwidths[0]  # only ratios matter; keeps the program well scaled
    is_nonzero = bandwidths != 0
    group_size = len(bandwidths)
    num_variables = group_size + 1  # [w_1, ..., w_N, xi]

    c = np.zeros(num_variables, dtype=np.float64)
    c[-1] = 1.0  # minimise xi
    # the optimum is often degenerate (e.g. two peers: traffic does not depend on the split); among optimal
    # solutions prefer loading faster peers, via a vanishing cost that grows with the bandwidth rank
    c[:group_size] = 1e-6 * np.arange(group_size) / group_size

    # the shares sum to one
    a_eq, b_eq = np.ones((1, num_variables)), np.ones(1)
    a_eq[0, -1] = 0.0

    # time of peer i: (1 - x_i + (n-1) x_i) / b_i = (1 + (n-2) x_i) / b_i <= xi, for peers with bandwidth;
    # x_i >= 0 for everybody, x_i <= 0 for peers without bandwidth
    nonnegative = np.concatenate([-np.eye(group_size), np.zeros((group_size, 1))], axis=1)
    time_rows = np.zeros((group_size, num_variables))
    time_rhs = np.zeros(group_size)
    for i in range(group_size):
        if is_nonzero[i]:
            time_rows[i, i] = (group_size - 2.0) / bandwidths[i]
            time_rows[i, -1] = -1.0
            time_rhs[i] = -1.0 / bandwidths[i]
        else:
            time_rows[i, i] = 1.0
    a_ub = np.concatenate([nonnegative, time_rows])
    b_ub = np.concatenate([np.zeros(group_size), time_rhs])

    solution = scipy.optimize.linprog(c, A_ub=a_ub, b_ub=b_ub, A_eq=a_eq, b_eq=b_eq, method="highs",
                                      bounds=[(None, None)] * num_variables)
    if solution.success:
        peer_scores = solution.x[:group_size]
        # peers that would get fewer than min_size elements are excluded and their share is redistributed
        if np.max(peer_scores) >= min_size / float(vector_size):
            peer_scores[peer_scores < min_size / float(vector_size)] = 0.0
        peer_scores = np.round(np.maximum(peer_scores, 0.0), LOAD_BALANCING_LP_DECIMALS)
    else:
        logger.error(f"Failed to solve load-balancing for bandwidths {bandwidths}")
        peer_scores = np.ones(group_size) * is_nonzero
    return peer_scores[np.argsort(permutation)]


def hagenbach_bishoff(vector_size: int, scores: Sequence[float]) -> Sequence[int]:
    """Split ``vector_size`` seats in proportion to ``scores``: floor shares first, then one seat at a time to the
    party with the highest score / (seats + 1)."""
    scores = np.asarray(scores, dtype=np.float64)
    total_score = scores.sum()
    allocated = np.floor(vector_size * scores / total_score).astype(np.int64)
    while allocated.sum() < vector_size:
        quotients = scores / (allocated + 1)
        allocated[int(np.argmax(quotients))] += 1
    return allocated.tolist()
