"""Block-period inference (reference: partitioning.py:1-398).

score(p) = mean over adjacent blocks of |mean_log(block j+1) - mean_log(block j)| with
mean_log = mean of log(g^2 + 1e-12) over the block, for every divisor p of numel that leaves at
least DMNB blocks; the period is the best strict local maximum among p > 8, capped above 1024 by
the smallest divisor > 1024 that divides it. Scores are computed on the GPU; this module holds the
integer logic around them.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

DMNB = 4                 # minimum number of blocks a candidate must leave (reference :6)
MIN_CANDIDATE_PERIOD = 8  # candidates must exceed this (reference :312)
PERIOD_CAP = 1024        # reference :328 ("PC")


def divisors(n: int, max_divisor: Optional[int] = None) -> List[int]:
    """The reference's divisor list, ascending (reference :13-30): every i <= sqrt(n) with i != n and
    every cofactor n // i != i. For n > 1 that is all divisors, n itself included (it comes in as
    the cofactor of 1); candidates with fewer than DMNB blocks are dropped by the callers.
    max_divisor limits the values listed."""
    if max_divisor is not None:
        max_divisor = int(max_divisor)
        if max_divisor < 1:
            raise ValueError("max_divisor must be positive, got {}.".format(max_divisor))
    small, large = [], []
    for i in range(1, math.isqrt(n) + 1):
        if n % i:
            continue
        if i != n and (max_divisor is None or i <= max_divisor):
            small.append(i)
        j = n // i
        if j != i and (max_divisor is None or j <= max_divisor):
            large.append(j)
    large.reverse()
    return small + large


def candidate_periods(n: int, max_period: Optional[int] = None, min_num_blocks: int = DMNB) -> List[int]:
    return [p for p in divisors(n, max_period) if n // p >= min_num_blocks]


def decision_periods(cands: Sequence[int]) -> List[int]:
    """The sub-list of candidates whose scores can influence the decision: every p > 8 plus the one
    candidate right before the first of them (its score is only ever a 'previous' neighbour)."""
    first = next((i for i, p in enumerate(cands) if p > MIN_CANDIDATE_PERIOD), None)
    if first is None:
        return []
    return list(cands[max(first - 1, 0):])


def _finalize_period_results(list_periods_and_scores: Sequence[Tuple[int, float]], print_results: bool,
                             flattened_length: int, threshold=None) -> int:
    """Local-maximum rule and cap (reference :277-347)."""
    ps = list(list_periods_and_scores)
    if not ps:
        raise ValueError("Expected at least one valid period candidate.")
    last_period = ps[-1][0]
    best = None
    for idx in range(1, len(ps) - 1):
        p, score = ps[idx]
        if p <= MIN_CANDIDATE_PERIOD or p == last_period:
            continue
        if score <= ps[idx - 1][1] or score <= ps[idx + 1][1]:
            continue
        if best is None or (score, p) > best:
            best = (score, p)
    if best is None:
        best_period = 1
    else:
        if not math.isfinite(best[0]):
            raise ValueError("Expected finite best score, got {}.".format(best[0]))
        best_period = best[1]
    if best_period > PERIOD_CAP:
        best_period = min(q for q in divisors(flattened_length)
                          if PERIOD_CAP < q <= best_period and best_period % q == 0)
    if print_results:
        print("Flattened length: {}".format(flattened_length))
        for idx, (p, score) in enumerate(ps):
            nxt = ps[idx + 1][1] if idx + 1 < len(ps) else None
            gap = 0.0 if nxt is None else (score / nxt if nxt != 0.0 else (0.0 if score == 0.0 else float("inf")))
            line = "p={} |  score={:.10f} | score gap = {:.3f}".format(p, score, gap)
            print("\033[92m{}\033[0m".format(line) if p == best_period else line)
    return best_period


def launch_period_scores(values: torch.Tensor, *, input_is_squared: bool, max_period: Optional[int] = None,
                         epsilon: float = 1e-12, min_num_blocks: int = DMNB, all_scores: bool = False):
    """Enqueues the score kernels for one tensor. Returns (flat_length, periods, device stats) or
    (flat_length, [], None) when there is nothing to score; no host synchronisation."""
    from .kernels.period_variance import period_scan_async

    flat = values.detach().reshape(-1)
    if not flat.is_contiguous():
        flat = flat.contiguous()
    n = flat.numel()
    cands = candidate_periods(n, max_period, min_num_blocks)
    periods = cands if all_scores else decision_periods(cands)
    if not periods:
        return n, [], None, bool(cands)
    stats = period_scan_async(flat, periods, input_is_squared=input_is_squared, epsilon=epsilon)
    return n, periods, stats, True


def decide_period(n: int, periods: Sequence[int], stats_host: Optional[torch.Tensor], print_results: bool = False) -> int:
    from .kernels.period_variance import scores_from_stats

    if not periods:
        return 1
    scores = scores_from_stats(stats_host)
    return _finalize_period_results(list(zip(periods, scores)), print_results, n)


def find_period_by_block_variance(squared_grad_flattened_values, print_results: bool = True, parameter_name=None,
                                  parameter_shape=None, backend: str = "cuda_kernel", input_is_squared: bool = True,
                                  max_period: Optional[int] = None, threshold: float = 0.25, epsilon: float = 1e-12,
                                  min_num_blocks: int = DMNB) -> int:
    """Same call as the reference (:350-398). Only the CUDA-kernel backend exists here."""
    del parameter_name, parameter_shape, threshold
    if backend != "cuda_kernel":
        raise ValueError("gefen_b200 computes period scores on the GPU only; backend must be 'cuda_kernel', "
                         "got {!r}".format(backend))
    values = squared_grad_flattened_values
    if not isinstance(values, torch.Tensor):
        raise TypeError("Expected torch.Tensor for cuda_kernel backend, got {}".format(type(values).__name__))
    if values.device.type != "cuda":
        raise ValueError("Expected a CUDA tensor for cuda_kernel backend, got device {}".format(values.device))
    n, periods, stats, _ = launch_period_scores(values, input_is_squared=input_is_squared, max_period=max_period,
                                                epsilon=epsilon, min_num_blocks=min_num_blocks,
                                                all_scores=print_results)
    return decide_period(n, periods, None if stats is None else stats.cpu(), print_results)
