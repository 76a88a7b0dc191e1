"""Shared test helpers: seeded inputs, tolerances and the oracle comparison."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import oracle  # noqa: E402

# Tolerance stated by the task for this floating-point path: kernel output (bf16)
# against the fp32-softmax oracle on identical bf16 inputs.
REL_L2_TOL = 1e-2
MAX_ABS_TOL = 2e-2


def seeded_bf16(*shape, seed: int) -> torch.Tensor:
    """i.i.d. N(0,1) from a seeded CPU generator, rounded to bf16 (RNE)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).bfloat16()


def assert_close(got: torch.Tensor, want: torch.Tensor, what: str = "", rel_tol: float = REL_L2_TOL,
                 abs_tol: float = MAX_ABS_TOL):
    rel, mx = oracle.error_metrics(got.detach().cpu(), want.detach().cpu())
    assert rel <= rel_tol and mx <= abs_tol, f"{what}: relL2={rel:.3e} (tol {rel_tol}), max-abs={mx:.3e} (tol {abs_tol})"
    return rel, mx


def sample_rows(seq: int, nq: int, n: int, seed: int) -> list[int]:
    """Flat (token*nq + head) row indices: the first and last tokens plus a seeded random sample."""
    g = torch.Generator().manual_seed(seed)
    total = seq * nq
    picks = set(torch.randint(0, total, (n,), generator=g).tolist())
    picks.update(range(min(nq, total)))
    picks.update(range(max(0, total - nq), total))
    return sorted(picks)
