"""Shared helpers of the test-suite."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerances stated by the benchmark definition: bf16 result against an fp32-accumulated
# reference on the same (already rounded) inputs, normalised by max|ref|; FP8 against the
# loop on the same quantised inputs.
BF16_REL_TOL = 1e-2
FP8_REL_TOL = 2e-2


def bf16_from_bits(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def load_npz(name):
    return np.load(os.path.join(GOLDEN, name))


def random_m_sizes(G, M, gen):
    """Sorted random cut points, as the reference's tests draw them
    (dev/triton_groupGEMM/testing/base_testing.py:106-116); groups may be empty."""
    if G == 1:
        return torch.tensor([M], dtype=torch.int32)
    ends, _ = torch.sort(torch.randint(0, M, (G - 1,), generator=gen))
    ends = ends.tolist()
    starts = [0] + ends
    ends = ends + [M]
    return torch.tensor([e - s for s, e in zip(starts, ends)], dtype=torch.int32)
