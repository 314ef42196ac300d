"""CPU restatement (numpy) of the WKV-7 state scan of the reference's TimeMix block.

TEST INFRASTRUCTURE ONLY: the parity checker of pb_wkv7_forward.  Nothing in the shipped package imports it.

PARITY UNPINNED: the reference ships no tests or vectors for this scan and cannot be imported here (jax
is not installed); this restatement follows its source text, pratchya/_nnx_impl/_module.py:187-207.
"""
from __future__ import annotations

import numpy as np


def wkv_state_scan(wkv_state, decay, iclr, removal_k, replacement_k, v, r, n_head: int, dtype=np.float32):
    """pratchya/_nnx_impl/_module.py:187-207.  The six inputs are [B, T, C]; wkv_state is [B, N, H, H] with
    C = N * H.  Returns (wkv_state [B, N, H, H], out [B, T, C]) -- `out` in the [B, T, C] order the reference
    has after its transpose (:210).  `dtype=np.float64` gives the high-precision value tolerances are
    measured against; np.float32 is the reference's own precision."""
    B, T, C = np.shape(decay)
    N = n_head
    H = C // N
    S = np.array(wkv_state, dtype=dtype).reshape(B, N, H, H)
    out = np.empty((T, B, C), dtype=dtype)
    col = lambda a, t: np.asarray(a[:, t], dtype=dtype).reshape(B, N, H, 1)           # :190-195
    for t in range(T):
        decay_t, iclr_t, removal_k_t = col(decay, t), col(iclr, t), col(removal_k, t)
        replacement_k_t, v_t, r_t = col(replacement_k, t), col(v, t), col(r, t)
        mT = lambda a: np.swapaxes(a, -1, -2)
        S = S * mT(decay_t) - S @ removal_k_t @ mT(iclr_t * removal_k_t)              # :197
        S = S + v_t @ mT(replacement_k_t)                                             # :198
        y = S @ r_t                                                                   # :199
        out[t] = y.reshape(B, C)                                                      # :201
    return S, np.ascontiguousarray(out.transpose(1, 0, 2))                            # :210
