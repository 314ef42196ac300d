"""Generates tests/golden/quant_golden.npz from the CPU oracle.

    python tests/golden/make_golden.py

The reference cannot be imported on this image (jax is not installed), so these vectors are
produced by the oracle (oracle/qarr_oracle.py), whose rule is pinned by the hand-derived known
answers of tests/test_oracle_kat.py.  They guard the oracle and the CUDA path against silent
changes; they are not outputs of the reference itself.
"""
import sys
from pathlib import Path

import ml_dtypes
import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import qarr_oracle as o  # noqa: E402

CASES = {
    "act_1x128": ((4, 1024), (1, 128), "outliers"),
    "weight_128x128": ((128, 256), (128, 128), "weights"),
    "lora_128x1": ((128, 16), (128, 1), "weights"),
    "small_1x16": ((8, 64), (1, 16), "outliers"),
    "small_4x4": ((8, 16), (4, 4), "outliers"),
    "heavy_tail": ((2, 1024), (1, 128), "student_t"),
}


def make_input(shape, kind, seed):
    rng = np.random.default_rng(seed)
    if kind == "student_t":
        return rng.standard_t(3, size=shape).astype(np.float32)
    if kind == "weights":
        return (rng.standard_normal(shape) * 0.02).astype(np.float32)
    x = rng.standard_normal(shape).astype(np.float32)
    x[rng.random(shape) < 0.01] *= 64
    return x


def main():
    out = {}
    for i, (name, (shape, grid, kind)) in enumerate(CASES.items()):
        x = make_input(shape, kind, 1000 + i).astype(ml_dtypes.bfloat16).astype(np.float32)   # bf16-representable
        q, s8, s32 = o.quantize_impl(x, grid)
        out[f"{name}.x"] = x
        out[f"{name}.grid"] = np.array(grid)
        out[f"{name}.q"] = q.view(np.uint8)
        out[f"{name}.sc8"] = s8
        out[f"{name}.sc32"] = s32
        out[f"{name}.dq_bf16"] = o.dequantize_impl(q, s8, s32, ml_dtypes.bfloat16, grid).view(np.uint16)
    np.savez_compressed(Path(__file__).with_name("quant_golden.npz"), **out)
    print("wrote", len(CASES), "cases")
    write_derived()


def relu2_middle(y, grid=(1, 128)):
    """ChannelMix between its two Linears: dq(q(y)) in f32, relu, square, quantize (the oracle's steps)."""
    k = o.dequantize_impl(*o.quantize_impl(y, grid), np.float32, grid).astype(np.float32)
    k = (np.maximum(k, 0) ** 2).astype(np.float32)
    return o.quantize_impl(k, grid)


def write_derived():
    """derived_golden.npz: the optimizer's momentum step and the ChannelMix middle, from the oracle."""
    out = {}
    for i, (name, shape, grid) in enumerate([("mom_tensor_wide", (64, 64), (16, 16)), ("mom_rows", (2, 1024), (1, 128))]):
        rng = np.random.default_rng(2000 + i)
        g = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
        m = (rng.standard_normal(shape) * 5e-4).astype(np.float32)
        gq, mq = o.quantize_impl(g, grid), o.quantize_impl(m, grid)
        c, nm = o.momentum_update(gq, mq, grid, 0.9, 0.99)
        out[f"{name}.g"], out[f"{name}.m"], out[f"{name}.grid"] = g, m, np.array(grid)
        out[f"{name}.c"] = c
        out[f"{name}.q"], out[f"{name}.sc8"], out[f"{name}.sc32"] = nm[0].view(np.uint8), nm[1], nm[2]
    y = make_input((2, 1024), "outliers", 3000)
    kq = relu2_middle(y)
    out["relu2.y"] = y
    out["relu2.q"], out["relu2.sc8"], out["relu2.sc32"] = kq[0].view(np.uint8), kq[1], kq[2]
    np.savez_compressed(Path(__file__).with_name("derived_golden.npz"), **out)
    print("wrote derived cases")


if __name__ == "__main__":
    main()
