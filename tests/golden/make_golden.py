"""Generates tests/golden/ref_vectors.npz: seeded inputs and the outputs VibeTensor's own CPU
code (oracle/_ref/libvbt_ref_cpu.so, built by oracle/build_ref.sh from the reference
checkout) produces for them.  Run where the reference checkout is mounted:

    python tests/golden/make_golden.py

The fixture lets machines without the reference build (and without oracle/_ref) still pin
the C restatement and the CUDA path to the reference's results.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402


def main():
    oracle.build(ref_dir=sys.argv[1] if len(sys.argv) > 1 else None)  # argument 1 or VBT_REFERENCE_DIR: the reference checkout
    R = oracle.ref()
    F32, I64 = oracle.F32, oracle.I64
    rng = np.random.default_rng(20240)
    g = {}

    # dim reductions, fp32 [64, 96] contiguous and transposed view
    x = rng.standard_normal((64, 96), dtype=np.float32)
    g["red_x"] = x
    g["red_sum_m1"] = R.sum(x, F32, [-1])
    g["red_sum_0"] = R.sum(x, F32, [0])
    g["red_mean_0"] = R.sum(x, F32, [0], mean=True)
    g["red_sum_all"] = R.sum(x, F32, [])
    g["red_amax_m1"] = R.minmax("amax", x, F32, -1)
    g["red_amin_0"] = R.minmax("amin", x, F32, 0)
    v, i = R.minmax("argmax", x, F32, -1)
    g["red_argmax_m1_val"], g["red_argmax_m1_idx"] = v, i
    xt = x.T
    g["red_t_sum_m1"] = R.sum(xt, F32, [-1])
    v, i = R.minmax("argmax", xt, F32, -1)
    g["red_t_argmax_m1_idx"] = i
    # ties: first maximum wins
    xtie = rng.integers(0, 4, (16, 33)).astype(np.float32)
    g["red_tie_x"] = xtie
    g["red_tie_argmax_idx"] = R.minmax("argmax", xtie, F32, -1)[1]
    g["red_tie_argmax0_idx"] = R.minmax("argmax", xtie, F32, 0)[1]
    xi = rng.integers(-1000, 1000, (17, 40)).astype(np.int64)
    g["red_i64_x"] = xi
    g["red_i64_sum_m1"] = R.sum(xi, I64, [-1])
    g["red_i64_amax_0"] = R.minmax("amax", xi, I64, 0)
    g["red_i64_argmax_m1_idx"] = R.minmax("argmax", xi, I64, -1)[1]
    x3 = rng.standard_normal((5, 7, 9), dtype=np.float32)
    g["red3_x"] = x3
    g["red3_sum_1"] = R.sum(x3, F32, [1])
    g["red3_sum_02"] = R.sum(x3, F32, [0, 2])
    g["red3_mean_12_keep"] = R.sum(x3, F32, [1, 2], keepdim=True, mean=True)

    # elementwise fp32 / int64 with broadcast
    a = rng.standard_normal((6, 1, 16), dtype=np.float32)
    b = rng.standard_normal((5, 16), dtype=np.float32)
    g["ew_a"], g["ew_b"] = a, b
    for op in ["add", "sub", "mul", "div"]:
        g["ew_" + op] = R.elementwise(op, a, b, F32)
    for op in ["eq", "ne", "lt", "gt", "le", "ge"]:
        g["ew_" + op] = R.elementwise(op, a, b, F32, out_dtype=oracle.BOOL)
    for op in ["relu", "abs", "neg", "reciprocal"]:
        g["ew_" + op] = R.elementwise(op, a, None, F32)
    ai = rng.integers(-50, 50, (4, 1, 8)).astype(np.int64)
    bi = rng.integers(-50, 50, (3, 8)).astype(np.int64)
    g["ew_ai"], g["ew_bi"] = ai, bi
    for op in ["add", "sub", "mul"]:
        g["ew_i64_" + op] = R.elementwise(op, ai, bi, I64)

    # row gather / scatter (index / index_put_ / embedding)
    table = rng.standard_normal((50, 12), dtype=np.float32)
    idx = rng.integers(-50, 50, 200).astype(np.int64)
    g["ix_table"], g["ix_idx"] = table, idx
    g["ix_gather"] = R.index_rows(table, idx, F32)
    g["ix_embedding"] = R.embedding(table, idx % 50)
    vals = rng.standard_normal((200, 12), dtype=np.float32)
    g["ix_vals"] = vals
    g["ix_put_acc"] = R.index_put_rows(np.zeros((50, 12), np.float32), idx, vals, F32, True)
    vi = rng.integers(-1000, 1001, (200, 12)).astype(np.int64)
    g["ix_vals_i64"] = vi
    g["ix_put_acc_i64"] = R.index_put_rows(np.zeros((50, 12), np.int64), idx, vi, I64, True)
    perm = rng.permutation(50).astype(np.int64)[:30]
    g["ix_perm"] = perm
    g["ix_put_overwrite"] = R.index_put_rows(table.copy(), perm, vals[:30].copy(), F32, False)

    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, os.path.getsize(out), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
