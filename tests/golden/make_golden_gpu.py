"""Generates ref_triton_vectors.npz: outputs of the reference's OWN Triton kernels (softmax,
log_softmax, RMSNorm forward and backward, gather, scatter_add) for the seeded inputs of
triton_cases.py, in fp32 and bf16.  Needs a GPU and baseline/_ref (baseline/install_ref.sh):

    python tests/golden/make_golden_gpu.py [output.npz]

The committed fixture pins both the CPU oracle and the CUDA path to what the reference's
kernels really compute, not only to torch.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)
import triton_cases as tc  # noqa: E402
from baseline import ref_kernels  # noqa: E402


def bits(t):
    t = t.detach().contiguous().cpu()
    return t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_triton_vectors.npz")
    R = ref_kernels.load()
    g = {}
    for shape in tc.ROW_SHAPES:
        x, dy, gamma = tc.row_case(shape)
        for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            key = f"{shape[0]}x{shape[1]}_{tag}"
            tx = torch.from_numpy(x).cuda().to(dt).requires_grad_(True)
            tdy = torch.from_numpy(dy).cuda().to(dt)
            tg = torch.from_numpy(gamma).cuda().requires_grad_(True)
            y = R.softmax(tx, -1)
            g[f"softmax_{key}"] = bits(y)
            g[f"softmax_bwd_{key}"] = bits(torch.autograd.grad(y, tx, tdy)[0])
            ly = R.log_softmax(tx, -1)
            g[f"log_softmax_{key}"] = bits(ly)
            g[f"log_softmax_bwd_{key}"] = bits(torch.autograd.grad(ly, tx, tdy)[0])
            o = R.rmsnorm_fn.apply(tx, tg, tc.EPS)
            g[f"rmsnorm_{key}"] = bits(o)
            try:
                g[f"rmsnorm_inv_{key}"] = o.grad_fn.saved_tensors[1].detach().float().cpu().numpy()
            except Exception:
                pass
            dx, dg = torch.autograd.grad(o, (tx, tg), tdy)
            g[f"rmsnorm_bwd_dx_{key}"] = bits(dx)
            g[f"rmsnorm_bwd_dgamma_{key}"] = dg.detach().float().cpu().numpy()
    table, idx_u, idx_z, upd = tc.index_case()
    tt = torch.from_numpy(table).cuda()
    g["gather_rows"] = R.gather(tt, 0, torch.from_numpy(idx_u).cuda()).cpu().numpy()
    acc = torch.zeros_like(tt)
    res = R.scatter_add(acc, 0, torch.from_numpy(idx_z).cuda(), torch.from_numpy(upd).cuda())
    g["scatter_add_rows"] = (res if res is not None else acc).cpu().numpy()
    torch.cuda.synchronize()
    np.savez_compressed(out_path, **g)
    print(f"wrote {out_path}: {len(g)} arrays, {sum(v.nbytes for v in g.values()) / 1e6:.1f} MB")


if __name__ == "__main__":
    main()
