"""Helpers shared by the GPU parity tests (device memory through torch, compute through libmgq)."""
import numpy as np

from oracle import oracle as O

REL_L2_TOL = 1e-4          # per output tensor, against the f64-accumulated oracle


def to_dev(arr):
    import torch
    return torch.from_numpy(np.ascontiguousarray(arr)).cuda()


def run_matmul(fmt, x, packed, k, n, addend=None, route="auto", canary=True):
    """x [m,k] numpy f32 (or torch bf16 tensor on the device) -> numpy [m,n] via the C ABI.

    With canary=True the output sits inside a larger buffer whose margins must stay untouched.
    """
    import torch
    from meganeura_b200 import ops
    xd = x if isinstance(x, torch.Tensor) else to_dev(np.asarray(x, dtype=np.float32).reshape(-1, k))
    m = xd.shape[0]
    wd = to_dev(packed)
    ad = to_dev(addend) if addend is not None else None
    if not canary:
        out = ops.matmul(fmt, xd, wd, k, n, addend=ad, route=route)
        torch.cuda.synchronize()
        return out.cpu().numpy()
    pad = 64
    buf = torch.full((m * n + 2 * pad,), 12345.0, dtype=torch.float32, device="cuda")
    out = buf[pad:pad + m * n].view(m, n)
    ops.matmul(fmt, xd, wd, k, n, addend=ad, out=out, route=route)
    torch.cuda.synchronize()
    host = buf.cpu().numpy()
    assert (host[:pad] == 12345.0).all() and (host[pad + m * n:] == 12345.0).all(), "kernel wrote outside its output"
    return host[pad:pad + m * n].reshape(m, n).copy()


def check_against_oracle(coracle, fmt, x, packed, k, n, got, addend=None, tol=REL_L2_TOL):
    want = coracle.matmul(fmt, x, packed, k, n, addend=addend, wide=True, nthreads=8)
    assert np.isfinite(got).all()
    err = O.rel_l2(got, want)
    assert err <= tol, f"rel-L2 {err:.3e} > {tol:g} (fmt={fmt}, k={k}, n={n})"
    # per-row check as well: each output row is its own tensor
    for r in range(want.shape[0]):
        assert O.rel_l2(got[r], want[r]) <= tol
    return err


def tile_columns(fmt, packed_dev, k, n, reps):
    """Device-side: the packed weight [k, n] repeated `reps` times along N (columns are independent)."""
    import torch
    bpc = k // 32
    if fmt == O.FMT_Q8:
        return packed_dev.repeat(reps)
    nb = bpc * n
    return torch.cat([packed_dev[: nb * 4].repeat(reps), packed_dev[nb * 4:].repeat(reps)])
