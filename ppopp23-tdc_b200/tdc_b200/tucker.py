"""Tucker-2 factorisation of a dense conv filter at load time, without tensorly.

The reference calls tensorly's `partial_tucker(dense_w, modes=[0, 1], rank=[R2, R1], init='svd')`
(inference/TKConv.py:75-80).  tensorly (0.7.x, reference README:14) is not vendored in the
reference and not installed here; what follows restates its published algorithm — higher-order
orthogonal iteration with an SVD start:

  start:   factor_m = leading rank_m left singular vectors of the mode-m unfolding
  sweep:   for each mode m: project the tensor on the OTHER mode's factor, take the leading
           rank_m left singular vectors of the mode-m unfolding of the result
  stop:    when the relative reconstruction error sqrt(|T|^2 - |core|^2) / |T| changes by less
           than `tol` between sweeps, or after `n_iter_max` sweeps
  core:    T x_0 U0^T x_1 U1^T

Parity with tensorly itself is unpinned (no tensorly to compare with); the tests hold the
properties that define the result: orthonormal factors, exact recovery of a tensor of exact
multilinear rank, and an error no larger than the truncated-SVD start.
Runs on whatever device the tensor is on (torch.linalg), in fp64, results returned in fp32.
"""
import torch


def _unfold(t, mode):
    return torch.movedim(t, mode, 0).reshape(t.shape[mode], -1)


def _leading(mat, rank):
    u, _, _ = torch.linalg.svd(mat, full_matrices=False)
    return u[:, :rank]


def partial_tucker_hosvd(dense_w, ranks, n_iter_max=100, tol=1e-4):
    """dense_w [K, C, kh, kw], ranks [R2, R1] -> core [R2, R1, kh, kw], (last_factor [K, R2],
    first_factor [C, R1]) — the return convention of tensorly's partial_tucker on modes (0, 1)."""
    t = dense_w.detach().double()
    r_out, r_in = int(ranks[0]), int(ranks[1])
    u0, u1 = _leading(_unfold(t, 0), r_out), _leading(_unfold(t, 1), r_in)
    norm = torch.linalg.norm(t)
    prev = None
    for _ in range(n_iter_max):
        u0 = _leading(_unfold(torch.einsum("kcrs,cb->kbrs", t, u1), 0), r_out)
        u1 = _leading(_unfold(torch.einsum("kcrs,ka->acrs", t, u0), 1), r_in)
        core = torch.einsum("kcrs,ka,cb->abrs", t, u0, u1)
        err = torch.sqrt(torch.clamp(norm ** 2 - torch.linalg.norm(core) ** 2, min=0.0)) / norm
        if prev is not None and abs(float(prev - err)) < tol:
            break
        prev = err
    core = torch.einsum("kcrs,ka,cb->abrs", t, u0, u1)
    return core.float(), (u0.float(), u1.float())


def tucker_to_dense(core, last_factor, first_factor):
    """W[k,c,r,s] = sum_{a,b} core[a,b,r,s] * last[k,a] * first[c,b] (tensorly's tucker_to_tensor)."""
    return torch.einsum("abrs,ka,cb->kcrs", core.double(), last_factor.double(), first_factor.double()).float()
