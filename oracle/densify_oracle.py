"""CPU restatement (plain torch) of the reference's densification.  TEST INFRASTRUCTURE ONLY.

Follows fast_2d_gs/gaussian_splatting.py:623-628 (densify), :608-622 (densify_and_clone), fast_2d_gs/network.py:1156-1185
(densify_and_split for 2-D scales), gaussian_splatting.py:570-580 (densification_postfix), :557-568 (prune_points) and
:498-548 (change_optimizer: 'concat' appends zero moments, 'prune' indexes them).  Pinned by tests/golden/densify.npz,
which the reference's own methods produced.
"""
import torch


def quat_to_matrix(q):
    x, y, z, w = torch.nn.functional.normalize(q, dim=-1).unbind(-1)
    return torch.stack([1 - 2 * y * y - 2 * z * z, 2 * x * y - 2 * w * z, 2 * w * y + 2 * x * z,
                        2 * x * y + 2 * w * z, 1 - 2 * x * x - 2 * z * z, 2 * y * z - 2 * w * x,
                        2 * x * z - 2 * w * y, 2 * w * x + 2 * y * z, 1 - 2 * x * x - 2 * y * y],
                       dim=-1).reshape(-1, 3, 3)


def densify(params, moments, accum, denom, max_grad, extent, percent_dense, z, N=2):
    """``params``: dict name -> [P, ...] with ``xyz, scaling, rotation`` among the names; ``moments``: dict name ->
    (exp_avg, exp_avg_sq); ``z``: standard-normal draws, one row of (at least) two per split child.
    Returns (new params, new moments, n_clone, n_split)."""
    grads = accum / denom
    grads[grads.isnan()] = 0.0
    grads = grads.reshape(-1)
    thr = percent_dense * extent
    big = params["scaling"].exp().amax(dim=1)
    clone = (grads >= max_grad) & (big <= thr)
    P = grads.shape[0]
    cur = {k: torch.cat([v, v[clone]]) for k, v in params.items()}
    mom = {k: tuple(torch.cat([m, torch.zeros_like(params[k][clone])]) for m in moments[k]) for k in moments}
    n_clone = int(clone.sum())
    padded = torch.zeros(P + n_clone)
    padded[:P] = grads
    split = (padded >= max_grad) & (cur["scaling"].exp().amax(dim=1) > thr)
    n_split = int(split.sum())
    stds = cur["scaling"].exp()[split].repeat(N, 1)
    stds = torch.cat([stds, torch.zeros_like(stds[:, :1])], dim=-1)
    samples = stds * torch.cat([z[:stds.shape[0], :2], torch.zeros(stds.shape[0], 1)], dim=-1)
    rots = quat_to_matrix(cur["rotation"][split]).repeat(N, 1, 1)
    new = {k: v[split].repeat(N, *[1] * (v.dim() - 1)) for k, v in cur.items()}
    new["xyz"] = torch.bmm(rots, samples[..., None]).squeeze(-1) + cur["xyz"][split].repeat(N, 1)
    new["scaling"] = torch.log(cur["scaling"].exp()[split].repeat(N, 1) / (0.8 * N))
    keep = torch.cat([~split, torch.ones(N * n_split, dtype=torch.bool)])
    out = {k: torch.cat([cur[k], new[k]])[keep] for k in cur}
    out_m = {k: tuple(torch.cat([m, torch.zeros_like(new[k])])[keep] for m in mom[k]) for k in mom}
    return out, out_m, n_clone, n_split
