"""CPU-only checks: the C ABI library loads and exports every declared symbol, headers and bindings agree,
synthetic workloads are reproducible, and the oracle's k-NN / Adam restatements hold against plain torch."""
import ctypes
import os
import re
import sys

import pytest
import torch

import oracle as orc
from conftest import ROOT


def test_library_exports_every_declared_symbol():
    from fsgs import _lib
    from fsgs.build import LIB, build
    build()
    handle = ctypes.CDLL(LIB)
    header = open(os.path.join(ROOT, "include", "fsgs.h")).read()
    declared = set(re.findall(r"\b(fsgs_[a-z0-9_]+)\s*\(", header))
    declared -= {"fsgs_status"}
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(handle, name), f"{name} declared in include/fsgs.h but not exported"
    assert declared == set(_lib.SYMBOLS), "python binding table and header disagree"
    _lib.lib()
    assert _lib.lib().fsgs_version() >= 100
    assert _lib.lib().fsgs_status_string(-3) == b"workspace too small"


def test_ctypes_structs_match_header_field_order():
    from fsgs import _lib
    header = open(os.path.join(ROOT, "include", "fsgs.h")).read()
    for cname, cls in (("fsgs_preprocess_args", _lib.PreprocessArgs), ("fsgs_bin_args", _lib.BinArgs),
                       ("fsgs_render_args", _lib.RenderArgs), ("fsgs_render_bwd_args", _lib.RenderBwdArgs),
                       ("fsgs_preprocess_bwd_args", _lib.PreprocessBwdArgs), ("fsgs_lbs", _lib.LBS),
                       ("fsgs_lbs_grads", _lib.LBSGrads), ("fsgs_adam_tensor", _lib.AdamTensor),
                       ("fsgs_view_args", _lib.ViewArgs)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), header, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = re.sub(r"^(const\s+)?[A-Za-z_0-9]+\s*", "", decl)
            fields += [n.strip().lstrip("*").strip() for n in names.split(",")]
        assert fields == [f[0] for f in cls._fields_], cname


def test_operators_refuse_cpu_tensors():
    from fsgs import ops
    with pytest.raises(RuntimeError):
        ops.cdist_top(torch.zeros(4, 3), torch.zeros(2, 3))
    with pytest.raises(RuntimeError):
        ops.AdamMasksedUpdated(torch.zeros(4, 3), torch.zeros(4, 3), torch.zeros(4, 3), torch.zeros(4, 3),
                               torch.ones(4, dtype=torch.bool), 1e-3, 0.9, 0.999, 1e-8, 4, 3)


def test_workloads_are_reproducible_and_shaped():
    from fsgs import workloads as wl
    a, b = wl.surfels(1000, seed=3), wl.surfels(1000, seed=3)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert a["sh_rest"].shape == (1000, 15, 3) and a["scales"].shape == (1000, 2)
    assert torch.allclose(a["rots"].norm(dim=-1), torch.ones(1000), atol=1e-6)
    cam = wl.camera(800, 800)
    assert torch.allclose(cam["Tw2v"][:3, 3], torch.tensor([0.0, 0.0, 4.0]))  # looks at the origin: no x/y translation
    assert abs(float(cam["Tv2s"][0, 0]) - 0.5 * 800 / torch.tan(torch.tensor(0.345)).item()) < 1e-2
    x, c = wl.knn_points_c1(2000, 64, seed=0)
    assert x.shape == (2000, 3) and c.shape == (64, 3) and float(x.abs().max()) <= 1.0


def test_oracle_knn_against_torch():
    from fsgs import workloads as wl
    x, c = wl.knn_points_c1(3000, 100, seed=1)
    d2, idx = orc.knn(x, c, 3)
    full = ((x[:, None, :] - c[None]) ** 2).sum(-1)
    ref_d, ref_i = torch.topk(full, 3, dim=-1, largest=False)
    assert torch.allclose(d2, ref_d, rtol=1e-5, atol=1e-7)
    assert float((idx == ref_i).float().mean()) > 0.999  # torch breaks near-ties its own way
    dist, i1 = orc.cdist_top(x, c)
    assert torch.equal(i1, idx[:, 0]) and torch.allclose(dist, d2[:, 0].sqrt())


def test_oracle_adam_against_torch():
    g = torch.Generator().manual_seed(0)
    N, M = 100, 5
    p, gr = torch.randn(N, M, generator=g), torch.randn(N, M, generator=g)
    m, v = torch.zeros(N, M), torch.zeros(N, M)
    vis = torch.rand(N, generator=g) > 0.5
    p0 = p.clone()
    orc.adam(p, gr, m, v, vis, 1e-2, 0.9, 0.999, 1e-8, N, M)
    m_ref = 0.1 * gr
    v_ref = 0.001 * gr * gr
    p_ref = p0 - 1e-2 * m_ref / (v_ref.sqrt() + 1e-8)
    assert torch.allclose(p[vis], p_ref[vis], rtol=1e-5, atol=1e-6) and torch.equal(p[~vis], p0[~vis])
    assert torch.allclose(m[vis], m_ref[vis], rtol=1e-5, atol=1e-8) and bool((m[~vis] == 0).all())


def test_dense_adam_rewrite_of_the_bias_corrected_update():
    """``DenseAdam`` feeds torch's bias-corrected Adam to a kernel that computes ``p -= lr' m / (sqrt(v) + eps')``: with
    ``lr' = lr sqrt(1 - b2^t) / (1 - b1^t)`` and ``eps' = eps sqrt(1 - b2^t)`` the two are the same update.  Checked
    here on the CPU with the oracle's masked Adam (one row per tensor behind a one-element gate) against
    ``torch.optim.Adam`` over six steps, and a closed gate leaves everything alone."""
    g = torch.Generator().manual_seed(3)
    lr, eps, b1, b2 = 3e-3, 1e-8, 0.9, 0.999
    p = torch.randn(1, 77, generator=g)
    q = torch.nn.Parameter(p.clone())
    ref = torch.optim.Adam([q], lr=lr, eps=eps, betas=(b1, b2))
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    gate = torch.ones(1, dtype=torch.bool)
    for t in range(1, 7):
        grad = torch.randn(1, 77, generator=g) * 10.0 ** (t - 3)
        q.grad = grad.clone()
        ref.step()
        root = (1.0 - b2 ** t) ** 0.5
        orc.adam(p, grad, m, v, gate, lr * root / (1.0 - b1 ** t), b1, b2, eps * root, 1, 77)
        assert torch.allclose(p, q.detach(), rtol=2e-5, atol=1e-7), t
        assert torch.allclose(m, ref.state[q]["exp_avg"], rtol=1e-5, atol=1e-9)
        assert torch.allclose(v, ref.state[q]["exp_avg_sq"], rtol=3e-5, atol=1e-12)
    before = (p.clone(), m.clone(), v.clone())
    orc.adam(p, torch.ones(1, 77), m, v, torch.zeros(1, dtype=torch.bool), 1.0, b1, b2, eps, 1, 77)
    assert torch.equal(p, before[0]) and torch.equal(m, before[1]) and torch.equal(v, before[2])


def test_generated_sh_polynomials_match_the_golden_basis_and_their_generator(tmp_path):
    """csrc/fsgs_sh_high.h (degrees 4..7 as Cartesian polynomials) is plain C: compile it for the host, compare the
    bands with the reference's general definition (golden fixture) and the adjoint with central differences."""
    import ctypes
    import subprocess
    import numpy as np
    from util import load_golden
    csrc = os.path.join(ROOT, "fast-sp-gs_b200", "csrc")
    src = tmp_path / "sh.c"
    src.write_text('#include "fsgs_sh_high.h"\n' + "".join(
        f"void band{l}(float x, float y, float z, float *b) {{ fsgs_sh_band{l}(x, y, z, b); }}\n"
        f"void adj{l}(float x, float y, float z, const float *t, float *g) "
        f"{{ fsgs_sh_band{l}_adjoint(x, y, z, t, g, g + 1, g + 2); }}\n" for l in range(4, 8)))
    so = tmp_path / "sh.so"
    subprocess.check_call(["gcc", "-O1", "-std=c99", "-ffp-contract=off", "-shared", "-fPIC", "-I", csrc, str(src),
                           "-o", str(so)])
    lib = ctypes.CDLL(str(so))
    g = load_golden("sh_basis_deg7.npz")
    dirs, Y = g["dirs"].numpy(), g["Y"].numpy()
    f = ctypes.c_float
    rng = np.random.default_rng(0)
    for l in range(4, 8):
        n = 2 * l + 1
        band, adj = getattr(lib, f"band{l}"), getattr(lib, f"adj{l}")
        for i in range(dirs.shape[0]):
            b = (f * n)()
            band(f(dirs[i, 0]), f(dirs[i, 1]), f(dirs[i, 2]), b)
            assert np.abs(np.array(b) - Y[i, l * l:l * l + n]).max() < 2e-6, (l, i)
        # adjoint = gradient of sum_m t_m Y_l^m, the three variables taken as independent
        t = rng.standard_normal(n).astype(np.float32)
        x0 = dirs[0].astype(np.float64)

        def value(p):
            b = (f * n)()
            band(f(p[0]), f(p[1]), f(p[2]), b)
            return float(np.dot(np.array(b, dtype=np.float64), t))

        grad = (f * 3)(0, 0, 0)
        adj(f(x0[0]), f(x0[1]), f(x0[2]), (f * n)(*t), grad)
        h = 1e-2
        fd = [(value(x0 + h * e) - value(x0 - h * e)) / (2 * h) for e in np.eye(3)]
        assert np.abs(np.array(grad) - np.array(fd)).max() < 2e-2 * max(1.0, np.abs(fd).max()), (l, list(grad), fd)
    # the committed header is what the generator prints
    out = subprocess.check_output([sys.executable, os.path.join(csrc, "gen_sh_high.py")], text=True)
    assert out == open(os.path.join(csrc, "fsgs_sh_high.h")).read()


def test_lbs_weight_forms():
    """The three weightings of the reference's calc_LBS_weight (network.py:506-518), element by element."""
    import math
    from fsgs.scene import lbs_weights
    g = torch.Generator().manual_seed(3)
    N, K, M = 50, 3, 7
    d2 = torch.rand(N, K, generator=g)
    idx = torch.randint(0, M, (N, K), generator=g)
    radius, weight, table = torch.rand(M, generator=g) + 0.2, torch.rand(M, generator=g), torch.randn(N, M, generator=g)
    w_dist = lbs_weights(d2, idx, "dist", temperature=0.5)
    w_kern = lbs_weights(d2, idx, "kernel", radius=radius, weight=weight)
    w_tab = lbs_weights(d2, idx, "table", table=table)
    for n in (0, 17, 49):
        e = [math.exp(-float(d2[n, k]) / 0.5) for k in range(K)]
        assert all(abs(float(w_dist[n, k]) - e[k] / sum(e)) < 1e-6 for k in range(K))
        e = [math.exp(-float(d2[n, k]) / (2 * float(radius[idx[n, k]]) ** 2)) * float(weight[idx[n, k]]) + 1e-7
             for k in range(K)]
        assert all(abs(float(w_kern[n, k]) - e[k] / sum(e)) < 1e-6 for k in range(K))
        e = [math.exp(float(table[n, idx[n, k]])) for k in range(K)]
        assert all(abs(float(w_tab[n, k]) - e[k] / sum(e)) < 1e-6 for k in range(K))
    with pytest.raises(ValueError):
        lbs_weights(d2, idx, "nearest")


def test_pairs_grouped_by_superpoint():
    from fsgs.renderer import group_pairs_by_superpoint
    g = torch.Generator().manual_seed(4)
    P, K, M = 500, 3, 17
    idx = torch.randint(0, M, (P, K), generator=g)
    offsets, pairs = group_pairs_by_superpoint(idx, M)
    assert offsets.dtype == torch.int32 and pairs.dtype == torch.int32 and offsets.shape == (M + 1,)
    assert int(offsets[0]) == 0 and int(offsets[-1]) == P * K
    flat = idx.reshape(-1)
    assert sorted(pairs.tolist()) == list(range(P * K))                 # a permutation of all pairs
    for m in range(M):
        run = pairs[int(offsets[m]):int(offsets[m + 1])].long()
        assert bool((flat[run] == m).all())                             # each run holds one superpoint's pairs
        assert run.tolist() == sorted(run.tolist())                     # in ascending pair order (stable)
