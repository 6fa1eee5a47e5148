"""CPU restatement of the reference's feature activation (test infrastructure only).

Numpy, float32 throughout, following utils/model_util.py:93-105 (activate_output),
:81-91 (offset_normalize), :63-79 (compute_vertex_colors_from_field), :10-12 (RGB2SH),
utils/eval_sh_py.py:121-179 (eval_sh) and utils/safe_math.py:146-158 (safe_div forward).
Pinned by tests against tests/golden/activate_output.npz, which holds outputs of the
reference's own function run on CPU.  Only tests, the smoke check and the benchmark's
checker may import this module; the product path never does.
"""
import numpy as np

C0 = np.float32(0.28209479177387814)
C1 = np.float32(0.4886025119029199)
C2 = [np.float32(v) for v in (1.0925484305920792, -1.0925484305920792, 0.31539156525252005, -1.0925484305920792,
                               0.5462742152960396)]
C3 = [np.float32(v) for v in (-0.5900435899266435, 2.890611442640554, -0.4570457994644658, 0.3731763325901154,
                               -0.4570457994644658, 1.445305721320277, -0.5900435899266435)]
C4 = [np.float32(v) for v in (2.5033429417967046, -1.7701307697799304, 0.9461746957575601, -0.6690465435572892,
                               0.10578554691520431, -0.6690465435572892, 0.47308734787878004, -1.7701307697799304,
                               0.6258357354491761)]


def safe_div(n, d):
    """utils/safe_math.py:146-158: clamp(n / d) to the finite float range, 0 where |d| is denormal."""
    tiny, big = np.float32(1.17549435e-38), np.float32(3.40282347e+38)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        r = np.clip(n / np.where(np.abs(d) < tiny, np.float32(1), d), -big, big)
    return np.where(np.abs(d) < tiny, np.float32(0), r).astype(np.float32)


def eval_sh(means, sh0, sh_rest, camera_center, deg):
    """utils/eval_sh_py.py:121-179; sh_rest [T,K,3] may be float16 (promoted to float32 per term)."""
    f = np.float32
    dirs = (means - camera_center.reshape(1, 3)).astype(f)
    nrm = np.maximum(np.sqrt((dirs * dirs).sum(-1, keepdims=True, dtype=f)), f(1e-8))
    dirs = dirs / nrm
    res = C0 * sh0 + f(0.5)
    if deg > 0:
        x, y, z = dirs[:, 0:1], dirs[:, 1:2], dirs[:, 2:3]
        s = lambda k: sh_rest[:, k, :].astype(f)
        res = res - C1 * y * s(0) + C1 * z * s(1) - C1 * x * s(2)
        if deg > 1:
            xx, yy, zz, xy, yz, xz = x * x, y * y, z * z, x * y, y * z, x * z
            res = (res + C2[0] * xy * s(3) + C2[1] * yz * s(4) + C2[2] * (f(2) * zz - xx - yy) * s(5)
                   + C2[3] * xz * s(6) + C2[4] * (xx - yy) * s(7))
            if deg > 2:
                res = (res + C3[0] * y * (f(3) * xx - yy) * s(8) + C3[1] * xy * z * s(9)
                       + C3[2] * y * (f(4) * zz - xx - yy) * s(10)
                       + C3[3] * z * (f(2) * zz - f(3) * xx - f(3) * yy) * s(11)
                       + C3[4] * x * (f(4) * zz - xx - yy) * s(12) + C3[5] * z * (xx - yy) * s(13)
                       + C3[6] * x * (xx - f(3) * yy) * s(14))
                if deg > 3:
                    res = (res + C4[0] * xy * (xx - yy) * s(15) + C4[1] * yz * (f(3) * xx - yy) * s(16)
                           + C4[2] * xy * (f(7) * zz - f(1)) * s(17) + C4[3] * yz * (f(7) * zz - f(3)) * s(18)
                           + C4[4] * (zz * (f(35) * zz - f(30)) + f(3)) * s(19)
                           + C4[5] * xz * (f(7) * zz - f(3)) * s(20) + C4[6] * (xx - yy) * (f(7) * zz - f(1)) * s(21)
                           + C4[7] * xz * (xx - f(3) * yy) * s(22)
                           + C4[8] * (xx * (xx - f(3) * yy) - yy * (f(3) * xx - yy)) * s(23))
    return res.astype(f)


def softplus(x, beta=10.0):
    """torch.nn.functional.softplus: linear where beta * x > 20."""
    b = np.float32(beta)
    with np.errstate(over="ignore"):
        soft = np.log1p(np.exp(np.minimum(b * x, np.float32(30)))) / b
    return np.where(b * x > np.float32(20), x, soft).astype(np.float32)


def activate_output(camera_center, density, rgb, grd, sh, indices, circumcenters, vertices, current_sh_deg):
    f = np.float32
    tets = vertices[indices].astype(f)                                   # [T,4,3]
    rgb = rgb.reshape(-1, 3).astype(f)
    g = grd.reshape(-1, 3).astype(f) * rgb.min(axis=1, keepdims=True)     # offset_normalize
    r0 = tets[:, 0] - circumcenters.astype(f)
    radius = np.sqrt((r0 * r0).sum(-1, keepdims=True, dtype=f))
    normed = safe_div(g, radius)
    base_v0 = rgb + (normed * r0).sum(-1, keepdims=True, dtype=f)         # vertex-0 colour of the linear field
    sh0 = (base_v0 - f(0.5)) / C0                                         # RGB2SH
    raw = eval_sh(tets.mean(axis=1, dtype=f), sh0, sh.reshape(len(indices), -1, 3), camera_center.astype(f),
                  current_sh_deg)
    return np.concatenate([density.reshape(-1, 1).astype(f), softplus(raw), normed], axis=1).astype(f)
