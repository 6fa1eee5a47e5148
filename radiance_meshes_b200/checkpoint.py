"""Frozen-model checkpoints: the on-disk format that feeds the rendering path.

The reference writes `ckpt.pth` (train.py:364-368: the model's state dict plus
`indices` and `empty_indices`) next to `config.json` (utils/args.py), and loads it
for rendering with FrozenTetModel.load_ckpt (models/frozen.py:86-148).  FrozenScene
reads the same two files and exposes what the rasterizer needs: the vertex and
index tensors, per-tet circumcentres, and per-camera cell values through the fused
activate_output kernel (models/frozen.py:198-222, tile_benchmark.py:53-67).
Loading is host-side plumbing in torch; nothing here sits on the timed path.
"""
import json
from pathlib import Path

import torch

REQUIRED_KEYS = ("interior_vertices", "ext_vertices", "indices", "density", "rgb", "gradient", "sh", "center",
                 "scene_scaling")


def circumcenters_f64(vertices, indices):
    """Per-tet circumcentres in float64, as pre_calc_cell_values does (utils/model_util.py:25-30 with
    utils/topo_utils.py:120-163): c = v0 + (|a|^2 (b x c) + |b|^2 (c x a) + |c|^2 (a x b)) / (2 a . (b x c)),
    the quotient through safe_div (0 where the denominator is denormal)."""
    t = vertices[indices.long()].double()
    a, b, c = t[:, 1] - t[:, 0], t[:, 2] - t[:, 0], t[:, 3] - t[:, 0]
    aa, bb, cc = (a * a).sum(-1, keepdim=True), (b * b).sum(-1, keepdim=True), (c * c).sum(-1, keepdim=True)
    bc, ca, ab = torch.cross(b, c, dim=-1), torch.cross(c, a, dim=-1), torch.cross(a, b, dim=-1)
    den = 2.0 * (a * bc).sum(-1, keepdim=True)
    num = aa * bc + bb * ca + cc * ab
    tiny = torch.finfo(torch.float32).tiny
    rel = torch.where(den.abs() < tiny, torch.zeros_like(num),
                      (num / torch.where(den.abs() < tiny, torch.ones_like(den), den)).clamp(-3.4028235e38,
                                                                                            3.4028235e38))
    return (t[:, 0] + rel).float()


class FrozenScene:
    """The tensors of a frozen tet model, on one device."""

    def __init__(self, interior_vertices, ext_vertices, indices, density, rgb, gradient, sh, center, scene_scaling,
                 density_offset=-1.0, max_sh_deg=2, base_min_t=None, device="cuda"):
        dev = torch.device(device)
        self.device = dev
        self.interior_vertices = interior_vertices.to(dev).float()
        self.ext_vertices = ext_vertices.to(dev).float()
        self.indices = indices.to(dev).int().contiguous()
        T = self.indices.shape[0]
        self.density = density.to(dev).float().reshape(T, 1)
        self.rgb = rgb.to(dev).float().reshape(T, 3)
        self.gradient = gradient.to(dev).float().reshape(T, 3)
        self.max_sh_deg = int(max_sh_deg)
        self.sh = sh.to(dev).half().reshape(T, (self.max_sh_deg + 1) ** 2 - 1, 3).contiguous()  # stored as half
        self.center = center.to(dev).reshape(1, 3)
        self.scene_scaling = torch.as_tensor(scene_scaling).to(dev)
        self.density_offset = float(density_offset)
        self.min_t = float(self.scene_scaling) * float(base_min_t) if base_min_t is not None else None
        self.vertices = torch.cat([self.interior_vertices, self.ext_vertices], dim=0).contiguous()
        if T and int(self.indices.max()) >= self.vertices.shape[0]:
            raise ValueError("checkpoint indices refer to vertices that are not in the checkpoint")
        self.circumcenters = circumcenters_f64(self.vertices, self.indices)

    @staticmethod
    def load_ckpt(path, device="cuda"):
        """`path`: directory holding ckpt.pth and config.json (models/frozen.py:86-148)."""
        path = Path(path)
        with open(path / "config.json", "r", encoding="utf-8") as f:
            config = json.load(f)
        ckpt = torch.load(path / "ckpt.pth", map_location="cpu", weights_only=True)
        missing = [k for k in REQUIRED_KEYS if k not in ckpt]
        if missing:
            raise KeyError(f"{path / 'ckpt.pth'} is not a frozen-model checkpoint: missing {missing}")
        return FrozenScene(ckpt["interior_vertices"], ckpt["ext_vertices"], ckpt["indices"], ckpt["density"],
                           ckpt["rgb"], ckpt["gradient"], ckpt["sh"], ckpt["center"], ckpt["scene_scaling"],
                           density_offset=config.get("density_offset", -1.0), max_sh_deg=config.get("max_sh_deg", 2),
                           base_min_t=config.get("base_min_t"), device=device)

    def save_ckpt(self, path, extra_config=None):
        """Writes ckpt.pth + config.json with the keys the reference writes (train.py:364-368)."""
        path = Path(path)
        path.mkdir(parents=True, exist_ok=True)
        sd = dict(interior_vertices=self.interior_vertices.cpu(), ext_vertices=self.ext_vertices.cpu(),
                  indices=self.indices.cpu(), empty_indices=torch.empty((0, 4), dtype=torch.int32),
                  density=self.density.cpu(), rgb=self.rgb.cpu(), gradient=self.gradient.cpu().reshape(-1, 1, 3),
                  sh=self.sh.cpu(), center=self.center.cpu(), scene_scaling=self.scene_scaling.cpu())
        torch.save(sd, path / "ckpt.pth")
        config = dict(density_offset=self.density_offset, max_sh_deg=self.max_sh_deg)
        if self.min_t is not None:
            config["base_min_t"] = self.min_t / float(self.scene_scaling)
        config.update(extra_config or {})
        with open(path / "config.json", "w", encoding="utf-8") as f:
            json.dump(config, f)

    def get_cell_values(self, camera_center):
        """[T,7] cell values for a camera position (models/frozen.py:198-222), by the fused kernel."""
        from .activate import activate_output
        with torch.no_grad():
            return activate_output(camera_center, self.density, self.rgb, self.gradient, self.sh, self.indices,
                                   self.circumcenters, self.vertices, self.max_sh_deg, self.max_sh_deg)


# ---------------------------------------------------------------------------
# ckpt.ply: the mesh export of models/base_model.py:107-151 (save2ply)
# ---------------------------------------------------------------------------
# The reference writes it through the un-vendored `tinyplypy` package and holds no reader for it
# in its tree, so the byte-level header of its files cannot be checked here.  The layout below is
# the standard binary little-endian PLY with the element and property names save2ply uses:
#   element vertex:       x y z (float32)
#   element tetrahedron:  indices (list of 4 int32), s (density), grd_x grd_y grd_z,
#                         sh_0_r sh_0_g sh_0_b (degree-0 SH = (rgb - 0.5) / C0), sh_i_r sh_i_g sh_i_b
SH_C0 = 0.28209479177387814


def write_ply(path, vertices, indices, density, grd, rgb, sh_rest):
    """vertices[V,3] f32, indices[T,4] i32, density[T], grd[T,3], rgb[T,3] (base colour at vertex 0,
    before activation), sh_rest[T,K,3]."""
    import numpy as np
    v = np.ascontiguousarray(np.asarray(vertices, np.float32))
    idx = np.ascontiguousarray(np.asarray(indices, np.int32))
    T, K = idx.shape[0], int(np.asarray(sh_rest).shape[1])
    names = ["s", "grd_x", "grd_y", "grd_z", "sh_0_r", "sh_0_g", "sh_0_b"]
    names += [f"sh_{i + 1}_{c}" for i in range(K) for c in "rgb"]
    cols = np.concatenate([np.asarray(density, np.float32).reshape(T, 1), np.asarray(grd, np.float32).reshape(T, 3),
                           (np.asarray(rgb, np.float32).reshape(T, 3) - 0.5) / SH_C0,
                           np.asarray(sh_rest, np.float32).reshape(T, 3 * K)], axis=1).astype("<f4")
    rec = np.zeros(T, dtype=[("n", "u1"), ("idx", "<i4", (4,)), ("f", "<f4", (cols.shape[1],))])
    rec["n"], rec["idx"], rec["f"] = 4, idx, cols
    header = ["ply", "format binary_little_endian 1.0", f"element vertex {v.shape[0]}", "property float x",
              "property float y", "property float z", f"element tetrahedron {T}", "property list uchar int indices"]
    header += [f"property float {n}" for n in names] + ["end_header"]
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "wb") as f:
        f.write(("\n".join(header) + "\n").encode("ascii"))
        f.write(v.astype("<f4").tobytes())
        f.write(rec.tobytes())


def read_ply(path):
    """Inverse of write_ply.  Returns dict(vertices, indices, density, grd, rgb, sh_rest) as NumPy arrays."""
    import numpy as np
    with open(path, "rb") as f:
        data = f.read()
    end = data.index(b"end_header\n") + len(b"end_header\n")
    lines = data[:end].decode("ascii").split("\n")
    if lines[0] != "ply" or "binary_little_endian" not in lines[1]:
        raise ValueError(f"{path}: not a binary little-endian PLY file")
    counts, props, cur = {}, {}, None
    for ln in lines[2:]:
        parts = ln.split()
        if parts[:1] == ["element"]:
            cur = parts[1]
            counts[cur] = int(parts[2])
            props[cur] = []
        elif parts[:1] == ["property"]:
            props[cur].append(parts[1:])
    if [p[-1] for p in props.get("vertex", [])] != ["x", "y", "z"] or "tetrahedron" not in props:
        raise ValueError(f"{path}: expected elements `vertex` (x y z) and `tetrahedron`")
    tp = props["tetrahedron"]
    if tp[0] != ["list", "uchar", "int", "indices"] or any(p[0] != "float" for p in tp[1:]):
        raise ValueError(f"{path}: unexpected tetrahedron properties")
    names = [p[1] for p in tp[1:]]
    V, T = counts["vertex"], counts["tetrahedron"]
    v = np.frombuffer(data, "<f4", 3 * V, end).reshape(V, 3)
    rec = np.frombuffer(data, np.dtype([("n", "u1"), ("idx", "<i4", (4,)), ("f", "<f4", (len(names),))]), T,
                        end + 12 * V)
    if T and not (rec["n"] == 4).all():
        raise ValueError(f"{path}: a tetrahedron does not have 4 indices")
    col = {n: rec["f"][:, i] for i, n in enumerate(names)}
    K = (len(names) - 7) // 3
    sh_rest = np.stack([np.stack([col[f"sh_{i + 1}_{c}"] for c in "rgb"], -1) for i in range(K)], 1) if K else \
        np.zeros((T, 0, 3), np.float32)
    return dict(vertices=v.copy(), indices=rec["idx"].copy(), density=col["s"].copy(),
                grd=np.stack([col["grd_x"], col["grd_y"], col["grd_z"]], -1),
                rgb=np.stack([col["sh_0_r"], col["sh_0_g"], col["sh_0_b"]], -1) * SH_C0 + 0.5, sh_rest=sh_rest)
