"""Split a camera dictionary into tensors (saved for backward) and plain values,
and put it back together (mirrors delaunay_rasterization/internal/util.py:3-23)."""
import torch


def split_tensors(tcam):
    keys = [k for k, v in tcam.items() if isinstance(v, torch.Tensor)]
    plain = {k: v for k, v in tcam.items() if not isinstance(v, torch.Tensor)}
    plain["_tensor_keys"] = keys
    return plain, [tcam[k] for k in keys]


def recombine_tensors(non_tensor_data, tensor_data):
    keys = non_tensor_data.pop("_tensor_keys")
    out = dict(zip(keys, tensor_data))
    out.update(non_tensor_data)
    return out
