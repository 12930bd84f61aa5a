"""Helpers of the Zelunex tests: write a model folder (config.json + model.safetensors) from a weight dict."""
import json
import struct

import numpy as np
import torch


def write_model_dir(path, cfg: dict, W: dict):
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    header, blobs, off = {}, [], 0
    for name, a in W.items():
        raw = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    return path


def device_tensors(W: dict, matrices_dtype=torch.bfloat16):
    out = {}
    for name, a in W.items():
        t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
        out[name] = t.to(matrices_dtype) if t.dim() == 2 else t
    return out


def rel_rms(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    a = a - a.mean(-1, keepdims=True)
    b = b - b.mean(-1, keepdims=True)
    return float(np.sqrt(((a - b) ** 2).mean(-1)).max() / max(np.sqrt((b ** 2).mean()), 1e-30))
