"""Host-side pieces of the Zelunex family that need no GPU: the oracle's own mechanisms, the JSON / safetensors readers and the
family registry's validation of a model folder."""
import ctypes as C
import json

import numpy as np
import pytest

import zelunex_oracle as O
from zelunex_util import write_model_dir

from ntransformer_b200._lib import lib


def describe(path):
    buf = C.create_string_buffer(1 << 16)
    rc = lib().nt_model_dir_describe(str(path).encode(), buf, len(buf))
    return rc, buf.value.decode()


def test_oracle_mask_and_softcap():
    assert O.visible(10, 10, 4, 2) and O.visible(10, 7, 4, 2) and not O.visible(10, 6, 4, 2)
    assert O.visible(10, 1, 4, 2) and not O.visible(10, 2, 4, 2) and not O.visible(3, 4, 4, 2)
    assert abs(O.softcap(1000.0, 20.0) - 20.0) < 1e-9 and abs(O.softcap(0.01, 20.0) - 0.01) < 1e-6
    x = np.array([[3.0, 4.0]])
    np.testing.assert_allclose(O.rms_norm(x, np.ones(2), 0.0), x / np.sqrt(12.5))


def test_oracle_prefix_invariance():
    rng = np.random.default_rng(5)
    cfg, W = O.random_model(rng, n_layers=2, window=5, keep=2)
    toks = rng.integers(0, cfg["vocab"], 20)
    full = O.forward(cfg, W, toks)
    np.testing.assert_allclose(O.forward(cfg, W, toks[:11]), full[:11], rtol=1e-9, atol=1e-9)


def test_model_folder_is_validated(tmp_path):
    rng = np.random.default_rng(1)
    cfg, W = O.random_model(rng, n_layers=3, share={2: 0}, no_mlp=(1,), heads=6, kv_heads=3, dim=16, vdim=8)
    d = write_model_dir(tmp_path / "ok", cfg, W)
    rc, text = describe(d)
    assert rc == 0, text
    assert "architecture=Zelunex" in text and "layers=3" in text and "weights_of=0" in text and "heads=6 kv=3 dim=16 vdim=8" in text
    assert "layer 1:" in text and "ff=0" in text.split("layer 1:")[1].split("\n")[0]
    # a tensor of the wrong shape, a missing tensor, an unknown architecture, a sharing cycle
    W2 = dict(W); W2["l0.mix.k"] = W["l0.mix.k"][:-1]
    assert describe(write_model_dir(tmp_path / "shape", cfg, W2))[0] == -1
    W3 = dict(W); del W3["l1.ls1"]
    rc, text = describe(write_model_dir(tmp_path / "missing", cfg, W3))
    assert rc == -1 and "l1.ls1" in text
    bad = json.loads(json.dumps(cfg)); bad["architecture"] = "Nope"
    assert describe(write_model_dir(tmp_path / "arch", bad, W))[0] == -1
    bad = json.loads(json.dumps(cfg)); bad["layers"][1]["weights_of"] = 2
    assert describe(write_model_dir(tmp_path / "cycle", bad, W))[0] == -1
    bad = json.loads(json.dumps(cfg)); del bad["layers"][0]["mixer"]["softcap"]
    assert describe(write_model_dir(tmp_path / "nokey", bad, W))[0] == -1
    (tmp_path / "trunc").mkdir()
    (tmp_path / "trunc" / "config.json").write_text(json.dumps(cfg))
    (tmp_path / "trunc" / "model.safetensors").write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    assert describe(tmp_path / "trunc")[0] == -1
