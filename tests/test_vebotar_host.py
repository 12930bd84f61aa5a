"""Host-side pieces of the Vebotar family that need no GPU: the oracle's own mechanisms, the rotary frequency table and the
family registry's validation of a model folder."""
import ctypes as C
import json
import math

import numpy as np

import vebotar_oracle as O
from zelunex_util import write_model_dir

from ntransformer_b200._lib import lib


def describe(path):
    buf = C.create_string_buffer(1 << 16)
    rc = lib().nt_model_dir_describe(str(path).encode(), buf, len(buf))
    return rc, buf.value.decode()


def test_oracle_mask_routing_and_rotation():
    assert O.visible(13, 7, 7) and not O.visible(13, 6, 7) and O.visible(6, 0, 7) and not O.visible(7, 6, 7) and not O.visible(3, 4, 7)
    ids, ws = O.route(np.array([1.0, 0.0]), np.array([[0.5, 0], [2.0, 0], [2.0, 0], [-1.0, 0]]), 2)
    assert list(ids) == [1, 2] and abs(ws.sum() - 1) < 1e-12 and abs(ws[0] - 0.5) < 1e-12          # ties: the lower index first
    x = np.arange(6.0)
    r = O.rotate(x, 5, {"dims": 4, "base": 100.0})
    assert np.allclose(r[4:], x[4:]) and abs(np.hypot(r[0], r[1]) - np.hypot(x[0], x[1])) < 1e-12      # the tail passes, pairs keep their length
    a = 5 * 100.0 ** (-2 / 4)
    assert np.allclose(r[2:4], [x[2] * math.cos(a) - x[3] * math.sin(a), x[3] * math.cos(a) + x[2] * math.sin(a)])
    np.testing.assert_allclose(O.expert(np.array([1.0, -1.0]), np.array([[2.0, 0.0], [0.0, 3.0]]), np.array([[1.0, 1.0]])), [4.0])


def test_oracle_prefix_invariance_and_block_isolation():
    rng = np.random.default_rng(5)
    cfg, W = O.random_model(rng, n_layers=2, chunk=6, kv_from={1: 0})
    toks = rng.integers(0, cfg["vocab"], 20)
    full = O.forward(cfg, W, toks)
    np.testing.assert_allclose(O.forward(cfg, W, toks[:11]), full[:11], rtol=1e-9, atol=1e-9)
    other = toks.copy(); other[:12] = rng.integers(0, cfg["vocab"], 12)        # blocks 0 and 1 replaced: block 2 onward cannot notice
    np.testing.assert_allclose(O.forward(cfg, W, other)[12:], full[12:], rtol=1e-9, atol=1e-9)


def test_rotary_table_matches_the_oracle():
    for rot in ({"dims": 8, "base": 10000.0}, {"dims": 6, "base": 50.0, "scaling": {"factor": 3.0, "original": 24, "fast": 6.0, "slow": 1.5}},
                {"dims": 16, "base": 1e6, "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}},
                {"dims": 2, "base": 7.0, "scaling": {"factor": 2.0, "original": 4, "fast": 1.0, "slow": 1.0}}):
        f, mag = O.rotary_frequencies(rot)
        out = np.zeros(rot["dims"] // 2, dtype=np.float32)
        sc = rot.get("scaling") or {"factor": 0.0, "original": 0.0, "fast": 0.0, "slow": 0.0}
        got = lib().nt_b200_rotary_table(out.ctypes.data_as(C.c_void_p), rot["dims"], rot["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"])
        np.testing.assert_allclose(out, f, rtol=1e-6)
        assert abs(got - mag) < 1e-6


def test_model_folder_is_validated(tmp_path):
    rng = np.random.default_rng(1)
    cfg, W = O.random_model(rng, n_layers=3, kv_from={2: 0}, no_mlp=(1,), heads=6, kv_heads=3, dim=16, vdim=8, rot_dims=6)
    d = write_model_dir(tmp_path / "ok", cfg, W)
    rc, text = describe(d)
    assert rc == 0, text
    assert "architecture=Vebotar" in text and "layers=3" in text and "heads=6 kv=3 dim=16 vdim=8" in text
    l2 = text.split("layer 2:")[1].split("\n")[0]
    assert "kv_from=0" in l2 and "chunk=7" in l2 and "maps=2" in l2 and "rot=6" in l2 and "experts=5 top=2 shared_ff=14 streams=3" in l2
    assert "ff=0" in text.split("layer 1:")[1].split("\n")[0]
    W2 = dict(W); W2["l0.mix.k"] = W["l0.mix.k"][:-1]
    assert describe(write_model_dir(tmp_path / "shape", cfg, W2))[0] == -1
    W3 = dict(W); del W3["l0.mlp.e3.down"]
    rc, text = describe(write_model_dir(tmp_path / "missing", cfg, W3))
    assert rc == -1 and "l0.mlp.e3.down" in text
    W4 = dict(W); W4["l2.mix.k"] = W["l0.mix.k"]                                   # a layer that reads another's cache needs no key projection
    assert describe(write_model_dir(tmp_path / "extra", cfg, W4))[0] == 0
    for name, edit in {"fwd": lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 2),
                       "chain": lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 0) or c["layers"][2]["mixer"].__setitem__("kv_from", 1),
                       "top": lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 6),
                       "odd_rot": lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 5),
                       "kind": lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"),
                       "nodiff": lambda c: c["layers"][0]["mixer"].pop("diff")}.items():
        bad = json.loads(json.dumps(cfg)); edit(bad)
        assert describe(write_model_dir(tmp_path / name, bad, W))[0] == -1, name
