"""Vebotar on the GPU against the plain float64 oracle (tests/vebotar_oracle.py): each mechanism's kernel alone, then whole models
through the engine's step function — prompt pass vs token-by-token decoding, portions down to two tokens, cache rows reused, keys at
the edges of a mask block, shared caches, odd sizes, long decoding, and greedy generation through the engine's own entry point."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import vebotar_oracle as O
from vebotar_util import device_tensors
from zelunex_util import rel_rms, write_model_dir

from ntransformer_b200._lib import lib
from ntransformer_b200.dtypes import DType
from ntransformer_b200.engine import Engine, Model

pytestmark = pytest.mark.gpu


def dev(a, dt=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(dt).contiguous()


def stream():
    return torch.cuda.current_stream().cuda_stream


def table(rot):
    f = np.zeros(max(1, rot["dims"] // 2), dtype=np.float32)
    sc = rot.get("scaling") or {"factor": 0.0, "original": 0.0, "fast": 0.0, "slow": 0.0}
    mag = lib().nt_b200_rotary_table(f.ctypes.data_as(C.c_void_p), rot["dims"], rot["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"])
    return dev(f), mag


# ---------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("cache", [DType.F32, DType.BF16])
@pytest.mark.parametrize("rot", [{"dims": 4, "base": 50.0}, {"dims": 10, "base": 1e4, "scaling": {"factor": 3.0, "original": 24, "fast": 6.0, "slow": 1.5}},
                                 {"dims": 0, "base": 10.0}])
def test_partial_rotation_and_cache_write(cache, rot):
    rng = np.random.default_rng(rot["dims"])
    T, p0, dim, qh, kh, vd = 9, 37, 10, 6, 4, 14          # 6 query map-heads, 4 key map-heads
    q = rng.standard_normal((T, qh * dim)); k = rng.standard_normal((T, kh * dim)); v = rng.standard_normal((T, vd))
    Q, K, V = dev(q), dev(k), dev(v)
    tdt = torch.float32 if cache == DType.F32 else torch.bfloat16
    kc = torch.zeros(64, kh * dim, device="cuda", dtype=tdt); vc = torch.zeros(64, vd, device="cuda", dtype=tdt)
    f, mag = table(rot)
    lib().nt_b200_rope_partial_kv_write(Q.data_ptr(), K.data_ptr(), V.data_ptr(), f.data_ptr(), mag, rot["dims"], 1, dim, kc.data_ptr(), vc.data_ptr(),
                                        int(cache), T, p0, qh * dim, kh * dim, vd, stream())
    r = rot if rot["dims"] else None
    qr = np.stack([np.concatenate([O.rotate(q[t, h * dim:(h + 1) * dim], p0 + t, r) for h in range(qh)]) for t in range(T)])
    kr = np.stack([np.concatenate([O.rotate(k[t, h * dim:(h + 1) * dim], p0 + t, r) for h in range(kh)]) for t in range(T)])
    tol = 2e-5 if cache == DType.F32 else 1e-2
    np.testing.assert_allclose(Q.cpu().numpy(), qr, rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(kc[p0:p0 + T].float().cpu().numpy(), kr, rtol=tol, atol=tol)
    np.testing.assert_allclose(vc[p0:p0 + T].float().cpu().numpy(), v, rtol=tol, atol=tol)
    assert float(kc[:p0].abs().max()) == 0 and float(kc[p0 + T:].abs().max()) == 0
    # queries only (a layer that reads another layer's cache): the cache is left alone
    Q2 = dev(q); before = kc.clone()
    lib().nt_b200_rope_partial_kv_write(Q2.data_ptr(), None, None, f.data_ptr(), mag, rot["dims"], 1, dim, kc.data_ptr(), vc.data_ptr(), int(cache), T, p0,
                                        qh * dim, kh * dim, vd, stream())
    np.testing.assert_allclose(Q2.cpu().numpy(), qr, rtol=2e-5, atol=2e-5)
    assert torch.equal(before, kc)


def maps_reference(q, k, v, pos, H, G, maps, dim, vdim, chunk, scale):
    """q [H*maps*dim] at position pos over cache rows k [n, G*maps*dim], v [n, G*vdim] -> [H, maps, vdim]."""
    out = np.zeros((H, maps, vdim))
    js = [j for j in range(pos + 1) if O.visible(pos, j, chunk)]
    for h in range(H):
        g = h // (H // G)
        for a in range(maps):
            qq = q[(h * maps + a) * dim:(h * maps + a + 1) * dim]
            s = np.array([scale * float(qq @ k[j, (g * maps + a) * dim:(g * maps + a + 1) * dim]) for j in js])
            p = O.softmax(s)
            out[h, a] = sum(w * v[j, g * vdim:(g + 1) * vdim] for w, j in zip(p, js))
    return out


@pytest.mark.parametrize("cache", [DType.F32, DType.BF16])
@pytest.mark.parametrize("H,G,maps,dim,vdim,chunk", [(4, 2, 2, 8, 12, 7), (3, 3, 2, 16, 16, 40), (2, 1, 1, 12, 40, 5), (2, 2, 2, 8, 8, 1), (2, 1, 2, 8, 20, 0)])
def test_attention_maps_block_mask(cache, H, G, maps, dim, vdim, chunk):
    rng = np.random.default_rng(H * 100 + chunk)
    n = 93
    tdt = torch.float32 if cache == DType.F32 else torch.bfloat16
    kc = dev(rng.standard_normal((n, G * maps * dim)), tdt); vc = dev(rng.standard_normal((n, G * vdim)), tdt)
    k = kc.double().cpu().numpy(); v = vc.double().cpu().numpy()
    for p0, T in ((0, n), (50, 20), (n - 1, 1), (41, 1), (42, 1)):      # a whole prompt, a portion, single decoded tokens (also across block borders)
        q = rng.standard_normal((T, H * maps * dim))
        Q = dev(q); out = torch.zeros(T, H * maps * vdim, device="cuda")
        lib().nt_b200_attention_maps(out.data_ptr(), Q.data_ptr(), kc.data_ptr(), vc.data_ptr(), int(cache), T, p0, H, G, dim, vdim, chunk, maps, 0.4, n, stream())
        ref = np.stack([maps_reference(q[t], k, v, p0 + t, H, G, maps, dim, vdim, chunk, 0.4).reshape(-1) for t in range(T)])
        np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=3e-5, atol=3e-5)


@pytest.mark.parametrize("H,G,maps,dim,vdim,chunk", [(2, 1, 2, 32, 64, 40), (4, 2, 2, 64, 128, 100), (2, 2, 1, 64, 64, 33), (2, 1, 2, 128, 128, 64), (2, 2, 2, 32, 64, 0)])
def test_attention_maps_tiled_form(H, G, maps, dim, vdim, chunk):
    """Prompt portions over a 16-bit cache with tile-friendly head widths take the tiled tensor-core form: same answers, also for
    portions that start inside a block and for query tiles that straddle a block border."""
    rng = np.random.default_rng(dim + chunk)
    n = 200
    kc = dev(rng.standard_normal((n, G * maps * dim)), torch.bfloat16); vc = dev(rng.standard_normal((n, G * vdim)), torch.bfloat16)
    k = kc.double().cpu().numpy(); v = vc.double().cpu().numpy()
    for p0, T in ((0, n), (50, 100), (121, 16), (7, 70)):
        q = rng.standard_normal((T, H * maps * dim))
        Q = dev(q); out = torch.zeros(T, H * maps * vdim, device="cuda")
        lib().nt_b200_attention_maps(out.data_ptr(), Q.data_ptr(), kc.data_ptr(), vc.data_ptr(), int(DType.BF16), T, p0, H, G, dim, vdim, chunk, maps, dim ** -0.5, n, stream())
        ref = np.stack([maps_reference(q[t], k, v, p0 + t, H, G, maps, dim, vdim, chunk, dim ** -0.5).reshape(-1) for t in range(T)])
        np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("cache", [DType.F32, DType.BF16])
def test_decoded_token_over_long_blocks(cache):
    """A single decoded token in a block of hundreds of positions: its keys are split over a cluster of CTAs and merged."""
    rng = np.random.default_rng(17)
    H, G, maps, dim, vdim, chunk, n = 2, 1, 2, 16, 24, 600, 1000
    tdt = torch.float32 if cache == DType.F32 else torch.bfloat16
    kc = dev(rng.standard_normal((n, G * maps * dim)), tdt); vc = dev(rng.standard_normal((n, G * vdim)), tdt)
    k = kc.double().cpu().numpy(); v = vc.double().cpu().numpy()
    for pos in (599, 600, 601, 999, 350):
        q = rng.standard_normal(H * maps * dim)
        Q = dev(q[None]); out = torch.zeros(1, H * maps * vdim, device="cuda")
        lib().nt_b200_attention_maps(out.data_ptr(), Q.data_ptr(), kc.data_ptr(), vc.data_ptr(), int(cache), 1, pos, H, G, dim, vdim, chunk, maps, 0.3, n, stream())
        ref = maps_reference(q, k, v, pos, H, G, maps, dim, vdim, chunk, 0.3).reshape(-1)
        np.testing.assert_allclose(out[0].cpu().numpy(), ref, rtol=3e-5, atol=3e-5)


@pytest.mark.parametrize("tokens_at_once", [True, False])
def test_block_edges_with_one_loud_key(tokens_at_once):
    """Among hundreds of quiet keys, a key aligned with the query wins the softmax when it sits on the first row of the query's block,
    however far back that is, and is invisible one row earlier."""
    rng = np.random.default_rng(3)
    chunk, n, dim, vdim = 128, 400, 16, 24
    q = rng.standard_normal(dim); q /= np.linalg.norm(q)
    for loud, seen in ((256, True), (255, False), (383, True), (0, False)):
        k = rng.standard_normal((n, dim)) * 0.05
        k[loud] = 30.0 * q
        v = rng.standard_normal((n, vdim))
        kc, vc = dev(k), dev(v)
        pos = 383
        out = torch.zeros(n if tokens_at_once else 1, vdim, device="cuda")
        if tokens_at_once:
            Q = dev(np.tile(q, (n, 1)))
            lib().nt_b200_attention_maps(out.data_ptr(), Q.data_ptr(), kc.data_ptr(), vc.data_ptr(), int(DType.F32), n, 0, 1, 1, dim, vdim, chunk, 1, 1.0, n, stream())
            got = out[pos].cpu().numpy()
        else:
            Q = dev(q[None])
            lib().nt_b200_attention_maps(out.data_ptr(), Q.data_ptr(), kc.data_ptr(), vc.data_ptr(), int(DType.F32), 1, pos, 1, 1, dim, vdim, chunk, 1, 1.0, n, stream())
            got = out[0].cpu().numpy()
        ref = maps_reference(q, k, v, pos, 1, 1, 1, dim, vdim, chunk, 1.0).reshape(-1)
        np.testing.assert_allclose(got, ref, rtol=3e-5, atol=3e-5)
        assert (np.abs(got - v[loud]).max() < 1e-3) == seen


def test_differential_combination():
    rng = np.random.default_rng(9)
    T, H, vdim, n_l, d, eps = 5, 3, 20, 6, 0.35, 1e-5
    A = rng.standard_normal((T, H, 2, vdim))
    l = {n: rng.standard_normal(n_l) * 0.4 for n in ("lq1", "lk1", "lq2", "lk2")}
    lam = O.diff_lambda({"p." + n: x for n, x in l.items()}, "p.", d)
    ref = O.rms_unit(A[:, :, 0] - lam * A[:, :, 1], eps) * (1 - d)
    out = torch.zeros(T, H * vdim, device="cuda")
    t = {n: dev(x) for n, x in l.items()}
    Ad = dev(A)
    lib().nt_b200_diff_combine(out.data_ptr(), Ad.data_ptr(), t["lq1"].data_ptr(), t["lk1"].data_ptr(), t["lq2"].data_ptr(), t["lk2"].data_ptr(), n_l, d, eps,
                               T, H, vdim, stream())
    np.testing.assert_allclose(out.cpu().numpy().reshape(T, H, vdim), ref, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("S", [1, 2, 5])
def test_residual_streams(S):
    rng = np.random.default_rng(S)
    T, width = 6, 50
    e = rng.standard_normal((T, width)); X = torch.zeros(T, S, width, device="cuda")
    ed = dev(e)
    lib().nt_b200_streams_spread(X.data_ptr(), ed.data_ptr(), 0.3, T, S, width, stream())
    np.testing.assert_allclose(X.cpu().numpy(), np.repeat(0.3 * e[:, None], S, 1), rtol=1e-6)
    x = rng.standard_normal((T, S, width)); a = rng.standard_normal(S); M = rng.standard_normal((S, S)); b = rng.standard_normal(S); y = rng.standard_normal((T, width))
    X = dev(x); u = torch.zeros(T, width, device="cuda")
    ad, Md, bd, yd = dev(a), dev(M), dev(b), dev(y)
    lib().nt_b200_streams_read(u.data_ptr(), X.data_ptr(), ad.data_ptr(), T, S, width, stream())
    np.testing.assert_allclose(u.cpu().numpy(), np.einsum("s,tsc->tc", a, x), rtol=2e-5, atol=2e-5)
    lib().nt_b200_streams_read(u.data_ptr(), X.data_ptr(), None, T, S, width, stream())
    np.testing.assert_allclose(u.cpu().numpy(), x.sum(1), rtol=2e-5, atol=2e-5)
    lib().nt_b200_streams_write(X.data_ptr(), yd.data_ptr(), Md.data_ptr(), bd.data_ptr(), T, S, width, stream())
    W = {"p.in": a, "p.mix": M, "p.out": b}
    ref = O.stream_write(np.transpose(x, (1, 0, 2)), y, W, "p.")
    np.testing.assert_allclose(X.cpu().numpy(), np.transpose(ref, (1, 0, 2)), rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dt", [DType.F32, DType.BF16])
@pytest.mark.parametrize("E,top,ff,width,sff", [(5, 2, 20, 48, 14), (3, 3, 7, 30, 0), (9, 1, 64, 64, 64), (70, 4, 16, 40, 24)])
def test_mixture_of_experts(dt, E, top, ff, width, sff):
    rng = np.random.default_rng(E * 10 + top)
    T = 75
    tdt = torch.float32 if dt == DType.F32 else torch.bfloat16
    W = {"p.router": rng.standard_normal((E, width)), "p.shared.sg": rng.standard_normal((1, width)) * 0.3}
    ups = [dev(rng.standard_normal((ff, width)) * width ** -0.5, tdt) for _ in range(E)]
    downs = [dev(rng.standard_normal((width, ff)) * ff ** -0.5, tdt) for _ in range(E)]
    for e in range(E):
        W["p.e%d.up" % e] = ups[e].double().cpu().numpy(); W["p.e%d.down" % e] = downs[e].double().cpu().numpy()
    mlp = {"router": {"experts": E, "top": top}}
    sup = sdown = None
    if sff:
        sup = dev(rng.standard_normal((sff, width)) * width ** -0.5, tdt); sdown = dev(rng.standard_normal((width, sff)) * sff ** -0.5, tdt)
        W["p.shared.up"] = sup.double().cpu().numpy(); W["p.shared.down"] = sdown.double().cpu().numpy()
        mlp["shared"] = {"ff": sff}
    h = rng.standard_normal((T, width))
    ref = O.moe(h, W, "p.", mlp)
    Hd = dev(h); router = dev(W["p.router"]); sg = dev(W["p.shared.sg"].reshape(-1))
    sel = torch.zeros(T, top, device="cuda", dtype=torch.int32); wt = torch.zeros(T, top, device="cuda"); sgate = torch.zeros(T, device="cuda")
    lib().nt_b200_moe_route(sel.data_ptr(), wt.data_ptr(), sgate.data_ptr(), Hd.data_ptr(), router.data_ptr(), sg.data_ptr() if sff else None, E, top, width, T, stream())
    for t in range(T):
        ids, ws = O.route(h[t], W["p.router"], top)
        assert list(sel[t].cpu().numpy()) == list(ids)
        np.testing.assert_allclose(wt[t].cpu().numpy(), ws, rtol=2e-5, atol=1e-6)
    up_tab = torch.tensor([u.data_ptr() for u in ups], dtype=torch.int64, device="cuda"); down_tab = torch.tensor([d.data_ptr() for d in downs], dtype=torch.int64, device="cuda")
    # prompt rows: the shared expert's output arrives separately
    shared_y = None
    if sff:
        shared_y = dev(np.stack([O.expert(h[t], W["p.shared.up"], W["p.shared.down"]) for t in range(T)]))
    y = torch.zeros(T, width, device="cuda")
    scratch = torch.zeros(4 * (2 * T * top + 2 * E + 8) + 4 * T * top * (ff + width), device="cuda", dtype=torch.uint8)
    lib().nt_b200_moe_experts(y.data_ptr(), Hd.data_ptr(), sel.data_ptr(), wt.data_ptr(), sgate.data_ptr(), up_tab.data_ptr(), down_tab.data_ptr(), None, None,
                              shared_y.data_ptr() if sff else None, int(dt), E, top, ff, width, sff, T, 1, scratch.data_ptr(), stream())
    np.testing.assert_allclose(y.cpu().numpy(), ref, rtol=1e-4, atol=1e-4)
    # one token at a time: the shared expert rides along
    for t in (0, 1, T - 1):
        y1 = torch.zeros(width, device="cuda"); act = torch.zeros(top * ff + sff, device="cuda")
        lib().nt_b200_moe_experts(y1.data_ptr(), Hd[t].data_ptr(), sel[t].data_ptr(), wt[t].data_ptr(), sgate[t:].data_ptr(), up_tab.data_ptr(), down_tab.data_ptr(),
                                  sup.data_ptr() if sff else None, sdown.data_ptr() if sff else None, None, int(dt), E, top, ff, width, sff, 1, 0, act.data_ptr(), stream())
        np.testing.assert_allclose(y1.cpu().numpy(), ref[t], rtol=1e-4, atol=1e-4)


# ---------------------------------------------------------------- whole models through the engine
def build(cfg, W, exact, max_context=256):
    return Model.from_config_json(cfg, device_tensors(W, exact), max_context=max_context, exact_f32=exact)


def run_portions(model, toks, sizes):
    rows, pos = [], 0
    for n in sizes:
        rows.append(model.forward_logits(toks[pos:pos + n], pos, list(range(n))))
        pos += n
    assert pos == len(toks)
    return np.concatenate(rows)


def per_position(a, b):
    a = np.asarray(a, dtype=np.float64); b = np.asarray(b, dtype=np.float64)
    a = a - a.mean(-1, keepdims=True); b = b - b.mean(-1, keepdims=True)
    return np.sqrt(((a - b) ** 2).mean(-1)) / np.sqrt((b ** 2).mean())


CONFIGS = {
    "base": dict(),
    "shared_cache_and_bare_layer": dict(n_layers=4, kv_from={2: 0, 3: 1}, no_mlp=(1,)),
    "one_stream_top_one": dict(streams=1, top=1, heads=3, kv_heads=3, dim=10, vdim=10, rot_dims=10, width=36, chunk=5),
    "plain_residual_all_experts": dict(streams=0, experts=3, top=3, shared_ff=0, scaling=False, kv_heads=1, chunk=16),
    "block_longer_than_prompt": dict(chunk=500, n_layers=2, rot_dims=2),
    "no_positions_no_mask": dict(rot_dims=0, chunk=0, n_layers=2, streams=4),
    # every matrix tile-aligned: with BF16 weights the projections, the routed experts and the shared expert run on the tensor cores
    "tensor_core_tiles": dict(width=128, heads=2, kv_heads=2, dim=32, vdim=64, ff=128, shared_ff=128, n_layers=2, kv_from={1: 0}, chunk=24, rot_dims=16, streams=2),
    # experts too narrow for a tile (gathered CUDA-core GEMMs) beside tile-aligned projections; an expert nobody chooses is likely with 9 of them
    "mixed_tiles": dict(width=128, heads=2, kv_heads=1, dim=64, vdim=64, ff=40, shared_ff=128, experts=9, top=1, n_layers=2, chunk=33, rot_dims=64, streams=2),
}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("exact", [True, False])
def test_model_schedules_agree_with_oracle(name, exact):
    rng = np.random.default_rng(len(name))
    cfg, W = O.random_model(rng, **CONFIGS[name])
    S = 61
    toks = rng.integers(0, cfg["vocab"], S).astype(np.int32)
    ref = O.forward(cfg, W, toks)
    m = build(cfg, W, exact)

    def close(got):
        if exact:
            return rel_rms(got, ref) < 2e-4
        # 16-bit cache rows: the difference of the two maps and the per-head re-normalisation after it magnify their rounding, and a
        # router logit within that rounding of the next one may pick the other expert at a position; most positions stay tight
        err = per_position(got, ref)
        return np.median(err) < 1.5e-2 and err.max() < 0.2

    whole = run_portions(m, toks, [S])
    assert close(whole)
    single = run_portions(m, toks, [1] * S)
    assert close(single)
    mixed = run_portions(m, toks, [2, 17, 3, 2, 20, 5, 1, 1, 8, 2])      # portions cut anywhere, also inside a mask block
    assert close(mixed)
    assert close(run_portions(m, toks, [40] + [1] * 21))
    if exact:                                                            # how a prompt is cut changes rounding only
        assert rel_rms(single, whole) < 5e-5 and rel_rms(mixed, whole) < 5e-5
    m.close()


def test_first_tokens_and_single_token_request():
    rng = np.random.default_rng(2)
    cfg, W = O.random_model(rng, chunk=3)
    toks = rng.integers(0, cfg["vocab"], 5).astype(np.int32)
    ref = O.forward(cfg, W, toks)
    m = build(cfg, W, True)
    assert rel_rms(run_portions(m, toks[:1], [1]), ref[:1]) < 2e-4
    assert rel_rms(run_portions(m, toks, [2, 3]), ref) < 2e-4


def test_cache_rows_are_reused_between_requests():
    rng = np.random.default_rng(21)
    cfg, W = O.random_model(rng, kv_from={2: 1})
    a = rng.integers(0, cfg["vocab"], 50).astype(np.int32)
    b = rng.integers(0, cfg["vocab"], 30).astype(np.int32)
    m = build(cfg, W, True)
    run_portions(m, a, [50])
    after_a = run_portions(m, b, [18] + [1] * 12)                         # b overwrites a's rows from position 0
    m2 = build(cfg, W, True)
    alone = run_portions(m2, b, [18] + [1] * 12)
    np.testing.assert_array_equal(after_a, alone)
    assert rel_rms(alone, O.forward(cfg, W, b)) < 2e-4


def test_long_decode_across_many_blocks_and_graph_replay():
    rng = np.random.default_rng(8)
    cfg, W = O.random_model(rng, n_layers=2, chunk=9, width=32, ff=12, heads=2, kv_heads=1, dim=8, vdim=16, vocab=50, kv_from={1: 0})
    S = 150
    toks = rng.integers(0, cfg["vocab"], S).astype(np.int32)
    ref = O.forward(cfg, W, toks)
    m = build(cfg, W, True)
    assert rel_rms(run_portions(m, toks, [3] + [1] * (S - 3)), ref) < 2e-4
    m.use_graph(False)
    m.clear_kv()
    assert rel_rms(run_portions(m, toks, [3] + [1] * (S - 3)), ref) < 2e-4


def test_a_token_matters_only_inside_its_block():
    """One layer, so attention is the only path between positions.  A token that occurs nowhere else sits on the first row of the last
    block or on the row before it: the last logits must move in the first case and cannot in the second, in a prompt and when decoding."""
    rng = np.random.default_rng(13)
    cfg, W = O.random_model(rng, n_layers=1, chunk=32, scale=1.5)
    S = 32 * 3 + 20
    toks = rng.integers(1, cfg["vocab"], S).astype(np.int32)
    base = O.forward(cfg, W, toks)
    for special_at in (96, 95):
        t = toks.copy(); t[special_at] = 0
        ref = O.forward(cfg, W, t)
        m = build(cfg, W, True)
        for sizes in ([S], [64, 20] + [1] * (S - 84), [95, 2, 19]):
            assert rel_rms(run_portions(m, t, sizes), ref) < 2e-4
        moved = rel_rms(ref[-1:], base[-1:])
        assert (moved > 1e-3) == (special_at == 96), (special_at, moved)


def test_greedy_generation_through_the_engine(tmp_path):
    rng = np.random.default_rng(4)
    cfg, W = O.random_model(rng, n_layers=3, kv_from={2: 0}, chunk=6)
    d = write_model_dir(tmp_path / "m", cfg, W)
    prompt = rng.integers(0, cfg["vocab"], 19).astype(np.int32)
    for exact in (True, False):
        e = Engine()
        assert e.load_path(d, max_context=128, exact_f32=exact)
        assert e.vocab_size == cfg["vocab"] and e.n_layers == 3
        new = e.generate_ids(prompt, max_tokens=24, temperature=0.0)
        assert len(new) == 24
        assert e.generate_ids(prompt, max_tokens=24, temperature=0.0) == new       # the cache is cleared and reused
        logits = O.forward(cfg, W, np.concatenate([prompt, np.asarray(new, dtype=np.int32)]))
        for i, tok in enumerate(new):                                         # every generated id is the oracle's greedy choice
            row = logits[len(prompt) - 1 + i]
            assert row[tok] >= row.max() - (1e-3 if exact else 0.1), (exact, i)
        sampled = e.generate_ids(prompt, max_tokens=8, temperature=0.8, top_k=10, top_p=0.9, repeat_penalty=1.1, seed=7)
        assert len(sampled) == 8 and all(0 <= s < cfg["vocab"] for s in sampled)
        e.close()


def test_model_folder_loads_like_device_tensors(tmp_path):
    rng = np.random.default_rng(6)
    cfg, W = O.random_model(rng, kv_from={1: 0})
    toks = rng.integers(0, cfg["vocab"], 33).astype(np.int32)
    a = Model.load_dir(write_model_dir(tmp_path / "m", cfg, W), max_context=64, exact_f32=True)
    b = build(cfg, W, True, max_context=64)
    np.testing.assert_array_equal(a.forward_logits(toks, 0, [0, 5, 32]), b.forward_logits(toks, 0, [0, 5, 32]))
