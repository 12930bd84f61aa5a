"""Zelunex on the GPU against the plain float64 oracle (tests/zelunex_oracle.py): each mechanism's kernel alone, then whole models
through the engine's step function — prompt pass vs token-by-token decoding, portions, cache reuse, window / kept-prefix edges,
odd sizes, and greedy generation through the engine's own entry point."""
import math

import numpy as np
import pytest
import torch

import zelunex_oracle as O
from zelunex_util import device_tensors, rel_rms, write_model_dir

from ntransformer_b200._lib import lib
from ntransformer_b200.dtypes import DType
from ntransformer_b200.engine import Engine, Model

pytestmark = pytest.mark.gpu
TORCH_DT = {DType.F32: torch.float32, DType.F16: torch.float16, DType.BF16: torch.bfloat16}


def dev(a, dt=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(dt).contiguous()


def stream():
    return torch.cuda.current_stream().cuda_stream


# ---------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dt", [DType.F32, DType.BF16, DType.F16])
@pytest.mark.parametrize("K", [64, 200, 51])          # 16-byte rows, and row lengths that force the scalar path
def test_gemv_dense_epilogues(dt, K):
    rng = np.random.default_rng(K)
    outs = [24, 7, 13]
    Ws = [dev(rng.standard_normal((o, K)) * 0.1, TORCH_DT[dt]) for o in outs]
    x = dev(rng.standard_normal(K))
    ref = [W.double().cpu().numpy() @ x.double().cpu().numpy() for W in Ws]
    ys = [torch.zeros(o, device="cuda") for o in outs]
    lib().nt_b200_gemv_dense(ys[0].data_ptr(), ys[1].data_ptr(), ys[2].data_ptr(), Ws[0].data_ptr(), Ws[1].data_ptr(), Ws[2].data_ptr(), *outs, 3, K,
                             x.data_ptr(), int(dt), 0, None, 1.0, stream())
    for y, r in zip(ys, ref):
        np.testing.assert_allclose(y.cpu().numpy(), r, rtol=2e-5, atol=2e-5)
    # y += alpha * gain * Wx
    y0 = dev(rng.standard_normal(outs[0]))
    gain = dev(rng.standard_normal(outs[0]))
    y = y0.clone()
    lib().nt_b200_gemv_dense(y.data_ptr(), None, None, Ws[0].data_ptr(), None, None, outs[0], 0, 0, 1, K, x.data_ptr(), int(dt), 2, gain.data_ptr(), 0.7, stream())
    np.testing.assert_allclose(y.cpu().numpy(), y0.cpu().numpy() + 0.7 * gain.cpu().numpy() * ref[0], rtol=2e-5, atol=2e-5)
    # gated units
    Wu = dev(rng.standard_normal((outs[0], K)) * 0.1, TORCH_DT[dt])
    u = Wu.double().cpu().numpy() @ x.double().cpu().numpy()
    for ep, act in ((4, O.gelu_tanh), (3, lambda z: z / (1 + np.exp(-z)))):
        y = torch.zeros(outs[0], device="cuda")
        lib().nt_b200_gemv_dense(y.data_ptr(), None, None, Ws[0].data_ptr(), Wu.data_ptr(), None, outs[0], outs[0], 0, 2, K, x.data_ptr(), int(dt), ep, None, 1.0, stream())
        np.testing.assert_allclose(y.cpu().numpy(), act(ref[0]) * u, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dt", [DType.F32, DType.BF16])
@pytest.mark.parametrize("T,N,K", [(1, 5, 3), (70, 130, 45), (64, 64, 64), (37, 192, 96)])
def test_gemm_dense(dt, T, N, K):
    rng = np.random.default_rng(T * N)
    A = dev(rng.standard_normal((T, K)))
    W = dev(rng.standard_normal((N, K)) * 0.1, TORCH_DT[dt])
    ref = A.double().cpu().numpy() @ W.double().cpu().numpy().T
    Cm = torch.zeros(T, N, device="cuda")
    lib().nt_b200_gemm_dense(Cm.data_ptr(), A.data_ptr(), W.data_ptr(), int(dt), T, N, K, 0, None, 1.0, stream())
    np.testing.assert_allclose(Cm.cpu().numpy(), ref, rtol=3e-5, atol=3e-5)
    C0 = dev(rng.standard_normal((T, N)))
    gain = dev(rng.standard_normal(N))
    Cm = C0.clone()
    lib().nt_b200_gemm_dense(Cm.data_ptr(), A.data_ptr(), W.data_ptr(), int(dt), T, N, K, 2, gain.data_ptr(), 0.3, stream())
    np.testing.assert_allclose(Cm.cpu().numpy(), C0.cpu().numpy() + 0.3 * gain.cpu().numpy() * ref, rtol=3e-5, atol=3e-5)


def test_glu_mul_gelu_tanh():
    z = torch.linspace(-9, 9, 1001, device="cuda")
    u = torch.full_like(z, 1.5)
    out = torch.empty_like(z)
    lib().nt_b200_glu_mul(out.data_ptr(), z.data_ptr(), u.data_ptr(), z.numel(), 1, stream())
    np.testing.assert_allclose(out.cpu().numpy(), O.gelu_tanh(z.double().cpu().numpy()) * 1.5, rtol=1e-5, atol=1e-6)


def run_window_attention(q, k, v, heads, kv, dim, vdim, window, keep, scale, cap, p0, cache_dt=DType.F32, max_seq=None):
    """Full-sequence q/k/v [S, ...]: the cache holds all S rows, queries are the rows from p0 on."""
    S = q.shape[0]
    max_seq = max_seq or S
    kc = torch.zeros(max_seq, kv * dim, device="cuda", dtype=TORCH_DT[cache_dt])
    vc = torch.zeros(max_seq, kv * vdim, device="cuda", dtype=TORCH_DT[cache_dt])
    kc[:S] = dev(k, TORCH_DT[cache_dt]); vc[:S] = dev(v, TORCH_DT[cache_dt])
    Q = dev(q[p0:])
    out = torch.zeros(S - p0, heads * vdim, device="cuda")
    lib().nt_b200_attention_window(out.data_ptr(), Q.data_ptr(), kc.data_ptr(), vc.data_ptr(), int(cache_dt), S - p0, p0, heads, kv, dim, vdim, window, keep,
                                   scale, cap, max_seq, stream())
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("heads,kv,dim,vdim,window,keep", [(4, 2, 32, 16, 8, 2), (3, 3, 24, 40, 5, 0), (4, 1, 16, 16, 1, 3), (2, 2, 64, 8, 100, 1), (6, 2, 8, 72, 7, 7)])
def test_attention_window_against_oracle(heads, kv, dim, vdim, window, keep):
    rng = np.random.default_rng(heads * 100 + window)
    S = 45
    q = rng.standard_normal((S, heads * dim)); k = rng.standard_normal((S, kv * dim)); v = rng.standard_normal((S, kv * vdim))
    scale, cap = 0.9 / math.sqrt(dim), 6.0
    ref = O.window_attention(q, k, v, heads, kv, dim, vdim, scale, cap, window, keep)
    for p0 in (0, 1, 20, S - 1):                 # a whole prompt, portions, one decoded token
        got = run_window_attention(q, k, v, heads, kv, dim, vdim, window, keep, scale, cap, p0)
        np.testing.assert_allclose(got, ref[p0:], rtol=2e-5, atol=2e-5)
    got = run_window_attention(q, k, v, heads, kv, dim, vdim, window, keep, scale, cap, 3, cache_dt=DType.BF16)
    assert np.abs(got - ref[3:]).max() < 0.05


def bf16_round(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).to(torch.float32).numpy()


@pytest.mark.parametrize("heads,kv,dim,window,keep", [(4, 2, 64, 70, 3), (2, 2, 128, 64, 66), (2, 1, 64, 1, 0), (2, 1, 64, 300, 130)])
def test_attention_window_tiled_tensor_core_form(heads, kv, dim, window, keep):
    """Prompt portions of >= 16 tokens over a BF16 cache with equal key / value width take the tiled mma form: windows and kept
    prefixes that straddle its 64-key tiles, portions that start inside a tile."""
    rng = np.random.default_rng(window)
    S = 200
    q = rng.standard_normal((S, heads * dim)); k = bf16_round(rng.standard_normal((S, kv * dim))); v = bf16_round(rng.standard_normal((S, kv * dim)))
    scale, cap = 1.2 / math.sqrt(dim), 8.0
    ref = O.window_attention(q, k, v, heads, kv, dim, dim, scale, cap, window, keep)
    for p0 in (0, 50, 131, S - 16):
        got = run_window_attention(q, k, v, heads, kv, dim, dim, window, keep, scale, cap, p0, cache_dt=DType.BF16, max_seq=S + 7)
        np.testing.assert_allclose(got, ref[p0:], rtol=2e-3, atol=2e-3)
    one = run_window_attention(q, k, v, heads, kv, dim, dim, window, keep, scale, cap, S - 1, cache_dt=DType.BF16)      # one token: the per-token form
    np.testing.assert_allclose(one, ref[S - 1:], rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("window,keep,S", [(600, 5, 700), (0 + 300, 300, 1500), (2000, 0, 900)])
def test_decoded_token_over_a_long_window_splits_across_a_cluster(window, keep, S):
    """One token against hundreds of keys: the head's keys are split over several CTAs and merged; kept prefix and window far apart."""
    heads, kv, dim, vdim = 4, 2, 32, 48
    rng = np.random.default_rng(S)
    q = rng.standard_normal((S, heads * dim)); k = rng.standard_normal((S, kv * dim)); v = rng.standard_normal((S, kv * vdim))
    scale, cap = 1.0 / math.sqrt(dim), 10.0
    ref = O.window_attention_row(q[S - 1], k, v, S - 1, heads, kv, dim, vdim, scale, cap, window, keep)
    got = run_window_attention(q, k, v, heads, kv, dim, vdim, window, keep, scale, cap, S - 1, max_seq=S + 100)
    np.testing.assert_allclose(got[0], ref, rtol=2e-5, atol=2e-5)
    got = run_window_attention(q, bf16_round(k), bf16_round(v), heads, kv, dim, vdim, window, keep, scale, cap, S - 1, cache_dt=DType.BF16, max_seq=S + 100)
    ref = O.window_attention_row(q[S - 1], bf16_round(k), bf16_round(v), S - 1, heads, kv, dim, vdim, scale, cap, window, keep)
    np.testing.assert_allclose(got[0], ref, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dim,vdim,cache_dt,S", [(16, 8, DType.F32, 40), (64, 64, DType.BF16, 150)])
def test_attention_window_edges_show(dim, vdim, cache_dt, S):
    """One key gets a score far above the rest and a marked value: the output tells whether the query saw it."""
    heads, kv, window, keep = 2, 1, 6, 3
    rng = np.random.default_rng(3)
    for i in (S - 1, S - 15):
        for j, seen in ((i - window + 1, True), (i - window, False), (keep - 1, True), (keep, False), (0, True), (i, True), (i - 1, True)):
            q = rng.standard_normal((S, heads * dim)) * 0.05; k = rng.standard_normal((S, kv * dim)) * 0.05; v = rng.standard_normal((S, kv * vdim)) * 0.01
            unit = np.zeros(dim); unit[5] = 1.0
            q[i] = np.tile(unit * 10.0, heads); k[j] = unit * 10.0
            v[j] = 0.0; v[j, 3] = 1.0
            for p0 in (0, i):                    # inside a prompt portion, and as a token decoded alone
                out = run_window_attention(q[:i + 1], k[:i + 1], v[:i + 1], heads, kv, dim, vdim, window, keep, 1.0, 30.0, p0, cache_dt=cache_dt, max_seq=S + 24)
                mark = out[i - p0].reshape(heads, vdim)[:, 3]
                assert (mark > 0.99).all() if seen else (np.abs(mark) < 0.05).all(), (i, j, p0, mark)


def test_qk_norm_over_whole_projection_and_cache_rows():
    rng = np.random.default_rng(11)
    T, qd, kd, vd, p0, max_seq, eps = 5, 48, 24, 40, 3, 16, 1e-3
    q = rng.standard_normal((T, qd)) * 3; k = rng.standard_normal((T, kd)) * 0.2; v = rng.standard_normal((T, vd))
    qg = rng.standard_normal(qd); kg = rng.standard_normal(kd)
    Q = dev(q); kc = torch.zeros(max_seq, kd, device="cuda"); vc = torch.zeros(max_seq, vd, device="cuda")
    Kd, Vd, qgd, kgd = dev(k), dev(v), dev(qg), dev(kg)
    lib().nt_b200_qk_norm_kv_write(Q.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), qgd.data_ptr(), kgd.data_ptr(), eps, kc.data_ptr(), vc.data_ptr(),
                                   int(DType.F32), T, p0, qd, kd, vd, stream())
    torch.cuda.synchronize()
    np.testing.assert_allclose(Q.cpu().numpy(), O.rms_norm(q, qg, eps), rtol=2e-5, atol=2e-6)     # one norm across all heads
    np.testing.assert_allclose(kc[p0:p0 + T].cpu().numpy(), O.rms_norm(k, kg, eps), rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(vc[p0:p0 + T].cpu().numpy(), v.astype(np.float32), rtol=1e-6)
    assert float(kc[:p0].abs().sum()) == 0.0 and float(kc[p0 + T:].abs().sum()) == 0.0


# ---------------------------------------------------------------- whole models through the engine
def build(cfg, W, exact, max_context=256):
    return Model.from_config_json(cfg, device_tensors(W, torch.float32 if exact else torch.bfloat16), max_context=max_context, exact_f32=exact)


def run_portions(model, toks, sizes):
    rows, pos = [], 0
    for n in sizes:
        rows.append(model.forward_logits(toks[pos:pos + n], pos, list(range(n))))
        pos += n
    assert pos == len(toks)
    return np.concatenate(rows)


CONFIGS = {
    "base": dict(),
    "shared_and_bare": dict(n_layers=4, share={2: 0, 3: 1}, no_mlp=(1,)),
    "mha_wide_values": dict(heads=3, kv_heads=3, dim=24, vdim=40, width=72, ff=50, window=6, keep=0, mult=1.0),
    "mqa_window_one": dict(heads=4, kv_heads=1, dim=16, vdim=16, window=1, keep=3, softcap_c=4.0),
    "window_longer_than_prompt": dict(window=500, keep=5, n_layers=2),
    # every matrix tile-aligned: with BF16 weights the prompt pass runs on the tensor cores (fused gated epilogue included)
    "tensor_core_tiles": dict(width=128, heads=4, kv_heads=4, dim=32, vdim=32, ff=256, n_layers=2),
    # key / value projections too narrow for a tile: tensor-core and CUDA-core GEMMs mixed inside one layer
    "tiled_attention": dict(width=64, heads=2, kv_heads=1, dim=64, vdim=64, ff=64, n_layers=2, window=20, keep=3),
    "mixed_tiles": dict(width=128, heads=4, kv_heads=1, dim=32, vdim=64, ff=128, n_layers=2, share={1: 0}),
}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("exact", [True, False])
def test_model_schedules_agree_with_oracle(name, exact):
    rng = np.random.default_rng(len(name))
    cfg, W = O.random_model(rng, **CONFIGS[name])
    S = 61
    toks = rng.integers(0, cfg["vocab"], S).astype(np.int32)
    ref = O.forward(cfg, W, toks)
    tol = 2e-4 if exact else 3e-2
    m = build(cfg, W, exact)
    whole = run_portions(m, toks, [S])                                   # the batched prompt pass
    assert rel_rms(whole, ref) < tol
    single = run_portions(m, toks, [1] * S)                              # the decode step, token by token
    assert rel_rms(single, ref) < tol
    mixed = run_portions(m, toks, [2, 17, 3, 2, 20, 5, 1, 1, 8, 2])      # portions cut anywhere, both paths
    assert rel_rms(mixed, ref) < tol
    prompt_then_decode = run_portions(m, toks, [40] + [1] * 21)
    assert rel_rms(prompt_then_decode, ref) < tol
    if exact:                                                            # how a prompt is cut changes rounding only
        assert rel_rms(single, whole) < 5e-5 and rel_rms(mixed, whole) < 5e-5
    m.close()


def test_cache_rows_are_reused_between_requests():
    rng = np.random.default_rng(21)
    cfg, W = O.random_model(rng, window=7, keep=3)
    a = rng.integers(0, cfg["vocab"], 50).astype(np.int32)
    b = rng.integers(0, cfg["vocab"], 30).astype(np.int32)
    m = build(cfg, W, True)
    run_portions(m, a, [50])
    after_a = run_portions(m, b, [18] + [1] * 12)                         # b overwrites a's rows from position 0
    m2 = build(cfg, W, True)
    alone = run_portions(m2, b, [18] + [1] * 12)
    np.testing.assert_array_equal(after_a, alone)
    assert rel_rms(alone, O.forward(cfg, W, b)) < 2e-4


def test_long_decode_past_window_and_graph_replay():
    rng = np.random.default_rng(8)
    cfg, W = O.random_model(rng, n_layers=2, window=9, keep=2, width=32, ff=40, heads=2, kv_heads=1, dim=16, vdim=16, vocab=50)
    S = 150
    toks = rng.integers(0, cfg["vocab"], S).astype(np.int32)
    ref = O.forward(cfg, W, toks)
    m = build(cfg, W, True)
    got = run_portions(m, toks, [3] + [1] * (S - 3))
    assert rel_rms(got, ref) < 2e-4
    m.use_graph(False)
    m.clear_kv()
    assert rel_rms(run_portions(m, toks, [3] + [1] * (S - 3)), ref) < 2e-4


def test_far_key_decides_the_logits():
    """A token that occurs nowhere else is put at position 1 (inside the kept prefix) or 2 (just past it): 100 positions on, the
    logits must depend on it in the first case and cannot in the second (one layer, so no other path carries it)."""
    rng = np.random.default_rng(13)
    cfg, W = O.random_model(rng, n_layers=1, window=4, keep=2, softcap_c=25.0, scale=2.0)
    S = 110
    toks = rng.integers(1, cfg["vocab"], S).astype(np.int32)
    for special_at in (1, 2):
        t = toks.copy(); t[special_at] = 0
        ref = O.forward(cfg, W, t)
        base = O.forward(cfg, W, toks)
        m = build(cfg, W, True)
        got = run_portions(m, t, [64, 20] + [1] * 26)
        assert rel_rms(got, ref) < 2e-4
        moved = rel_rms(ref[-1:], base[-1:])
        assert (moved > 1e-3) == (special_at < 2), (special_at, moved)     # inside the kept prefix it matters, just outside it cannot


def test_greedy_generation_through_the_engine(tmp_path):
    rng = np.random.default_rng(4)
    cfg, W = O.random_model(rng, n_layers=3, share={2: 0}, window=6, keep=2)
    d = write_model_dir(tmp_path / "m", cfg, W)
    prompt = rng.integers(0, cfg["vocab"], 19).astype(np.int32)
    for exact in (True, False):
        e = Engine()
        assert e.load_path(d, max_context=128, exact_f32=exact)
        assert e.vocab_size == cfg["vocab"] and e.n_layers == 3
        new = e.generate_ids(prompt, max_tokens=24, temperature=0.0)
        assert len(new) == 24
        again = e.generate_ids(prompt, max_tokens=24, temperature=0.0)       # the cache is cleared and reused
        assert again == new
        logits = O.forward(cfg, W, np.concatenate([prompt, np.asarray(new, dtype=np.int32)]))
        for i, tok in enumerate(new):                                         # every generated id is the oracle's greedy choice
            row = logits[len(prompt) - 1 + i]
            assert row[tok] >= row.max() - (1e-3 if exact else 0.1), (exact, i)
        sampled = e.generate_ids(prompt, max_tokens=8, temperature=0.8, top_k=10, top_p=0.9, repeat_penalty=1.1, seed=7)
        assert len(sampled) == 8 and all(0 <= s < cfg["vocab"] for s in sampled)
        e.close()


def test_model_folder_loads_like_device_tensors(tmp_path):
    rng = np.random.default_rng(6)
    cfg, W = O.random_model(rng)
    toks = rng.integers(0, cfg["vocab"], 33).astype(np.int32)
    a = Model.load_dir(write_model_dir(tmp_path / "m", cfg, W), max_context=64, exact_f32=True)
    b = build(cfg, W, True, max_context=64)
    np.testing.assert_array_equal(a.forward_logits(toks, 0, [0, 5, 32]), b.forward_logits(toks, 0, [0, 5, 32]))
    np.testing.assert_allclose(a.forward(toks, 0), b.forward_logits(toks, 0, [32])[0], rtol=0, atol=0)
