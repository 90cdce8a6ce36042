"""Per-kernel parity on the GPU: every CUDA kernel, called through the C ABI on device pointers,
against the CPU oracle on the same seeded inputs."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G(dcd):
    import torch
    assert torch.cuda.is_available()
    import gpu_util
    return gpu_util


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


# ---------------------------------------------------------------------------------------------
# tcgen05 GEMM
# ---------------------------------------------------------------------------------------------
GEMM_SHAPES = [(128, 256, 64), (128, 256, 128), (256, 512, 256), (128, 256, 1024), (300, 776, 256), (77, 48, 688), (1000, 640, 5120),
               (2048, 5120, 1024), (640, 17408, 512), (2048, 16480, 256)]


@pytest.mark.parametrize("M,N,K", [(300, 776, 256), (2048, 5120, 1024)])
def test_gemm_tc_residual_epilogue_bit_exact(G, oracle, M, N, K):
    """C = bf16(resid + bf16(X W^T)) must equal the two-step form (GEMM, then the bf16 add) bit for bit."""
    import torch
    r = rng(M + N + K)
    dX = G.dev(oracle.rb(r.standard_normal((M, K), dtype=np.float32)), 1)
    dW = G.dev(oracle.rb(r.standard_normal((N, K), dtype=np.float32) * 0.05), 1)
    dR = G.dev(oracle.rb(r.standard_normal((M, N), dtype=np.float32)), 1)
    plain = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    fused = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    G.call("dcd_k_gemm_bf16_tc", dX, dW, plain, M, N, K, N, 0, G.sm_count(), err, None)
    G.call("dcd_k_gemm_bf16_tc_resid", dX, dW, dR, fused, M, N, K, N, G.sm_count(), err, None)
    assert int(err.item()) == 0
    want = (dR.float() + plain.float()).to(torch.bfloat16)
    assert torch.equal(fused, want)


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_tc_vs_fp32_matmul(G, oracle, M, N, K):
    import torch
    r = rng(M * 7 + N * 3 + K)
    X = oracle.rb(r.standard_normal((M, K), dtype=np.float32))
    W = oracle.rb(r.standard_normal((N, K), dtype=np.float32) * 0.05)
    dX, dW = G.dev(X, 1), G.dev(W, 1)
    dC = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    G.call("dcd_k_gemm_bf16_tc", G.p(dX), G.p(dW), G.p(dC), M, N, K, N, 0, G.sm_count(), G.p(err), None)
    assert int(err.item()) == 0, "a bounded wait gave up inside the kernel"
    got = G.host(dC)
    want = (dX.float() @ dW.float().T).cpu().numpy()  # exact bf16 products, f32 accumulation
    bad = ~(np.abs(got - want) <= 8e-3 * np.abs(want) + 2e-3)
    if bad.any():
        rows, cols = np.nonzero(bad)
        pytest.fail(f"{bad.mean():.4%} mismatched; nan={np.isnan(got).mean():.4%}; rows {rows.min()}..{rows.max()} cols {cols.min()}..{cols.max()}; "
                    f"first bad (r{rows[0]},c{cols[0]}): got {got[rows[0], cols[0]]} want {want[rows[0], cols[0]]}; "
                    f"row-hist(32) {np.bincount(rows // 32)[:16]} col-hist(32) {np.bincount(cols // 32)[:16]}")
    if M * N * K <= 300 * 776 * 256:
        np.testing.assert_allclose(got, oracle.k_gemm(X, W, True), rtol=8e-3, atol=2e-3)


def test_gemm_tc_swiglu_epilogue(G, oracle):
    import torch
    M, I, K = 200, 688, 256
    tiles = (I + 127) // 128
    r = rng(5)
    X = oracle.rb(r.standard_normal((M, K), dtype=np.float32))
    Wg = oracle.rb(r.standard_normal((I, K), dtype=np.float32) * 0.08)
    Wu = oracle.rb(r.standard_normal((I, K), dtype=np.float32) * 0.08)
    Wi = np.zeros((tiles * 256, K), np.float32)
    for j in range(I):
        Wi[(j // 128) * 256 + j % 128] = Wg[j]
        Wi[(j // 128) * 256 + 128 + j % 128] = Wu[j]
    dX, dW = G.dev(X, 1), G.dev(Wi, 1)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    G.call("dcd_k_gemm_bf16_tc", G.p(dX), G.p(dW), G.p(out), M, tiles * 256, K, I, 1, G.sm_count(), G.p(err), None)
    assert int(err.item()) == 0
    g, u = oracle.k_gemm(X, Wg, True), oracle.k_gemm(X, Wu, True)
    want = oracle.rb(oracle.rb(g / (1 + np.exp(-g))) * u)
    np.testing.assert_allclose(G.host(out), want, rtol=2e-2, atol=3e-3)


@pytest.mark.parametrize("dtype", [0, 1])
def test_gemm_fma(G, oracle, dtype):
    M, N, K = 70, 130, 100
    r = rng(9)
    X = r.standard_normal((M, K), dtype=np.float32)
    W = r.standard_normal((N, K), dtype=np.float32) * 0.1
    if dtype:
        X, W = oracle.rb(X), oracle.rb(W)
    out = G.empty((M, N), dtype)
    G.call("dcd_k_gemm_fma", G.p(G.dev(X, dtype)), G.p(G.dev(W, dtype)), G.p(out), M, N, K, dtype, None)
    rt, at = G.tol(dtype)
    np.testing.assert_allclose(G.host(out), oracle.k_gemm(X, W, bool(dtype)), rtol=rt, atol=at * 5)


# ---------------------------------------------------------------------------------------------
# norms and elementwise
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("rows,cols", [(5, 256), (37, 5120), (3, 64)])
def test_rmsnorm_and_add_rmsnorm(G, oracle, dtype, rows, cols):
    r = rng(rows + cols)
    x = r.standard_normal((rows, cols), dtype=np.float32) * 3
    m = r.standard_normal((rows, cols), dtype=np.float32)
    w = r.standard_normal(cols, dtype=np.float32) * 0.1
    if dtype:
        x, m, w = oracle.rb(x), oracle.rb(m), oracle.rb(w)
    rt, at = G.tol(dtype)
    for zc in (1, 0):
        out = G.empty((rows, cols), dtype)
        G.call("dcd_k_rmsnorm", G.p(G.dev(x, dtype)), G.p(G.dev(w, dtype)), G.p(out), rows, cols, C.c_float(1e-6), zc, dtype, None)
        np.testing.assert_allclose(G.host(out), oracle.k_rmsnorm(x, w, 1e-6, bool(zc), bool(dtype)), rtol=rt, atol=at)
    res, out = G.empty((rows, cols), dtype), G.empty((rows, cols), dtype)
    G.call("dcd_k_add_rmsnorm", G.p(G.dev(x, dtype)), G.p(G.dev(m, dtype)), G.p(G.dev(w, dtype)), G.p(res), G.p(out), rows, cols, C.c_float(1e-6), dtype, None)
    wres, wout = oracle.k_add_rmsnorm(x, m, w, 1e-6, bool(dtype))
    np.testing.assert_array_equal(G.host(res), wres)  # a single rounded add: bit-exact
    np.testing.assert_allclose(G.host(out), wout, rtol=rt, atol=at)


@pytest.mark.parametrize("dtype", [0, 1])
def test_rmsnorm_gated_strided(G, oracle, dtype):
    tokens, heads, dv, extra = 9, 4, 128, 40
    r = rng(3)
    x = r.standard_normal((tokens * heads, dv), dtype=np.float32)
    zfull = r.standard_normal((tokens, heads * dv + extra), dtype=np.float32) * 2
    w = 1 + r.standard_normal(dv, dtype=np.float32) * 0.05
    if dtype:
        x, zfull, w = oracle.rb(x), oracle.rb(zfull), oracle.rb(w)
    out = G.empty((tokens * heads, dv), dtype)
    dz = G.dev(zfull, dtype)
    G.call("dcd_k_rmsnorm_gated", G.p(G.dev(x, dtype)), C.c_void_p(dz.data_ptr() + 8 * dz.element_size()), heads * dv + extra, G.p(G.dev(w, dtype)), G.p(out),
           tokens, heads, dv, C.c_float(1e-6), dtype, None)
    z = zfull[:, 8:8 + heads * dv].reshape(tokens * heads, dv)
    rt, at = G.tol(dtype)
    np.testing.assert_allclose(G.host(out), oracle.k_rmsnorm_gated(x, z, w, 1e-6, bool(dtype)), rtol=rt * 2, atol=at * 2)


@pytest.mark.parametrize("dtype", [0, 1])
def test_silu_mul_and_add(G, oracle, dtype):
    n = 5000
    r = rng(4)
    g, u = r.standard_normal(n, dtype=np.float32) * 3, r.standard_normal(n, dtype=np.float32)
    if dtype:
        g, u = oracle.rb(g), oracle.rb(u)
    R = oracle.rb if dtype else (lambda v: v)
    out = G.empty((n,), dtype)
    G.call("dcd_k_silu_mul", G.p(G.dev(g, dtype)), G.p(G.dev(u, dtype)), G.p(out), n, dtype, None)
    rt, at = G.tol(dtype)
    np.testing.assert_allclose(G.host(out), R(R(g / (1 + np.exp(-g))) * u), rtol=rt, atol=at)
    G.call("dcd_k_add", G.p(G.dev(g, dtype)), G.p(G.dev(u, dtype)), G.p(out), n, dtype, None)
    np.testing.assert_array_equal(G.host(out), R(g + u))


# ---------------------------------------------------------------------------------------------
# GDN pieces
# ---------------------------------------------------------------------------------------------
def _pack(oracle, lens):
    cu, pos, tq, last = oracle.pack(lens, 0)
    return cu, tq


@pytest.mark.parametrize("dtype", [0, 1])
def test_conv1d_silu_seeded_packed(G, oracle, dtype):
    lens, ch, stride = [1, 2, 3, 4, 17, 40], 96, 120
    total = sum(lens)
    r = rng(6)
    xf = r.standard_normal((total, stride), dtype=np.float32)
    hist = r.standard_normal((3, ch), dtype=np.float32)
    w = r.uniform(-0.5, 0.5, (ch, 4)).astype(np.float32)
    if dtype:
        xf, hist, w = oracle.rb(xf), oracle.rb(hist), oracle.rb(w)
    cu, tq = _pack(oracle, lens)
    rt, at = G.tol(dtype)
    for h in (hist, None):
        out = G.empty((total, ch), dtype)
        G.call("dcd_k_conv1d_silu", G.p(G.dev(xf, dtype)), stride, G.p(None if h is None else G.dev(h, dtype)), G.p(G.dev(w, dtype)), G.p(out),
               G.p(G.devi(cu)), G.p(G.devi(tq)), total, ch, dtype, None)
        want = np.concatenate([oracle.k_conv1d(xf[cu[i]:cu[i + 1], :ch], h, w, bool(dtype)) for i in range(len(lens))])
        np.testing.assert_allclose(G.host(out), want, rtol=rt, atol=at)


@pytest.mark.parametrize("dtype,nk,nv,dk,dv", [(0, 2, 4, 64, 64), (1, 2, 4, 64, 64), (1, 16, 48, 128, 128)])
def test_gdn_prepare(G, oracle, dtype, nk, nv, dk, dv):
    T = 11
    cd = 2 * nk * dk + nv * dv
    r = rng(8)
    conv = r.standard_normal((T, cd), dtype=np.float32)
    ba = r.standard_normal((T, 2 * nv + 6), dtype=np.float32) * 2
    A_log = r.uniform(0, 2.77, nv).astype(np.float32)
    dtb = r.uniform(-6.9, -2.3, nv).astype(np.float32)
    if dtype:
        conv, ba = oracle.rb(conv), oracle.rb(ba)
    qf, kf = G.devf(np.zeros((T, nk, dk))), G.devf(np.zeros((T, nk, dk)))
    g, beta = G.devf(np.zeros((T, nv))), G.devf(np.zeros((T, nv)))
    dba = G.dev(ba, dtype)
    es = dba.element_size()
    G.call("dcd_k_gdn_prepare", G.p(G.dev(conv, dtype)), cd, C.c_void_p(dba.data_ptr()), C.c_void_p(dba.data_ptr() + nv * es), 2 * nv + 6,
           G.p(G.devf(A_log)), G.p(G.devf(dtb)), G.p(qf), G.p(kf), G.p(g), G.p(beta), T, nk, nv, dk, dtype, None)
    wq, wk, wv, wg, wb = oracle.k_gdn_prepare(conv, ba[:, :nv], ba[:, nv:2 * nv], A_log, dtb, nk, nv, dk, dv, bool(dtype))
    rep = nv // nk
    np.testing.assert_allclose(G.host(qf), wq[:, ::rep], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(G.host(kf), wk[:, ::rep], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(G.host(g), wg, rtol=2e-5, atol=1e-7)
    np.testing.assert_allclose(G.host(beta), wb, rtol=8e-3 if dtype else 1e-5, atol=1e-6)


def _host_data(n, a, b):
    """Deterministic synthetic data of the reference's GDN tests (native/tests/gdn_chunked.rs:14-22)."""
    i = np.arange(n, dtype=np.float32)
    return (np.sin(0.017 * i) * a + np.cos(0.071 * i) * b).astype(np.float32)


def _gdn_inputs(oracle, T, nk, nv, dk, dv, dtype):
    cd = 2 * nk * dk + nv * dv
    conv = _host_data(T * cd, 0.6, 0.4).reshape(T, cd)
    if dtype:
        conv = oracle.rb(conv)
    q = _host_data(T * nk * dk, 1.0, 0.5).reshape(T, nk, dk)
    k = _host_data(T * nk * dk, 0.7, -0.9).reshape(T, nk, dk)
    q = (q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) / np.sqrt(dk)).astype(np.float32)
    k = (k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)).astype(np.float32)
    g = (-0.015 + 0.01 * _host_data(T * nv, 0.5, 0.5).reshape(T, nv)).astype(np.float32)   # in [-0.025,-0.005]
    beta = (0.5 + 0.4 * _host_data(T * nv, 0.5, -0.5).reshape(T, nv)).astype(np.float32)   # in [0.1,0.9]
    return conv, q, k, g, beta


@pytest.mark.parametrize("dtype,nk,nv,dk,dv,narrow", [(0, 2, 4, 64, 64, 0), (1, 2, 4, 64, 64, 1), (1, 16, 48, 128, 128, 0), (1, 16, 48, 128, 128, 1)])
def test_gdn_recurrent_vs_oracle(G, oracle, dtype, nk, nv, dk, dv, narrow):
    """Known-shape test after native/tests/gdn_chunked.rs: out max < 2e-2, mean < 2e-4, state max < 2e-3."""
    lens = [73, 64, 89] if dk == 128 else [5, 1, 30]
    T = sum(lens)
    conv, q, k, g, beta = _gdn_inputs(oracle, T, nk, nv, dk, dv, dtype)
    cd = conv.shape[1]
    seed = (0.05 * _host_data(nv * dk * dv, 1.0, 1.0)).reshape(nv, dk, dv).astype(np.float32)
    cu, _ = _pack(oracle, lens)
    out = G.empty((T, nv * dv), dtype)
    fin = G.devf(np.zeros((len(lens), nv, dk, dv)))
    G.call("dcd_k_gdn_recurrent", G.p(G.devf(q)), G.p(G.devf(k)), G.p(G.dev(conv, dtype)), cd, G.p(G.devf(g)), G.p(G.devf(beta)), G.p(G.devf(seed)),
           G.p(fin), G.p(out), G.p(G.devi(cu)), len(lens), nk, nv, dk, dv, narrow, dtype, None)
    rep = nv // nk
    got, gfin = G.host(out), G.host(fin)
    for i, L in enumerate(lens):
        sl = slice(cu[i], cu[i + 1])
        v = conv[sl, 2 * nk * dk:].reshape(L, nv, dv)
        want, wstate = oracle.k_gdn_recurrent(np.repeat(q[sl], rep, 1), np.repeat(k[sl], rep, 1), v, g[sl], beta[sl], seed, bool(dtype))
        d = np.abs(got[sl].reshape(L, nv, dv) - want)
        assert d.max() < 2e-2 and d.mean() < 2e-4, (d.max(), d.mean())
        assert np.abs(gfin[i] - wstate).max() < 2e-3
    # batched == per-sequence, bit-exact (native/tests/gdn_chunked.rs:314-315)
    for i, L in enumerate(lens):
        sl = slice(cu[i], cu[i + 1])
        o1 = G.empty((L, nv * dv), dtype)
        G.call("dcd_k_gdn_recurrent", G.p(G.devf(q[sl])), G.p(G.devf(k[sl])), G.p(G.dev(conv[sl], dtype)), cd, G.p(G.devf(g[sl])), G.p(G.devf(beta[sl])),
               G.p(G.devf(seed)), None, G.p(o1), G.p(G.devi([0, L])), 1, nk, nv, dk, dv, narrow, dtype, None)
        np.testing.assert_array_equal(G.host(o1), got[sl])


# ---------------------------------------------------------------------------------------------
# attention pieces
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,heads,kv,hd,rot", [(0, 4, 1, 64, 16), (1, 4, 1, 64, 16), (1, 24, 4, 256, 64), (0, 6, 2, 128, 128)])
def test_qk_norm_rope(G, oracle, dtype, heads, kv, hd, rot):
    T, max_pos, theta = 13, 4096, 1e7
    r = rng(11)
    qstride = heads * 2 * hd + 2 * kv * hd
    fused = r.standard_normal((T, qstride), dtype=np.float32)
    qw, kw = r.standard_normal(hd, dtype=np.float32) * 0.1, r.standard_normal(hd, dtype=np.float32) * 0.1
    pos = r.integers(0, max_pos, T).astype(np.int32)
    R = oracle.rb if dtype else (lambda v: v)
    if dtype:
        fused, qw, kw = R(fused), R(qw), R(kw)
    cos_t, sin_t = oracle.k_rope_tables(rot, theta, max_pos, bool(dtype))
    dq, dk_ = G.empty((T, heads, hd), dtype), G.empty((T, kv, hd), dtype)
    err = G.devi([0])
    df = G.dev(fused, dtype)
    es = df.element_size()
    G.call("dcd_k_qk_norm_rope", G.p(df), qstride, C.c_void_p(df.data_ptr() + heads * 2 * hd * es), qstride, G.p(G.dev(qw, dtype)), G.p(G.dev(kw, dtype)),
           G.p(G.dev(cos_t, dtype)), G.p(G.dev(sin_t, dtype)), G.p(G.devi(pos)), max_pos, G.p(dq), G.p(dk_), T, heads, kv, hd, rot, C.c_float(1e-6), G.p(err), dtype, None)
    assert int(err.item()) == 0
    q_in = fused[:, :heads * 2 * hd].reshape(T, heads, 2 * hd)[:, :, :hd]
    k_in = fused[:, heads * 2 * hd:heads * 2 * hd + kv * hd].reshape(T, kv, hd)
    wq = oracle.k_rope(oracle.k_rmsnorm(q_in.reshape(-1, hd), qw, 1e-6, True, bool(dtype)).reshape(T, heads, hd), pos, rot, theta, bool(dtype))
    wk = oracle.k_rope(oracle.k_rmsnorm(k_in.reshape(-1, hd), kw, 1e-6, True, bool(dtype)).reshape(T, kv, hd), pos, rot, theta, bool(dtype))
    rt, at = G.tol(dtype)
    np.testing.assert_allclose(G.host(dq), wq, rtol=rt * 2, atol=at * 4)
    np.testing.assert_allclose(G.host(dk_), wk, rtol=rt * 2, atol=at * 4)


@pytest.mark.parametrize("dtype,heads,kv,hd", [(0, 4, 1, 64), (1, 4, 1, 64), (1, 24, 4, 256)])
def test_attention_state_plus_own_and_split(G, oracle, dtype, heads, kv, hd):
    lens, S = [1, 15, 16, 33], 70
    T = sum(lens)
    r = rng(13)
    R = oracle.rb if dtype else (lambda v: v)
    q = R(r.standard_normal((T, heads, hd), dtype=np.float32))
    ko = R(r.standard_normal((T, kv, hd), dtype=np.float32))
    vo = R(r.standard_normal((T, kv, hd), dtype=np.float32))
    ks = R(r.standard_normal((S, kv, hd), dtype=np.float32))
    vs = R(r.standard_normal((S, kv, hd), dtype=np.float32))
    qg = R(r.standard_normal((T, heads, 2 * hd), dtype=np.float32))
    cu, pos, tq, last = oracle.pack(lens, 0)
    out = G.empty((T, heads, hd), dtype)
    G.call("dcd_k_attention", G.p(G.dev(q, dtype)), G.p(G.dev(ko, dtype)), kv * hd, G.p(G.dev(vo, dtype)), kv * hd, G.p(G.dev(ks, dtype)), G.p(G.dev(vs, dtype)), S,
           G.p(G.dev(qg, dtype)), heads * 2 * hd, G.p(out), G.p(G.devi(cu)), G.p(G.devi(tq)), T, heads, kv, hd, 0, dtype, None)
    gate = R(1 / (1 + np.exp(-qg[:, :, hd:])))
    want = np.concatenate([oracle.k_attention(q[cu[i]:cu[i + 1]], ks, vs, ko[cu[i]:cu[i + 1]], vo[cu[i]:cu[i + 1]], bool(dtype)) for i in range(len(lens))])
    rt, at = (1e-4, 1e-5) if dtype == 0 else (2e-2, 6e-3)
    np.testing.assert_allclose(G.host(out), R(want * gate), rtol=rt, atol=at)
    # per-row reference mask: one sequence, rows < split see keys < split
    split = 20
    out2 = G.empty((T, heads, hd), dtype)
    G.call("dcd_k_attention", G.p(G.dev(q, dtype)), G.p(G.dev(ko, dtype)), kv * hd, G.p(G.dev(vo, dtype)), kv * hd, None, None, 0, None, 0, G.p(out2),
           G.p(G.devi([0, T])), G.p(G.devi(np.zeros(T))), T, heads, kv, hd, split, dtype, None)
    w_state = oracle.k_attention(q[:split], ko[:split], vo[:split], None, None, bool(dtype))
    w_q = oracle.k_attention(q[split:], ko[:split], vo[:split], ko[split:], vo[split:], bool(dtype))
    np.testing.assert_allclose(G.host(out2), np.concatenate([w_state, w_q]), rtol=rt, atol=at)


def test_readout_f32(G, oracle):
    B, H, Rr = 7, 5120, 255
    r = rng(17)
    x, W = r.standard_normal((B, H), dtype=np.float32), r.standard_normal((Rr, H), dtype=np.float32) * 0.02
    out = G.devf(np.zeros((B, Rr)))
    G.call("dcd_k_readout", G.p(G.devf(x)), G.p(G.devf(W)), G.p(out), B, H, Rr, None)
    np.testing.assert_allclose(G.host(out), oracle.k_gemm(x, W, False), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("lens,S", [([1, 15, 16, 33], 70), ([130, 21, 22, 64, 65], 200), ([300], 0), ([5, 40], 64),
                                    # around the 128-key tile edges: full tiles only, one key short, one key over, several state tiles
                                    ([127, 128, 129], 128), ([1, 256, 257], 255), ([40, 3], 385), ([128], 0)])
def test_attention_tcgen05_vs_oracle(G, oracle, lens, S):
    """The tensor-core attention kernel (d3 shape: 24 query heads, 4 KV heads, head_dim 256) over
    [state || own] keys for a ragged packed batch, and as state self-attention (S = 0)."""
    import torch
    heads, kv, hd = 24, 4, 256
    T = sum(lens)
    r = rng(31 + T + S)
    R = oracle.rb
    q = R(r.standard_normal((T, heads, hd), dtype=np.float32))
    # own K/V live inside a wider fused row (stride > kv*hd), as in the engine
    stride = kv * hd + 64
    kof = R(r.standard_normal((T, stride), dtype=np.float32))
    vof = R(r.standard_normal((T, stride), dtype=np.float32))
    ko, vo = kof[:, :kv * hd].reshape(T, kv, hd), vof[:, :kv * hd].reshape(T, kv, hd)
    ks = R(r.standard_normal((max(S, 1), kv, hd), dtype=np.float32))
    vs = R(r.standard_normal((max(S, 1), kv, hd), dtype=np.float32))
    qg = R(r.standard_normal((T, heads, 2 * hd), dtype=np.float32))
    cu, pos, tq, last = oracle.pack(lens, 0)
    out = torch.full((T, heads, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    err = G.devi([0])
    tile_cu = G.devi(np.zeros(len(lens) + 1))
    G.call("dcd_k_attention_tc", G.dev(q, 1), G.dev(kof, 1), stride, G.dev(vof, 1), stride, G.dev(ks, 1) if S else None, G.dev(vs, 1) if S else None, S,
           G.dev(qg, 1), heads * 2 * hd, out, G.devi(cu), tile_cu, len(lens), T, heads, kv, hd, err, None)
    assert int(err.item()) == 0, "a bounded wait gave up inside the kernel"
    gate = R(1 / (1 + np.exp(-qg[:, :, hd:])))
    parts = []
    for i in range(len(lens)):
        sl = slice(cu[i], cu[i + 1])
        if S:
            parts.append(oracle.k_attention(q[sl], ks, vs, ko[sl], vo[sl], True))
        else:
            parts.append(oracle.k_attention(q[sl], ko[sl], vo[sl], None, None, True))
    want = R(np.concatenate(parts) * gate)
    got = G.host(out)
    bad = ~(np.abs(got - want) <= 2e-2 * np.abs(want) + 8e-3)
    if bad.any():
        t_, h_, d_ = np.nonzero(bad)
        pytest.fail(f"{bad.mean():.4%} mismatched, nan {np.isnan(got).mean():.4%}; tokens {np.unique(t_)[:20]} heads {np.unique(h_)[:24]} dims {d_.min()}..{d_.max()}; "
                    f"first got {got[t_[0], h_[0], d_[0]]} want {want[t_[0], h_[0], d_[0]]}; max abs {np.nanmax(np.abs(got - want))}")


@pytest.mark.parametrize("lens,S,n_split", [([16], 4096, 0), ([16, 16], 4096, 0), ([16], 16384, 0), ([16, 16], 16384, 0),
                                            ([16, 5], 1000, 3), ([40], 300, 5), ([130, 3], 2048, 2)])
def test_attention_split_kv_vs_oracle(G, oracle, lens, S, n_split):
    """Few rows over a long state: the key tiles of each (token tile, KV head) split over several CTAs and merged with the base-2
    log-sum-exp identity (n_split = 0: the engine's rule for this device; 5 parts over 4 key tiles leaves one part empty), against
    the oracle and against the unsplit kernel."""
    import torch
    heads, kv, hd = 24, 4, 256
    T = sum(lens)
    r = rng(77 + T + S)
    R = oracle.rb
    q = R(r.standard_normal((T, heads, hd), dtype=np.float32))
    stride = kv * hd + 64
    kof = R(r.standard_normal((T, stride), dtype=np.float32))
    vof = R(r.standard_normal((T, stride), dtype=np.float32))
    ko, vo = kof[:, :kv * hd].reshape(T, kv, hd), vof[:, :kv * hd].reshape(T, kv, hd)
    ks = R(r.standard_normal((S, kv, hd), dtype=np.float32))
    vs = R(r.standard_normal((S, kv, hd), dtype=np.float32))
    qg = R(r.standard_normal((T, heads, 2 * hd), dtype=np.float32))
    cu, pos, tq, last = oracle.pack(lens, 0)
    err = G.devi([0])
    tile_cu = G.devi(np.zeros(len(lens) + 1))
    dev = (G.dev(q, 1), G.dev(kof, 1), stride, G.dev(vof, 1), stride, G.dev(ks, 1), G.dev(vs, 1), S, G.dev(qg, 1), heads * 2 * hd)
    tail = (G.devi(cu), tile_cu, len(lens), T, heads, kv, hd, err)
    plain = torch.full((T, heads, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_attention_tc", *dev, plain, *tail, None)
    ws_bytes = 2 * G.sm_count() * 128 * 1032
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    out = torch.full((T, heads, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_attention_tc_split", *dev, out, *tail, n_split, ws, C.c_size_t(ws_bytes), None)
    assert int(err.item()) == 0, "a bounded wait gave up inside the kernel"
    gate = R(1 / (1 + np.exp(-qg[:, :, hd:])))
    want = R(np.concatenate([oracle.k_attention(q[cu[i]:cu[i + 1]], ks, vs, ko[cu[i]:cu[i + 1]], vo[cu[i]:cu[i + 1]], True) for i in range(len(lens))]) * gate)
    got, ref = G.host(out), G.host(plain)
    assert np.isfinite(got).all()
    assert (np.abs(got - want) <= 2e-2 * np.abs(want) + 8e-3).all(), float(np.abs(got - want).max())
    assert (np.abs(got - ref) <= 2e-2 * np.abs(ref) + 2e-3).all(), float(np.abs(got - ref).max())


@pytest.mark.parametrize("n_split", [16, 0])
def test_attention_split_kv_same_bits_every_run(G, n_split):
    """The parts of a split launch run two to four key tiles each, their K/V comes cold from HBM, and the softmax warps reach the
    epilogue while the product of the tile before the last still waits for its V tile: the end of the LAST product has a barrier
    of its own (a phase-parity wait on the per-tile barrier read as complete one product early and left whole tiles out of the
    partial outputs). Repeated with whatever the workspace held before and with the caches flushed: the same bits every time,
    and the unsplit kernel's result within rounding."""
    import torch
    heads, kv, hd, S, T = 24, 4, 256, 16384, 16
    torch.manual_seed(5)
    q = torch.randn(T, heads, hd, device="cuda").bfloat16()
    ko = torch.randn(T, kv * hd, device="cuda").bfloat16()
    vo = torch.randn(T, kv * hd, device="cuda").bfloat16()
    ks = torch.randn(S, kv, hd, device="cuda").bfloat16()
    vs = torch.randn(S, kv, hd, device="cuda").bfloat16()
    qg = torch.randn(T, heads, 2 * hd, device="cuda").bfloat16()
    cu = G.devi(np.array([0, T]))
    tile_cu = G.devi(np.zeros(2))
    err = G.devi([0])
    dev = (q, ko, kv * hd, vo, kv * hd, ks, vs, S, qg, heads * 2 * hd)
    tail = (cu, tile_cu, 1, T, heads, kv, hd, err)
    plain = torch.full((T, heads, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_attention_tc", *dev, plain, *tail, None)
    ws_bytes = 2 * G.sm_count() * 128 * 1032
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    first = None
    for _ in range(12):
        ws.random_(0, 256)
        flush.zero_()
        out = torch.full((T, heads, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        G.call("dcd_k_attention_tc_split", *dev, out, *tail, n_split, ws, C.c_size_t(ws_bytes), None)
        torch.cuda.synchronize()
        if first is None:
            first = out.clone()
            assert float((first.float() - plain.float()).abs().max()) < 1e-3
        else:
            assert torch.equal(out.view(torch.int16), first.view(torch.int16))
    assert int(err.item()) == 0


@pytest.mark.parametrize("dtype,nk,nv,dv,narrow", [(1, 16, 48, 128, 0), (1, 16, 48, 128, 1), (0, 2, 6, 64, 0), (0, 2, 6, 64, 1)])
def test_gdn_chunked_vs_oracle(G, oracle, dtype, nk, nv, dv, narrow):
    """Chunked tensor-core gated delta rule against the sequential oracle, with the tolerances of the
    reference's own chunked-vs-sequential test (native/tests/gdn_chunked.rs:109-111): out max < 2e-2,
    mean < 2e-4, state max < 2e-3; lengths straddle the 32-token chunk (1, 31, 33, 64, 73, 89)."""
    dk = 128
    lens = [73, 64, 89, 1, 31, 33]
    T = sum(lens)
    conv, q, k, g, beta = _gdn_inputs(oracle, T, nk, nv, dk, dv, dtype)
    cd = conv.shape[1]
    seed = (0.05 * _host_data(nv * dk * dv, 1.0, 1.0)).reshape(nv, dk, dv).astype(np.float32)
    cu, _ = _pack(oracle, lens)
    out = G.empty((T, nv * dv), dtype)
    fin = G.devf(np.zeros((len(lens), nv, dk, dv)))
    G.call("dcd_k_gdn_chunked", G.devf(q), G.devf(k), G.dev(conv, dtype), cd, G.devf(g), G.devf(beta), G.devf(seed), fin, out, G.devi(cu), len(lens),
           nk, nv, dk, dv, narrow, dtype, None)
    rep = nv // nk
    got, gfin = G.host(out), G.host(fin)
    worst = (0.0, 0.0, 0.0)
    for i, L in enumerate(lens):
        sl = slice(cu[i], cu[i + 1])
        v = conv[sl, 2 * nk * dk:].reshape(L, nv, dv)
        want, wstate = oracle.k_gdn_recurrent(np.repeat(q[sl], rep, 1), np.repeat(k[sl], rep, 1), v, g[sl], beta[sl], seed, bool(dtype))
        d = np.abs(got[sl].reshape(L, nv, dv) - want)
        ds = np.abs(gfin[i] - wstate).max()
        worst = (max(worst[0], d.max()), max(worst[1], d.mean()), max(worst[2], ds))
    print("gdn chunked vs sequential oracle: out max %.3g mean %.3g state max %.3g" % worst)
    assert worst[0] < 2e-2 and worst[1] < 2e-4 and worst[2] < 2e-3, worst
    # zero seed (capture) and no final-state store
    out2 = G.empty((T, nv * dv), dtype)
    G.call("dcd_k_gdn_chunked", G.devf(q), G.devf(k), G.dev(conv, dtype), cd, G.devf(g), G.devf(beta), None, None, out2, G.devi(cu), len(lens),
           nk, nv, dk, dv, narrow, dtype, None)
    sl = slice(cu[2], cu[3])
    v = conv[sl, 2 * nk * dk:].reshape(lens[2], nv, dv)
    want, _ = oracle.k_gdn_recurrent(np.repeat(q[sl], rep, 1), np.repeat(k[sl], rep, 1), v, g[sl], beta[sl], np.zeros_like(seed), bool(dtype))
    assert np.abs(G.host(out2)[sl].reshape(lens[2], nv, dv) - want).max() < 2e-2


# ---------------------------------------------------------------------------------------------
# FP8 (E4M3) path
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [0, 1])
def test_quant_fp8_rows_bit_exact(G, oracle, dtype):
    import torch
    rows, cols, stride = 9, 688, 720
    r = rng(41)
    xf = (r.standard_normal((rows, stride), dtype=np.float32) * np.exp(r.uniform(-6, 4, (rows, 1)))).astype(np.float32)
    xf[3] = 0.0                      # an all-zero row: scale floor 1e-10/448
    if dtype:
        xf = oracle.rb(xf)
    codes = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
    scales = G.devf(np.zeros(rows))
    G.call("dcd_k_quant_fp8_rows", G.dev(xf, dtype), stride, codes, scales, rows, cols, C.c_float(1.0), dtype, None)
    wc, ws = oracle.k_quant_fp8_rows(xf[:, :cols])
    assert G.host(scales).tobytes() == ws.tobytes()
    assert np.array_equal(codes.cpu().numpy(), wc)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 776, 256), (77, 48, 688), (1000, 640, 5120), (700, 5120, 17408)])
def test_gemm_fp8_tc_vs_oracle(G, oracle, M, N, K):
    import torch
    r = rng(M + N + K)
    X = oracle.rb(r.standard_normal((M, K), dtype=np.float32))
    W = oracle.rb(r.standard_normal((N, K), dtype=np.float32) * 0.02)
    xq = torch.zeros((M, K), dtype=torch.uint8, device="cuda")
    wq = torch.zeros((N, K), dtype=torch.uint8, device="cuda")
    xs, ws = G.devf(np.zeros(M)), G.devf(np.zeros(N))
    G.call("dcd_k_quant_fp8_rows", G.dev(X, 1), K, xq, xs, M, K, C.c_float(1.0), 1, None)
    G.call("dcd_k_quant_fp8_rows", G.dev(W, 1), K, wq, ws, N, K, C.c_float(1.0), 1, None)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    err = G.devi([0])
    G.call("dcd_k_gemm_fp8_tc", xq, wq, out, M, N, K, N, 0, xs, ws, G.sm_count(), err, None)
    assert int(err.item()) == 0
    got = G.host(out)
    if M * N * K <= 1000 * 640 * 5120:
        want = oracle.k_gemm_fp8(X, W, True)
    else:  # same arithmetic with torch: exact e4m3 products, f32 accumulation, the two scales, bf16 rounding
        xv = torch.from_numpy(oracle.e4m3_to_f32(xq.cpu().numpy())).cuda()
        wv = torch.from_numpy(oracle.e4m3_to_f32(wq.cpu().numpy())).cuda()
        want = ((xv @ wv.T) * ws[None, :] * xs[:, None]).to(torch.bfloat16).float().cpu().numpy()
    bad = ~(np.abs(got - want) <= 8e-3 * np.abs(want) + 2e-3 * np.abs(want).max())
    assert not bad.any(), f"{bad.mean():.4%} mismatched, nan {np.isnan(got).mean():.4%}, max abs {np.nanmax(np.abs(got - want))}"
    # and the quantisation error itself stays at the e4m3 level against the unquantised product
    ref = X @ W.T
    assert np.abs(got - ref).max() < 0.12 * np.abs(ref).max()


# ---------------------------------------------------------------------------------------------
# W4A16 group 128
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("N,K", [(7, 688), (300, 5120), (64, 17408)])
def test_w4_quant_dequant_bit_exact(G, oracle, N, K):
    import torch
    r = rng(N + K)
    W = oracle.rb((r.standard_normal((N, K)) * 0.02).astype(np.float32))
    W[1] = 0.0
    W[2, :128] *= 1e-4
    packed = torch.zeros((N, K // 8), dtype=torch.int32, device="cuda")
    scales = torch.zeros((N, (K + 127) // 128), dtype=torch.float16, device="cuda")
    G.call("dcd_k_quant_w4_g128", G.dev(W, 1), packed, scales, N, K, None)
    wp, ws = oracle.k_quant_w4(W)
    assert np.array_equal(packed.cpu().numpy().view(np.uint32), wp)
    assert np.array_equal(scales.cpu().numpy().view(np.uint16), ws)
    out = torch.zeros((N, K), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_dequant_w4_g128", packed, scales, out, N, K, None)
    assert G.host(out).tobytes() == oracle.k_dequant_w4(wp, ws, K).tobytes()


@pytest.mark.parametrize("M,N,K,epi,with_resid", [(300, 512, 256, 0, False), (77, 96, 128, 0, False), (129, 264, 384, 0, True), (520, 1024, 5120, 1, False),
                                                   (2048, 5120, 1024, 0, True), (1000, 16480, 640, 0, False),
                                                   # the d3 projections at question-pass heights
                                                   (350, 34816, 5120, 1, False), (700, 5120, 17408, 0, True), (350, 14336, 5120, 0, False),
                                                   (700, 5120, 6144, 0, True)])
def test_gemm_w4a16_fused_bit_identical_to_dequant_plus_bf16_gemm(G, oracle, M, N, K, epi, with_resid):
    """The W4A16 GEMM that dequantises inside its producer warps gives the bits of the two-step route (int4 -> bf16 matrix, then the
    bf16 tensor-core GEMM): every weight is bf16(float(q - 8) * float(scale)) as dequant_w4a16_bf16 rounds it
    (native/kernels/kernels.cu:867-892) and each accumulator sees the same K steps in the same order. Ragged M and N, a weight
    row of zeros, groups with tiny values, the SwiGLU and the residual epilogues."""
    import torch
    r = rng(M + N + K)
    X = oracle.rb(r.standard_normal((M, K), dtype=np.float32))
    W = oracle.rb((r.standard_normal((N, K)) * 0.02).astype(np.float32))
    W[1] = 0.0
    W[2, :128] *= 1e-4
    dX, dW = G.dev(X, 1), G.dev(W, 1)
    packed = torch.zeros((N, K // 8), dtype=torch.int32, device="cuda")
    scales = torch.zeros((N, K // 128), dtype=torch.float16, device="cuda")
    G.call("dcd_k_quant_w4_g128", dW, packed, scales, N, K, None)
    Wd = torch.zeros((N, K), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_dequant_w4_g128", packed, scales, Wd, N, K, None)
    out_w = N // 2 if epi else N
    resid = G.dev(oracle.rb(r.standard_normal((M, out_w), dtype=np.float32)), 1) if with_resid else None
    want = torch.full((M, out_w), float("nan"), dtype=torch.bfloat16, device="cuda")
    err = G.devi([0])
    if with_resid:
        G.call("dcd_k_gemm_bf16_tc_resid", dX, Wd, resid, want, M, N, K, out_w, G.sm_count(), err, None)
    else:
        G.call("dcd_k_gemm_bf16_tc", dX, Wd, want, M, N, K, out_w, epi, G.sm_count(), err, None)
    pp = torch.zeros_like(packed)
    st = torch.zeros((K // 128, N), dtype=torch.float16, device="cuda")
    G.call("dcd_k_w4_repack", packed, scales, pp, st, N, K, None)
    got = torch.full((M, out_w), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_gemm_w4a16_tc", dX, pp, st, resid, got, M, N, K, out_w, epi, G.sm_count(), err, None)
    assert int(err.item()) == 0, "a bounded wait gave up inside the kernel"
    assert not torch.isnan(got.float()).any()
    again = torch.full((M, out_w), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_gemm_w4a16_tc", dX, pp, st, resid, again, M, N, K, out_w, epi, G.sm_count(), err, None)
    assert torch.equal(again, got), "two runs of the fused kernel differ"
    same = torch.equal(got, want)
    if not same:
        d = (got.float() - want.float()).abs()
        bad = (d > 0).nonzero()
        pytest.fail(f"{bad.shape[0]} of {got.numel()} differ; max abs {float(d.max())}; first at {bad[0].tolist()}: got {float(got[tuple(bad[0])])} want {float(want[tuple(bad[0])])}; "
                    f"rows {bad[:, 0].unique()[:16].tolist()} cols {bad[:, 1].unique()[:16].tolist()}")


# ---------------------------------------------------------------------------------------------
# NVFP4
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("glob", [1.0, 26880.0])
def test_nvfp4_rows_bit_exact(G, oracle, glob):
    import torch
    rows, K, stride = 7, 688, 704
    r = rng(51)
    scale = 1.0 if glob == 1.0 else 0.02
    xf = oracle.rb((r.standard_normal((rows, stride)) * scale * np.exp(r.uniform(-2, 2, (rows, 1)))).astype(np.float32))
    xf[2] = 0.0
    packed = torch.zeros((rows, K // 2), dtype=torch.uint8, device="cuda")
    scales = torch.zeros((rows, K // 16), dtype=torch.uint8, device="cuda")
    dx = G.dev(xf, 1)
    G.call("dcd_k_nvfp4_quant_rows", dx, stride, C.c_float(glob), packed, scales, rows, K, None)
    wp, ws, wd = oracle.k_nvfp4_rows(xf[:, :K], glob)
    assert np.array_equal(scales.cpu().numpy(), ws)
    assert np.array_equal(packed.cpu().numpy(), wp)
    out = torch.zeros((rows, K), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_nvfp4_dequant_rows", packed, scales, out, rows, K, None)
    assert G.host(out).tobytes() == wd.tobytes()          # e2m1 x e4m3 is exact in bf16
    assert oracle.rb(wd).tobytes() == wd.tobytes()
    out2 = torch.zeros((rows, K), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_nvfp4_fakequant_rows", dx, stride, C.c_float(glob), out2, rows, K, None)
    assert G.host(out2).tobytes() == wd.tobytes()


@pytest.mark.parametrize("dtype,nk,nv,lens", [(1, 16, 48, [73, 64, 89, 1, 31, 33]), (1, 2, 6, [128, 129, 200, 63, 65, 2]), (0, 2, 6, [70, 5, 64]),
                                              (1, 2, 4, [700])])
@pytest.mark.parametrize("entry", ["dcd_k_gdn_wy_tc", "dcd_k_gdn_chunked_tc"])  # WY form (inverse once per chunk) / substitution per column
def test_gdn_chunked_tcgen05_vs_oracle(G, oracle, dtype, nk, nv, lens, entry):
    """tcgen05 (kind::tf32, chunk 64) gated delta rule against the sequential oracle with the tolerances of
    the reference's chunked-vs-sequential test (native/tests/gdn_chunked.rs:109-111); lengths straddle
    the 64-token chunk, one case runs 11 chunks in a row. Also: batched == per-sequence, bit-exact."""
    dk = dv = 128
    T = sum(lens)
    conv, q, k, g, beta = _gdn_inputs(oracle, T, nk, nv, dk, dv, dtype)
    cd = conv.shape[1]
    seed = (0.05 * _host_data(nv * dk * dv, 1.0, 1.0)).reshape(nv, dk, dv).astype(np.float32)
    cu, _ = _pack(oracle, lens)
    out = G.empty((T, nv * dv), dtype)
    fin = G.devf(np.zeros((len(lens), nv, dk, dv)))
    err = G.devi([0])
    G.call(entry, G.devf(q), G.devf(k), G.dev(conv, dtype), cd, G.devf(g), G.devf(beta), G.devf(seed), fin, out, G.devi(cu), len(lens),
           T, nk, nv, dk, dv, err, dtype, None)
    assert int(err.item()) == 0
    rep = nv // nk
    got, gfin = G.host(out), G.host(fin)
    assert np.isfinite(got).all() and np.isfinite(gfin).all()
    worst = (0.0, 0.0, 0.0)
    for i, L in enumerate(lens):
        sl = slice(cu[i], cu[i + 1])
        v = conv[sl, 2 * nk * dk:].reshape(L, nv, dv)
        want, wstate = oracle.k_gdn_recurrent(np.repeat(q[sl], rep, 1), np.repeat(k[sl], rep, 1), v, g[sl], beta[sl], seed, bool(dtype))
        d = np.abs(got[sl].reshape(L, nv, dv) - want)
        ds = np.abs(gfin[i] - wstate).max()
        worst = (max(worst[0], d.max()), max(worst[1], d.mean()), max(worst[2], ds))
    print(entry, "vs sequential oracle: out max %.3g mean %.3g state max %.3g" % worst)
    assert worst[0] < 2e-2 and worst[1] < 2e-4 and worst[2] < 2e-3, worst
    for i, L in enumerate(lens[:3]):
        sl = slice(cu[i], cu[i + 1])
        o1 = G.empty((L, nv * dv), dtype)
        G.call(entry, G.devf(q[sl]), G.devf(k[sl]), G.dev(conv[sl], dtype), cd, G.devf(g[sl]), G.devf(beta[sl]), G.devf(seed), None, o1,
               G.devi([0, L]), 1, L, nk, nv, dk, dv, err, dtype, None)
        np.testing.assert_array_equal(G.host(o1), got[sl])
    assert int(err.item()) == 0


@pytest.mark.parametrize("tile_n", [128, 256, 1128, 1256])  # + 1000: scale copies on a thread of their own
@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (128, 128, 1024), (300, 776, 512), (2048, 5120, 1024), (77, 264, 5120), (130, 392, 768)])
def test_gemm_nvfp4_block_scaled_vs_dequantised_matmul(G, oracle, M, N, K, tile_n):
    """The native block-scaled FP4 GEMM against an f32 matmul of the dequantised operands (decode(code) * decode(scale)
    is exact in bf16, so the two differ only by the f32 summation order and the final bf16 rounding)."""
    import torch
    r = rng(M + 3 * N + 7 * K)
    X = oracle.rb((r.standard_normal((M, K)) * np.exp(r.uniform(-1, 1, (M, 1)))).astype(np.float32))
    W = oracle.rb((r.standard_normal((N, K)) * 0.05).astype(np.float32))
    dX, dW = G.dev(X, 1), G.dev(W, 1)
    xq = torch.zeros((M, K // 2), dtype=torch.uint8, device="cuda"); xs = torch.zeros((M, K // 16), dtype=torch.uint8, device="cuda")
    wq = torch.zeros((N, K // 2), dtype=torch.uint8, device="cuda"); ws = torch.zeros((N, K // 16), dtype=torch.uint8, device="cuda")
    wglobal = 2688.0 / float(np.abs(W).max())
    G.call("dcd_k_nvfp4_quant_rows", dX, K, C.c_float(1.0), xq, xs, M, K, None)
    G.call("dcd_k_nvfp4_quant_rows", dW, K, C.c_float(wglobal), wq, ws, N, K, None)
    xd = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda"); wd = torch.zeros((N, K), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_nvfp4_dequant_rows", xq, xs, xd, M, K, None)
    G.call("dcd_k_nvfp4_dequant_rows", wq, ws, wd, N, K, None)
    alpha = torch.tensor([1.0 / wglobal], dtype=torch.float32, device="cuda")
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    G.call("dcd_k_gemm_nvfp4_tc", xq, xs, wq, ws, out, M, N, K, N, alpha, G.sm_count(), err, tile_n, None)
    assert int(err.item()) == 0, "a bounded wait gave up inside the kernel"
    want = ((xd.float() @ wd.float().T) / wglobal).cpu().numpy()
    got = G.host(out)
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, want, rtol=1e-2, atol=1e-2 * float(np.abs(want).max()) / 8)


@pytest.mark.parametrize("M,N,K,tile_n", [(300, 768, 512, 1256), (300, 768, 512, 256), (300, 776, 512, 1128), (1100, 5120, 1024, 1256), (77, 512, 5120, 1256)])
def test_gemm_nvfp4_epilogues_bit_identical_to_the_separate_kernels(G, oracle, M, N, K, tile_n):
    """The residual epilogue equals the plain GEMM followed by a bf16 add; the SwiGLU + quantisation epilogue (256-wide tiles)
    equals the plain GEMM followed by dcd_k_nvfp4_swiglu_quant_tiled: same bytes of codes and of tiled scales."""
    import torch
    r = rng(M + N + K)
    X = (r.standard_normal((M, K)) * np.exp(r.uniform(-1, 1, (M, 1)))).astype(np.float32)
    W = (r.standard_normal((N, K)) * 0.05).astype(np.float32)
    xq = torch.zeros((M, K // 2), dtype=torch.uint8, device="cuda"); xs = torch.zeros((M, K // 16), dtype=torch.uint8, device="cuda")
    wq = torch.zeros((N, K // 2), dtype=torch.uint8, device="cuda"); ws = torch.zeros((N, K // 16), dtype=torch.uint8, device="cuda")
    wglobal = 2688.0 / float(np.abs(W).max())
    G.call("dcd_k_nvfp4_quant_rows", G.dev(X, 1), K, C.c_float(1.0), xq, xs, M, K, None)
    G.call("dcd_k_nvfp4_quant_rows", G.dev(W, 1), K, C.c_float(wglobal), wq, ws, N, K, None)

    def tiled(sc, rows):
        t = torch.zeros(((rows + 127) // 128) * (K // 64) * 512, dtype=torch.uint8, device="cuda")
        G.call("dcd_k_nvfp4_tile_scales", sc, t, rows, K, None)
        return t

    xt, wt = tiled(xs, M), tiled(ws, N)
    alpha = torch.tensor([1.0 / wglobal], dtype=torch.float32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    plain = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_gemm_nvfp4_tc_tiled", xq, xt, wq, wt, plain, M, N, K, N, alpha, G.sm_count(), err, tile_n, None, None, None, None)
    ref = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_gemm_nvfp4_tc", xq, xs, wq, ws, ref, M, N, K, N, alpha, G.sm_count(), err, tile_n, None)
    assert torch.equal(plain, ref)
    resid = torch.from_numpy(r.standard_normal((M, N)).astype(np.float32)).cuda().bfloat16()
    fused = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_gemm_nvfp4_tc_tiled", xq, xt, wq, wt, fused, M, N, K, N, alpha, G.sm_count(), err, tile_n, resid, None, None, None)
    assert torch.equal(fused, (resid.float() + plain.float()).bfloat16())
    inplace = resid.clone()  # the engine adds into the residual stream in place
    G.call("dcd_k_gemm_nvfp4_tc_tiled", xq, xt, wq, wt, inplace, M, N, K, N, alpha, G.sm_count(), err, tile_n, inplace, None, None, None)
    assert torch.equal(inplace, fused)
    if tile_n % 1000 == 256 and N % 256 == 0:
        inter = N // 2

        def buffers():
            return (torch.full((M, inter // 2), 0xAA, dtype=torch.uint8, device="cuda"),
                    torch.zeros(((M + 127) // 128) * (inter // 64) * 512, dtype=torch.uint8, device="cuda"))

        want_p, want_t = buffers()
        G.call("dcd_k_nvfp4_swiglu_quant_tiled", plain, N, want_p, want_t, M, inter, None)
        got_p, got_t = buffers()
        G.call("dcd_k_gemm_nvfp4_tc_tiled", xq, xt, wq, wt, None, M, N, K, inter, alpha, G.sm_count(), err, tile_n, None, got_p, got_t, None)
        torch.cuda.synchronize()
        assert torch.equal(got_p, want_p)
        assert torch.equal(got_t, want_t)
    assert int(err.item()) == 0


@pytest.mark.parametrize("rows,K", [(3, 128), (300, 512), (128, 5120)])
def test_nvfp4_scale_tiling_bit_exact(G, oracle, rows, K):
    import torch
    src = rng(rows + K).integers(0, 256, (rows, K // 16)).astype(np.uint8)
    want = oracle.nvfp4_scale_repack(src, K)
    tiled = torch.full((want.size,), 0xAA, dtype=torch.uint8, device="cuda")
    G.call("dcd_k_nvfp4_tile_scales", torch.from_numpy(src).cuda(), tiled, rows, K, None)
    assert np.array_equal(tiled.cpu().numpy(), want)


@pytest.mark.parametrize("rows,K,stride", [(7, 704, 704), (300, 512, 640), (129, 5120, 5120)])
def test_nvfp4_act_quant_tiled_matches_row_quantiser(G, oracle, rows, K, stride):
    """The fused activation quantiser (threshold compares, tiled scales) gives the codes and scales of the oracle bit for bit."""
    import torch
    r = rng(rows * 3 + K)
    xf = oracle.rb((r.standard_normal((rows, stride)) * np.exp(r.uniform(-12, 6, (rows, 1)))).astype(np.float32))
    xf[1] = 0.0
    xf[2, :40] = 0.0
    xf[3] = oracle.rb(np.float32(1e-30) * r.standard_normal(stride).astype(np.float32))
    wp, ws, _ = oracle.k_nvfp4_rows(xf[:, :K], 1.0)
    want_tiled = oracle.nvfp4_scale_repack(ws, K)
    packed = torch.zeros((rows, K // 2), dtype=torch.uint8, device="cuda")
    tiled = torch.zeros((want_tiled.size,), dtype=torch.uint8, device="cuda")
    G.call("dcd_k_nvfp4_quant_act_tiled", G.dev(xf, 1), stride, packed, tiled, rows, K, None)
    assert np.array_equal(packed.cpu().numpy(), wp)
    assert np.array_equal(tiled.cpu().numpy(), want_tiled)


def test_nvfp4_act_quant_on_ties_negative_zero_and_empty_groups(G, oracle):
    """The activation quantiser takes its codes from the e2m1 conversion instruction (round to nearest even); the reference's rule
    rounds a tie up and gives -0 no sign bit. Groups built to sit on every tie (c * scale for the seven midpoints, both signs), on
    the bf16 neighbours of the ties, on -0, and groups so small that their scale decodes to zero, bit for bit against the oracle."""
    import torch
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    scales = [2.0 ** -9, 2.0 ** -7 * 1.125, 0.4375, 1.0, 1.875, 52.0, 448.0 / 8]  # e4m3 values (subnormal, odd mantissas, large)

    def bf16_step(v, up):  # the neighbouring bf16 value
        bits = (np.float32(v).view(np.uint32) >> 16).astype(np.int64)
        return ((bits + (1 if up else -1)).astype(np.uint32) << 16).view(np.float32)

    groups = []
    for sc in scales:
        t = (ties * np.float32(sc)).astype(np.float32)
        assert oracle.rb(t).tobytes() == t.tobytes()  # the ties are bf16 values
        groups.append(np.concatenate([[6 * sc], t, [-0.0], -t]).astype(np.float32))
        groups.append(np.concatenate([[-6 * sc], bf16_step(t, True), [0.0], bf16_step(t, False)]).astype(np.float32))
        groups.append(np.concatenate([[6 * sc], -bf16_step(t, True), [-0.0], -bf16_step(t, False)]).astype(np.float32))
    tiny = np.float32(2.0 ** -12)
    groups.append(np.array([0.0, -0.0, tiny, -tiny] * 4, dtype=np.float32))          # scale decodes to zero: code 7 throughout
    groups.append(np.zeros(16, dtype=np.float32))
    groups.append(np.full(16, -0.0, dtype=np.float32))
    while len(groups) % 4:
        groups.append(np.arange(16, dtype=np.float32) - 7.5)
    xf = oracle.rb(np.concatenate(groups).reshape(-1, 64))
    rows, K = xf.shape
    wp, ws, _ = oracle.k_nvfp4_rows(xf, 1.0)
    want_tiled = oracle.nvfp4_scale_repack(ws, K)
    packed = torch.zeros((rows, K // 2), dtype=torch.uint8, device="cuda")
    tiled = torch.zeros((want_tiled.size,), dtype=torch.uint8, device="cuda")
    G.call("dcd_k_nvfp4_quant_act_tiled", G.dev(xf, 1), K, packed, tiled, rows, K, None)
    assert np.array_equal(tiled.cpu().numpy(), want_tiled)
    got = packed.cpu().numpy()
    assert np.array_equal(got, wp), f"first differing bytes at {np.argwhere(got != wp)[:8].tolist()}"


@pytest.mark.parametrize("rows,I", [(5, 256), (131, 1024)])
def test_nvfp4_swiglu_quant_tiled(G, oracle, rows, I):
    """SwiGLU fused with the NVFP4 quantiser against the two-step oracle (bf16 SwiGLU, then quantise). The kernel uses the
    fast exponential, so an activation may round to the neighbouring bf16 value now and then: nearly all codes and scales
    must agree exactly, and the dequantised result must stay within one NVFP4 step of the oracle's activation."""
    import torch
    r = rng(rows + I)
    gu = oracle.rb(r.standard_normal((rows, 2 * I)).astype(np.float32) * 2.0)
    gu[1] = 0.0
    g = gu.reshape(rows, I // 128, 2, 128)[:, :, 0].reshape(rows, I)
    u = gu.reshape(rows, I // 128, 2, 128)[:, :, 1].reshape(rows, I)
    act = oracle.rb(oracle.rb(g / (1 + np.exp(-g))) * u)
    wp, ws, wd = oracle.k_nvfp4_rows(act, 1.0)
    want_tiled = oracle.nvfp4_scale_repack(ws, I)
    packed = torch.zeros((rows, I // 2), dtype=torch.uint8, device="cuda")
    tiled = torch.zeros((want_tiled.size,), dtype=torch.uint8, device="cuda")
    G.call("dcd_k_nvfp4_swiglu_quant_tiled", G.dev(gu, 1), 2 * I, packed, tiled, rows, I, None)
    gp, gt = packed.cpu().numpy(), tiled.cpu().numpy()
    assert (gp == wp).mean() > 0.995 and (gt == want_tiled).mean() > 0.995
    # dequantise what the kernel wrote (scales back to row-major through the inverse of the tiling)
    lin = np.zeros_like(ws)
    for o in range(rows):
        for j in range(I // 16):
            lin[o, j] = gt[((j // 4) + (o // 128) * (I // 64)) * 512 + (o % 32) * 16 + ((o % 128) // 32) * 4 + (j % 4)]
    out = torch.zeros((rows, I), dtype=torch.bfloat16, device="cuda")
    G.call("dcd_k_nvfp4_dequant_rows", torch.from_numpy(gp).cuda(), torch.from_numpy(lin).cuda(), out, rows, I, None)
    step = np.repeat(np.abs(act).reshape(rows, I // 16, 16).max(-1), 16, axis=1) / 6.0 + 1e-9
    assert (np.abs(G.host(out) - act) <= 1.07 * step).all()   # half the 4..6 spacing times a scale rounded up by at most 1/16
