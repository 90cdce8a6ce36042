"""Pins the CPU oracle against the reference's OWN kernels on the GPU.

`oracle/Makefile ref` compiles the reference's `native/kernels/kernels.cu` for sm_100a (with its own flags,
`-fmad=false` included) straight from the reference checkout into `oracle/_ref/ref_kernels.cubin`; nothing
is copied. This file loads that cubin through the CUDA driver API, launches the reference kernels with the
grid/block/shared-memory values of the reference's launch wrappers (`native/src/kernels.rs`) on seeded
inputs, and requires the oracle (the CPU restatement every parity test is judged against) to reproduce
their outputs: bit-exact where the arithmetic is order-free, within one bf16 ulp (and >= 99 % identical)
where only the order of an f32 reduction or a libm-vs-device `expf` differs.

The cubin travels with the repository snapshot; where it is absent the tests skip."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
CUBIN = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "ref_kernels.cubin"


class Ref:
    def __init__(self):
        import torch
        from cuda.bindings import driver
        self.torch, self.drv = torch, driver
        torch.zeros(1, device="cuda")  # primary context current on this thread
        err, self.mod = driver.cuModuleLoad(str(CUBIN).encode())
        assert err == driver.CUresult.CUDA_SUCCESS, err
        self.fns = {}

    def launch(self, name, grid, block, smem, args):
        """args: list of torch tensors (passed as pointers), ints (c_int) or floats (c_float)."""
        drv, torch = self.drv, self.torch
        if name not in self.fns:
            err, fn = drv.cuModuleGetFunction(self.mod, name.encode())
            assert err == drv.CUresult.CUDA_SUCCESS, (name, err)
            self.fns[name] = fn
        vals, types = [], []
        for a in args:
            if isinstance(a, torch.Tensor):
                vals.append(a.data_ptr()); types.append(C.c_void_p)
            elif isinstance(a, float):
                vals.append(a); types.append(C.c_float)
            else:
                vals.append(int(a)); types.append(C.c_int)
        g = tuple(grid) + (1,) * (3 - len(grid))
        b = tuple(block) + (1,) * (3 - len(block))
        stream = drv.CUstream(torch.cuda.current_stream().cuda_stream)
        (err,) = drv.cuLaunchKernel(self.fns[name], g[0], g[1], g[2], b[0], b[1], b[2], smem, stream, (tuple(vals), tuple(types)), 0)
        assert err == drv.CUresult.CUDA_SUCCESS, (name, err)
        torch.cuda.synchronize()


@pytest.fixture(scope="module")
def ref():
    if not CUBIN.exists():
        pytest.skip("oracle/_ref/ref_kernels.cubin not built (needs the reference checkout: make -C oracle ref)")
    return Ref()


@pytest.fixture(scope="module")
def G(dcd):
    import gpu_util
    return gpu_util


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def close_bf16(got, want, min_exact=0.99):
    """Within one bf16 ulp everywhere (values below 1e-5 in magnitude: within 1e-7 absolute) and identical
    almost everywhere."""
    np.testing.assert_allclose(got, want, rtol=8e-3, atol=1e-7)
    exact = float((got == want).mean())
    assert exact >= min_exact, exact
    return exact


def elem_block(cols):  # native/src/kernels.rs:366-368
    p = 1
    while p < cols:
        p *= 2
    return min(max(p, 32), 256)


@pytest.mark.parametrize("rows,cols", [(37, 5120), (96, 256)])
def test_oracle_vs_reference_norm_kernels(ref, G, oracle, rows, cols):
    r = rng(rows + cols)
    x = oracle.rb(r.standard_normal((rows, cols), dtype=np.float32) * 3)
    m = oracle.rb(r.standard_normal((rows, cols), dtype=np.float32))
    w = oracle.rb(r.standard_normal(cols, dtype=np.float32) * 0.1)
    blk = elem_block(cols)
    dx, dm, dw = G.dev(x, 1), G.dev(m, 1), G.dev(w, 1)
    out = G.empty((rows, cols), 1)
    ref.launch("rmsnorm_bf16", (rows,), (blk,), blk * 4, [dx, dw, out, cols, 1e-6, 1])
    close_bf16(G.host(out), oracle.k_rmsnorm(x, w, 1e-6, True, True))
    res = G.empty((rows, cols), 1)
    ref.launch("add_rmsnorm_bf16", (rows,), (blk,), blk * 4, [dx, dm, dw, res, out, cols, 1e-6, 1])
    wres, wout = oracle.k_add_rmsnorm(x, m, w, 1e-6, True)
    assert G.host(res).tobytes() == wres.tobytes()
    close_bf16(G.host(out), wout)


def test_oracle_vs_reference_gated_norm_and_elementwise(ref, G, oracle):
    rows, cols = 48 * 5, 128
    r = rng(5)
    x = oracle.rb(r.standard_normal((rows, cols), dtype=np.float32))
    z = oracle.rb(r.standard_normal((rows, cols), dtype=np.float32) * 2)
    w = oracle.rb(1 + r.standard_normal(cols, dtype=np.float32) * 0.05)
    out = G.empty((rows, cols), 1)
    ref.launch("rmsnorm_gated_bf16", (rows,), (128,), 128 * 4, [G.dev(x, 1), G.dev(z, 1), G.dev(w, 1), out, cols, 1e-6])  # kernels.rs rmsnorm_gated: block 128
    close_bf16(G.host(out), oracle.k_rmsnorm_gated(x, z, w, 1e-6, True), 0.985)
    n = rows * cols
    g, u = x.reshape(-1) * 3, z.reshape(-1)
    g = oracle.rb(g)
    o = G.empty((n,), 1)
    ref.launch("silu_mul_bf16", ((n + 255) // 256,), (256,), 0, [G.dev(g, 1), G.dev(u, 1), o, n])
    close_bf16(G.host(o), oracle.rb(oracle.rb(g / (1 + np.exp(-g))) * u), 0.995)
    ref.launch("sigmoid_gate_bf16", ((n + 255) // 256,), (256,), 0, [G.dev(u, 1), G.dev(g, 1), o, n])
    close_bf16(G.host(o), oracle.rb(u * oracle.rb(1 / (1 + np.exp(-g)))), 0.995)
    ref.launch("add_bf16", ((n + 255) // 256,), (256,), 0, [G.dev(g, 1), G.dev(u, 1), o, n])
    assert G.host(o).tobytes() == oracle.rb(g + u).tobytes()


def test_oracle_vs_reference_rope(ref, G, oracle):
    T, nq, nk, hd, rot, theta = 19, 24, 4, 256, 64, 1e7
    r = rng(7)
    q = oracle.rb(r.standard_normal((T, nq, hd), dtype=np.float32))
    k = oracle.rb(r.standard_normal((T, nk, hd), dtype=np.float32))
    pos = (2048 + np.arange(T)).astype(np.int32)
    cos_t, sin_t = oracle.k_rope_tables(rot, theta, 2048 + T, True)
    dq, dk_ = G.dev(q, 1), G.dev(k, 1)
    ref.launch("rope_bf16", (T, nq + nk), (rot // 2,), 0, [dq, dk_, G.dev(cos_t[pos], 1), G.dev(sin_t[pos], 1), nq, nk, hd, rot // 2])
    assert G.host(dq).tobytes() == oracle.k_rope(q, pos, rot, theta, True).tobytes()
    assert G.host(dk_).tobytes() == oracle.k_rope(k, pos, rot, theta, True).tobytes()


def test_oracle_vs_reference_conv_and_gdn(ref, G, oracle):
    nk, nv, dk, dv = 16, 48, 128, 128
    cd = 2 * nk * dk + nv * dv
    lens = [17, 1, 40]
    T = sum(lens)
    r = rng(9)
    x = oracle.rb(r.standard_normal((T, cd), dtype=np.float32))
    hist = oracle.rb(r.standard_normal((3, cd), dtype=np.float32))
    w = oracle.rb(r.uniform(-0.5, 0.5, (cd, 4)).astype(np.float32))
    offs = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    out = G.empty((T, cd), 1)
    # kernels.rs:2442-2477: grid (ceil(ch/256), ceil(maxL/16), B), block 256
    ref.launch("conv1d_silu_seeded_tiled_bf16", ((cd + 255) // 256, (max(lens) + 15) // 16, len(lens)), (256,), 0,
               [G.dev(x, 1), G.dev(hist, 1), G.dev(w, 1), out, G.devi(offs), G.devi(lens), len(lens), cd])
    conv = np.concatenate([oracle.k_conv1d(x[o:o + n], hist, w, True) for o, n in zip(offs, lens)])
    close_bf16(G.host(out), conv, 0.995)

    b = oracle.rb(r.standard_normal((T, nv), dtype=np.float32) * 2)
    a = oracle.rb(r.standard_normal((T, nv), dtype=np.float32))
    A_log = r.uniform(0, 2.77, nv).astype(np.float32)
    dtb = r.uniform(-6.9, -2.3, nv).astype(np.float32)
    qf, kf, vf = G.devf(np.zeros((T, nv, dk))), G.devf(np.zeros((T, nv, dk))), G.devf(np.zeros((T, nv, dv)))
    g, beta = G.devf(np.zeros((T, nv))), G.devf(np.zeros((T, nv)))
    ref.launch("gdn_prepare", (T, nv), (128,), 128 * 4, [G.dev(conv, 1), G.dev(b, 1), G.dev(a, 1), G.devf(A_log), G.devf(dtb), qf, kf, vf, g, beta, nk, nv, dk, dv])
    wq, wk, wv, wg, wb = oracle.k_gdn_prepare(conv, b, a, A_log, dtb, nk, nv, dk, dv, True)
    np.testing.assert_allclose(G.host(qf), wq, rtol=2e-6, atol=1e-9)
    np.testing.assert_allclose(G.host(kf), wk, rtol=2e-6, atol=1e-9)
    assert G.host(vf).tobytes() == wv.tobytes()
    np.testing.assert_allclose(G.host(g), wg, rtol=1e-5, atol=1e-9)
    close_bf16(G.host(beta), wb, 0.99)

    # scalar recurrence (kernels.cu:834-865): same order as the oracle -> the f32 state agrees to rounding of expf
    L = lens[2]
    sl = slice(int(offs[2]), int(offs[2]) + L)
    seed = (0.05 * r.standard_normal((nv, dk, dv))).astype(np.float32)
    state = G.devf(seed)
    o1 = G.empty((L, nv, dv), 1)
    ref.launch("gdn_recurrent", (nv,), (dv,), 0, [G.devf(wq[sl]), G.devf(wk[sl]), G.devf(wv[sl]), G.devf(wg[sl]), G.devf(wb[sl]), state, o1, L, nv, dk, dv])
    want, wstate = oracle.k_gdn_recurrent(wq[sl], wk[sl], wv[sl], wg[sl], wb[sl], seed, True)
    close_bf16(G.host(o1), want, 0.99)
    np.testing.assert_allclose(G.host(state), wstate, rtol=1e-4, atol=1e-6)
    # production seeded kernel (kernels.cu:2245-2300; kernels.rs:2480-2527: grid (heads*chunks, B), block vc*4)
    rep = nv // nk
    o2 = G.empty((T, nv, dv), 1)
    ref.launch("gdn_recurrent_reg_split_seeded_bf16", (nv * 2, len(lens)), (256,), 0,
               [G.devf(wq[:, ::rep]), G.devf(wk[:, ::rep]), G.devf(wv), G.devf(wg), G.devf(wb), G.devf(seed), o2, G.devi(offs), G.devi(lens), nv, nk, dk, dv, 64, 2])
    got2 = G.host(o2)
    for o, n in zip(offs, lens):
        want, _ = oracle.k_gdn_recurrent(wq[o:o + n], wk[o:o + n], wv[o:o + n], wg[o:o + n], wb[o:o + n], seed, True)
        d = np.abs(got2[o:o + n] - want)
        assert d.max() < 2e-2 and d.mean() < 2e-4, (d.max(), d.mean())


def test_oracle_vs_reference_quantisers(ref, G, oracle):
    import torch
    rows, k = 11, 5120
    r = rng(13)
    x = oracle.rb((r.standard_normal((rows, k)) * np.exp(r.uniform(-4, 3, (rows, 1)))).astype(np.float32))
    codes = torch.zeros((rows, k), dtype=torch.uint8, device="cuda")
    scales = G.devf(np.zeros(rows))
    ref.launch("quant_fp8_per_token_bf16", (rows,), (256,), 256 * 4, [G.dev(x, 1), codes, scales, rows, k, 1.0])
    wc, ws = oracle.k_quant_fp8_rows(x)
    assert G.host(scales).tobytes() == ws.tobytes()
    assert np.array_equal(codes.cpu().numpy(), wc)
    # W4A16 dequantisation (kernels.cu:867-892) with group 128, symmetric zero-point 8; the reference reads bf16
    # scales, so use scales that are exact in both bf16 and fp16
    N, K = 24, 640
    W = oracle.rb((r.standard_normal((N, K)) * 0.02).astype(np.float32))
    packed, sc16 = oracle.k_quant_w4(W)
    sc = (np.ldexp(1.0 + r.integers(0, 8, sc16.shape) / 8.0, -r.integers(5, 9, sc16.shape))).astype(np.float32)  # 3 mantissa bits
    sc16 = sc.astype(np.float16).view(np.uint16)
    zp = torch.full(((N + 7) // 8, K // 128), -2004318072, dtype=torch.int32, device="cuda")  # 0x88888888
    out = torch.zeros((N, K), dtype=torch.bfloat16, device="cuda")
    n = N * K
    ref.launch("dequant_w4a16_bf16", ((n + 255) // 256,), (256,), 0,
               [torch.from_numpy(packed.view(np.int32)).cuda(), G.dev(sc, 1), zp, out, N, K, 128])
    assert G.host(out).tobytes() == oracle.k_dequant_w4(packed, sc16, K).tobytes()
    # the checkpoint form of the same kernel: asymmetric zero points (one nibble per output row and group), groups of
    # 64 and 128, arbitrary bf16 scales, an output count that is not a multiple of 8
    for N, K, gs in ((21, 384, 64), (40, 640, 128)):
        groups = K // gs
        pk = r.integers(0, 2**32, (N, K // 8), dtype=np.uint64).astype(np.uint32).view(np.int32)
        sc = oracle.rb(r.uniform(0.001, 0.01, (N, groups)).astype(np.float32))
        zpw = r.integers(0, 2**32, ((N + 7) // 8, groups), dtype=np.uint64).astype(np.uint32).view(np.int32)
        out = torch.zeros((N, K), dtype=torch.bfloat16, device="cuda")
        ref.launch("dequant_w4a16_bf16", ((N * K + 255) // 256,), (256,), 0,
                   [torch.from_numpy(pk).cuda(), G.dev(sc, 1), torch.from_numpy(zpw).cuda(), out, N, K, gs])
        assert G.host(out).tobytes() == oracle.ct_w4_dequant(pk, sc, zpw, K, gs).tobytes()
