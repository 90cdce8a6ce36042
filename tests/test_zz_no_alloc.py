"""The allocation-free attention entry point, for hosts that may not call cudaMalloc on the thread that
drives the kernels (device-wide synchronisation) or that have no spare device memory to hand out.

It must give what dcd_k_attention_tc gives, call after call, although all calls share one built-in
scratch array that keeps whatever the previous call left in it. The file name sorts last so that a run
which stops at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(oracle, G, lens, S, seed):
    heads, kv, hd = 24, 4, 256
    T = sum(lens)
    r = np.random.Generator(np.random.PCG64(seed))
    R = oracle.rb
    d = {
        "q": G.dev(R(r.standard_normal((T, heads, hd), dtype=np.float32)), 1),
        "k": G.dev(R(r.standard_normal((T, kv * hd), dtype=np.float32)), 1),
        "v": G.dev(R(r.standard_normal((T, kv * hd), dtype=np.float32)), 1),
        "ks": G.dev(R(r.standard_normal((S, kv, hd), dtype=np.float32)), 1),
        "vs": G.dev(R(r.standard_normal((S, kv, hd), dtype=np.float32)), 1),
        "qg": G.dev(R(r.standard_normal((T, heads, 2 * hd), dtype=np.float32)), 1),
        "cu": G.devi(oracle.pack(lens, 0)[0]),
    }
    return d, T, heads, kv, hd


def _run(G, name, d, lens, S, T, heads, kv, hd, extra):
    import torch
    out = torch.full((T, heads, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    err = G.devi([0])
    args = [d["q"], d["k"], kv * hd, d["v"], kv * hd, d["ks"], d["vs"], S, d["qg"], heads * 2 * hd, out, d["cu"]]
    G.call(name, *args, *extra(len(lens), T, heads, kv, hd, err))
    assert int(err.item()) == 0
    return G.host(out)


def test_noalloc_attention_matches_the_ordinary_entry_point_twice_in_a_row(dcd, oracle):
    import torch
    import gpu_util as G
    from decidra_b200 import _lib
    msg = C.create_string_buffer(256)
    # two different batches back to back: the second is smaller, so the shared scratch still holds
    # entries of the first beyond what the second rewrites
    for lens, S, seed in (([130, 21, 22, 64, 65, 7, 300], 200, 1), ([33, 5], 70, 2)):
        d, T, heads, kv, hd = _case(oracle, G, lens, S, seed)
        tile_cu = G.devi(np.zeros(len(lens) + 1))
        want = _run(G, "dcd_k_attention_tc", d, lens, S, T, heads, kv, hd, lambda B, T_, h, k, e, err: [tile_cu, B, T_, h, k, e, err, None])
        got = _run(G, "dcd_k_attention_tc_noalloc", d, lens, S, T, heads, kv, hd, lambda B, T_, h, k, e, err: [B, T_, h, k, e, err, None, msg, 256])
        assert np.isfinite(want).all()
        np.testing.assert_allclose(got, want, rtol=2e-2, atol=8e-3)   # the tolerance of the attention parity tests
        assert np.array_equal(got, want)                               # and in fact the same bits: same kernels, same tiles
    # a batch beyond the built-in scratch is refused with a clear message, before any launch
    d, T, heads, kv, hd = _case(oracle, G, [4], 8, 3)
    rc = _lib.load().dcd_k_attention_tc_noalloc(C.c_void_p(d["q"].data_ptr()), C.c_void_p(d["k"].data_ptr()), kv * hd, C.c_void_p(d["v"].data_ptr()), kv * hd,
                                                C.c_void_p(d["ks"].data_ptr()), C.c_void_p(d["vs"].data_ptr()), 8, None, 0, C.c_void_p(d["q"].data_ptr()),
                                                C.c_void_p(d["cu"].data_ptr()), 4097, 4, heads, kv, hd, None, None, msg, 256)
    torch.cuda.synchronize()
    assert rc == 1 and b"4096" in msg.value and b"exceed" in msg.value
