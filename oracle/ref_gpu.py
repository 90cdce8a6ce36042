"""GPU oracle made of the REFERENCE's own CUDA code (test infrastructure; never imported by the product).

juanqui/decidra's engine is a Rust host (native/src/engine.rs) around three things that do all the
arithmetic: its own kernels (native/kernels/kernels.cu), a FlashInfer FA2 shim with a plain C ABI
(native/third_party/flashinfer/fi_prefill.cu) and cuBLAS. The Rust host cannot be built without a Rust
toolchain, but the other three run as they are: ``make -C oracle ref REF=<reference checkout>`` compiles
the two CUDA units for sm_100a with the reference's own flags (nothing is copied) into ``oracle/_ref/``:

    ref_kernels.cubin   native/kernels/kernels.cu   (-std=c++17 -O3 -fmad=false, native/build.rs:55-59)
    libfi_prefill.so    fi_prefill.cu               (native/build.rs:110-143)

This module replays the launch sequence of the Rust host over them, call by call, with the grid, block and
shared-memory values of the launch wrappers (native/src/kernels.rs) and with ``torch.matmul`` standing where
the host calls cuBLAS (bf16 operands, f32 accumulation, ``C = X . W^T``: Engine::gemm_core,
native/src/engine.rs:4321-4350; f32 readout: blas_gemm_f32, :3873-3901):

    RefEngine.capture_state               Engine::capture_state_mm            native/src/engine.rs:4616-4763
    RefEngine.readout_state_once_batch    state_once_batch_rows_inner         :4936-4987
    RefEngine.decision_logits_split       decision_logits_split/forward_split :4585-4601, 1459-1475
    _layer_single / _layer_batch          run_layer / run_layer_batch         :2705-2792, 1725-1788
    _full_attention / _full_attention_batch                                   :2887-3147, 1790-2142
    _gdn / _gdn_batch                                                         :3321-3694, 2144-2591
    _mlp                                                                      :2794-2885

Only d3-shaped models run here: the shim is compiled for 24 query heads, 4 KV heads, head_dim 256
(fi_prefill.cu:22-34) and the recurrent kernels for dk = dv = 128. Server defaults are followed
(src/config.rs:104-106): chunked TF32 gated delta rule from 16 tokens up, register recurrence for
question batches whose questions all have at most 256 tokens.

Weights come from the same seeded generator as everywhere else in this repository (integer hashing plus
one float multiply), evaluated here with torch integer ops on the GPU for the large matrices, so that the
three implementations (this one, the CPU restatement, the product) hold bit-identical tensors.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
CUBIN = _HERE / "_ref" / "ref_kernels.cubin"
FI_SO = _HERE / "_ref" / "libfi_prefill.so"

# tensor kinds of the seeded generator (same numbering as DCD_T_* / the CPU oracle)
T_EMBED, T_FINAL_NORM, T_READOUT = 0, 1, 2
T_INPUT_NORM, T_POST_NORM, T_GATE, T_UP, T_DOWN = 10, 11, 12, 13, 14
T_Q, T_K, T_V, T_O, T_QNORM, T_KNORM = 20, 21, 22, 23, 24, 25
T_IN_QKV, T_IN_Z, T_IN_B, T_IN_A, T_OUT, T_CONV, T_A_LOG, T_DT_BIAS, T_GNORM = 30, 31, 32, 33, 34, 35, 36, 37, 38

GDN_CHUNK_C, GDN_CHUNK_VC, CONV_TILE = 32, 64, 16  # native/src/kernels.rs:1696,1759,1761
GDN_CHUNK_MIN = 16                                # src/config.rs:105-106 (server default)


def available() -> bool:
    return CUBIN.exists() and FI_SO.exists()


# ------------------------------------------------------------------------------------------------
# the seeded generator on the GPU (normal tensors only; the small uniform ones come from the CPU oracle)
# ------------------------------------------------------------------------------------------------
_M64 = (1 << 64) - 1


def _mix64_py(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def _s64(u: int) -> int:
    return u - (1 << 64) if u >= (1 << 63) else u


def _lsr(z, s: int):
    return (z >> s) & ((1 << (64 - s)) - 1)


def _mix64_t(z):
    z = z + _s64(0x9E3779B97F4A7C15)
    z = (z ^ _lsr(z, 30)) * _s64(0xBF58476D1CE4E5B9)
    z = (z ^ _lsr(z, 27)) * _s64(0x94D049BB133111EB)
    return z ^ _lsr(z, 31)


def gen_normal_gpu(seed: int, layer: int, kind: int, n: int, std: float = 0.02, bf16: bool = True, device: str = "cuda"):
    """Element i = (sum of the eight 16-bit lanes of mix64(key+2i), mix64(key+2i+1) - 262140) * (std / 53509.919921)."""
    import torch
    key = _mix64_py(_mix64_py(seed) ^ ((layer + 1) * 64 + kind))
    c = float(np.float32(np.float64(np.float32(std)) / 53509.919921))
    out = torch.empty(n, dtype=torch.bfloat16 if bf16 else torch.float32, device=device)
    step = 1 << 24
    for first in range(0, n, step):
        m = min(step, n - first)
        i2 = torch.arange(first, first + m, dtype=torch.int64, device=device) * 2 + _s64(key)
        a, b = _mix64_t(i2), _mix64_t(i2 + 1)
        s = torch.zeros(m, dtype=torch.int64, device=device)
        for j in range(4):
            s += (a >> (16 * j)) & 0xFFFF
            s += (b >> (16 * j)) & 0xFFFF
        v = (s - 262140).to(torch.float32) * c
        out[first:first + m] = v.to(out.dtype)
    return out


# ------------------------------------------------------------------------------------------------
# the reference's compiled code
# ------------------------------------------------------------------------------------------------
class RefKernels:
    """ref_kernels.cubin through the CUDA driver API (what cudarc does for the Rust host, native/src/cuda.rs)."""

    # CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES values set at load time, native/src/kernels.rs:100-185
    SMEM_ATTR = {"gdn_chunked_tc": 90112, "gdn_chunked_tc_batched": 90112, "gdn_chunked_f32": 90112}

    def __init__(self):
        import torch
        from cuda.bindings import driver
        self.torch, self.drv = torch, driver
        torch.zeros(1, device="cuda")  # the primary context becomes current on this thread
        err, self.mod = driver.cuModuleLoad(str(CUBIN).encode())
        if err != driver.CUresult.CUDA_SUCCESS:
            raise RuntimeError(f"cuModuleLoad({CUBIN}) failed: {err}")
        self.fns = {}
        self.launches = 0

    def fn(self, name):
        drv = self.drv
        if name not in self.fns:
            err, f = drv.cuModuleGetFunction(self.mod, name.encode())
            if err != drv.CUresult.CUDA_SUCCESS:
                raise RuntimeError(f"{name}: {err}")
            if name in self.SMEM_ATTR:
                (err,) = drv.cuFuncSetAttribute(f, drv.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, self.SMEM_ATTR[name])
                if err != drv.CUresult.CUDA_SUCCESS:
                    raise RuntimeError(f"{name}: shared-memory attribute: {err}")
            self.fns[name] = f
        return self.fns[name]

    def launch(self, name, grid, block, smem, args, sync=False):
        """args: torch tensors (device pointers), Python floats (f32) or ints (i32)."""
        drv, torch = self.drv, self.torch
        vals, types = [], []
        for a in args:
            if isinstance(a, torch.Tensor):
                vals.append(a.data_ptr()); types.append(C.c_void_p)
            elif isinstance(a, float):
                vals.append(a); types.append(C.c_float)
            else:
                vals.append(int(a)); types.append(C.c_int)
        g = tuple(int(v) for v in grid) + (1,) * (3 - len(grid))
        b = tuple(int(v) for v in block) + (1,) * (3 - len(block))
        stream = drv.CUstream(torch.cuda.current_stream().cuda_stream)
        (err,) = drv.cuLaunchKernel(self.fn(name), g[0], g[1], g[2], b[0], b[1], b[2], int(smem), stream, (tuple(vals), tuple(types)), 0)
        if err != drv.CUresult.CUDA_SUCCESS:
            raise RuntimeError(f"launch {name}: {err}")
        self.launches += 1
        if sync:
            torch.cuda.synchronize()


class FlashInferShim:
    """libfi_prefill.so: the C entry points the Rust host binds with dlopen (native/src/flashinfer.rs:78-144)."""

    def __init__(self):
        import torch
        self.torch = torch
        self.lib = C.CDLL(str(FI_SO))
        P, I = C.c_void_p, C.c_int
        self.lib.fi_prefill_bf16_noncausal.argtypes = [P, P, P, P, I, P]
        self.lib.fi_prefill_bf16_custom.argtypes = [P, P, P, P, P, I, P]
        self.lib.fi_prefill_bf16_ext.argtypes = [P, P, P, P, I, I, P]
        self.lib.fi_prefill_bf16_ext_lse.argtypes = [P, P, P, P, P, I, I, P]
        self.calls = 0

    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def _check(self, rc, what):
        self.calls += 1
        if rc != 0:
            raise RuntimeError(f"FlashInfer {what} failed with cudaError {rc}")

    def prefill_noncausal(self, q, k, v, out, seq):        # fi_prefill.cu:100-110
        self._check(self.lib.fi_prefill_bf16_noncausal(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), seq, self._stream()), "noncausal prefill")

    def prefill_custom(self, q, k, v, mask, out, seq):     # fi_prefill.cu:130-140
        self._check(self.lib.fi_prefill_bf16_custom(q.data_ptr(), k.data_ptr(), v.data_ptr(), mask.data_ptr(), out.data_ptr(), seq, self._stream()), "custom-mask prefill")

    def prefill_ext(self, q, k, v, out, qo_len, kv_len):   # fi_prefill.cu:161-173; bounds of flashinfer.rs:526-531
        assert q.numel() >= qo_len * 24 * 256 and k.numel() >= kv_len * 4 * 256 and v.numel() >= kv_len * 4 * 256 and out.numel() >= qo_len * 24 * 256
        self._check(self.lib.fi_prefill_bf16_ext(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), qo_len, kv_len, self._stream()), "extended prefill")

    def prefill_ext_lse(self, q, k, v, out, lse, qo_len, kv_len):  # fi_prefill.cu:145-159
        self._check(self.lib.fi_prefill_bf16_ext_lse(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), qo_len, kv_len, self._stream()), "extended prefill with LSE")


def _elem_block(cols: int) -> int:  # native/src/kernels.rs:366-368
    p = 1
    while p < cols:
        p *= 2
    return min(max(p, 32), 256)


class RefState:
    """StateCache (native/src/engine.rs:533-543) as torch tensors."""

    def __init__(self, state_len, pos_end, n_layers):
        self.state_len, self.pos_end = state_len, pos_end
        self.kv = [None] * n_layers
        self.gdn_state = [None] * n_layers
        self.gdn_hist = [None] * n_layers

    def tensor(self, layer: int, what: int):
        """0 K [S,kv,hd], 1 V, 2 gdn_state [nv,dk,dv], 3 gdn_hist [3,conv_dim], flat f32 (None when the layer has none)."""
        t = None
        if what in (0, 1) and self.kv[layer] is not None:
            t = self.kv[layer][what]
        elif what == 2:
            t = self.gdn_state[layer]
        elif what == 3:
            t = self.gdn_hist[layer]
        return None if t is None else t.float().cpu().numpy().reshape(-1)


class RefEngine:
    """The reference engine's forward, replayed over its own compiled kernels."""

    def __init__(self, cfg, seed: int = 0, attn_split: bool = False, gdn_chunked: bool = True, progress=None):
        import torch
        from oracle import cpu_oracle as O
        if not available():
            raise RuntimeError("oracle/_ref is not built (make -C oracle ref REF=<reference checkout>)")
        if (cfg.heads, cfg.kv_heads, cfg.head_dim) != (24, 4, 256) or (cfg.gdn_dk, cfg.gdn_dv) != (128, 128) or cfg.dtype != 1:
            raise ValueError("the reference's FlashInfer shim and recurrent kernels are compiled for the d3 shape only (bf16, 24/4/256, dk = dv = 128)")
        self.torch, self.cfg = torch, cfg
        self.k = RefKernels()
        self.fi = FlashInferShim()
        self.attn_split = attn_split      # DECIDRA_ATTN_SPLIT (native/src/engine.rs:1908)
        self.gdn_chunked = gdn_chunked    # DECIDRA_NATIVE_GDN_CHUNKED (src/config.rs:104), default on
        self.taps = None                  # dict name -> tensor when enabled (Engine::set_dump names)
        H, I = cfg.hidden, cfg.intermediate
        self.H, self.I = H, I
        self.heads, self.kvh, self.hd = cfg.heads, cfg.kv_heads, cfg.head_dim
        self.nk, self.nv, self.dk, self.dv = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv
        self.conv_dim = 2 * self.nk * self.dk + self.nv * self.dv
        self.vd = self.nv * self.dv
        self.rhalf = cfg.rotary_dim // 2
        self.eps = float(cfg.rms_eps)

        def small(layer, kind, n, f32=False):
            a = O.gen_tensor(seed, layer, kind, n, bf16=True)
            t = torch.from_numpy(a).cuda()
            return t if f32 else t.to(torch.bfloat16)

        def big(layer, kind, rows, cols):
            return gen_normal_gpu(seed, layer, kind, rows * cols).view(rows, cols)

        self.embed = big(-1, T_EMBED, cfg.vocab, H)
        self.final_norm = small(-1, T_FINAL_NORM, H)
        self.readout = gen_normal_gpu(seed, -1, T_READOUT, cfg.readout_rows * H, bf16=False).view(cfg.readout_rows, H)
        self.layers = []
        qcols, kvcols = self.heads * 2 * self.hd, self.kvh * self.hd
        for i in range(cfg.num_layers):
            w = {"full": bool(cfg.layer_is_full[i]),
                 "input_norm": small(i, T_INPUT_NORM, H), "post_norm": small(i, T_POST_NORM, H),
                 "gate": big(i, T_GATE, I, H), "up": big(i, T_UP, I, H), "down": big(i, T_DOWN, H, I)}
            if w["full"]:
                w.update(q=big(i, T_Q, qcols, H), k=big(i, T_K, kvcols, H), v=big(i, T_V, kvcols, H), o=big(i, T_O, H, self.heads * self.hd),
                         q_norm=small(i, T_QNORM, self.hd), k_norm=small(i, T_KNORM, self.hd))
            else:
                w.update(in_qkv=big(i, T_IN_QKV, self.conv_dim, H), in_z=big(i, T_IN_Z, self.vd, H), in_b=big(i, T_IN_B, self.nv, H),
                         in_a=big(i, T_IN_A, self.nv, H), out=big(i, T_OUT, H, self.vd), conv=small(i, T_CONV, self.conv_dim * 4),
                         A_log=small(i, T_A_LOG, self.nv, f32=True), dt_bias=small(i, T_DT_BIAS, self.nv, f32=True), norm=small(i, T_GNORM, self.dv))
            self.layers.append(w)
            if progress:
                progress(i)
        self._rope_cache = None
        torch.cuda.synchronize()

    # ---- elementary launches (shapes: native/src/kernels.rs) -----------------------------------------
    def _bf(self, *shape):
        return self.torch.empty(shape, dtype=self.torch.bfloat16, device="cuda")

    def _f32(self, *shape):
        return self.torch.empty(shape, dtype=self.torch.float32, device="cuda")

    def _tap(self, name, t):
        if self.taps is not None:
            self.taps[name] = t.clone()

    def gemm(self, x, w):  # Engine::gemm_core, bf16 branch
        return self.torch.matmul(x, w.t())

    def rmsnorm(self, x, w, rows, cols):  # kernels.rs:407-435
        out = self._bf(rows, cols)
        blk = _elem_block(cols)
        self.k.launch("rmsnorm_bf16", (rows,), (blk,), blk * 4, [x, w, out, cols, self.eps, 1])
        return out

    def add_rmsnorm(self, x, mix, w, rows, cols):  # kernels.rs:372-405
        res, out = self._bf(rows, cols), self._bf(rows, cols)
        blk = _elem_block(cols)
        self.k.launch("add_rmsnorm_bf16", (rows,), (blk,), blk * 4, [x, mix, w, res, out, cols, self.eps, 1])
        return res, out

    def add(self, a, b):  # kernels.rs:467-484
        out = self.torch.empty_like(a)
        n = a.numel()
        self.k.launch("add_bf16", ((n + 255) // 256,), (256,), 0, [a, b, out, n])
        return out

    def rope_tables(self, positions):
        """Engine::rope_tables_positions (native/src/engine.rs:1619-1643): f32 powf/cosf/sinf on the host, rounded to bf16."""
        from oracle import cpu_oracle as O
        n = int(max(positions)) + 1
        if self._rope_cache is None or self._rope_cache[0].shape[0] < n:
            cos_t, sin_t = O.k_rope_tables(self.cfg.rotary_dim, float(self.cfg.rope_theta), max(n, 4096), True)
            self._rope_cache = (cos_t, sin_t)
        cos_t, sin_t = self._rope_cache
        idx = np.asarray(positions, dtype=np.int64)
        to = lambda a: self.torch.from_numpy(np.ascontiguousarray(a[idx])).cuda().to(self.torch.bfloat16)
        return to(cos_t), to(sin_t)

    def rope(self, q, k, cos, sin, T):  # kernels.rs:552-587: in place
        self.k.launch("rope_bf16", (T, self.heads + self.kvh), (self.rhalf,), 0, [q, k, cos, sin, self.heads, self.kvh, self.hd, self.rhalf])

    def _mlp(self, h2, T, w):  # Engine::mlp, native/src/engine.rs:2794-2885 (bf16 branch)
        gate, up = self.gemm(h2, w["gate"]), self.gemm(h2, w["up"])
        act = self._bf(T, self.I)
        n = T * self.I
        self.k.launch("silu_mul_bf16", ((n + 255) // 256,), (256,), 0, [gate, up, act, n])
        return self.gemm(act, w["down"])

    def _qkv_common(self, h, T, w, cos, sin):
        """q/gate/k/v projections, split, q/k norm, RoPE (common to :1790-1895 and :2887-3010)."""
        heads, kvh, hd = self.heads, self.kvh, self.hd
        qg, kk, vv = self.gemm(h, w["q"]), self.gemm(h, w["k"]), self.gemm(h, w["v"])
        q, gate = self._bf(T, heads * hd), self._bf(T, heads * hd)
        n = T * heads * hd
        self.k.launch("split_q_gate_bf16", ((n + 255) // 256,), (256,), 0, [qg, q, gate, T, heads, hd])
        qn = self.rmsnorm(q, w["q_norm"], T * heads, hd).view(T, heads * hd)
        kn = self.rmsnorm(kk, w["k_norm"], T * kvh, hd).view(T, kvh * hd)
        self.rope(qn, kn, cos, sin, T)
        return qn, kn, vv, gate

    def _gate_and_o(self, attn, gate, T, w):
        o = self.torch.empty_like(attn)
        n = attn.numel()
        self.k.launch("sigmoid_gate_bf16", ((n + 255) // 256,), (256,), 0, [attn, gate, o, n])
        self._tap("attn_gated", o)
        return self.gemm(o, w["o"])

    # ---- single sequence (capture, per-row reference) --------------------------------------------------
    def _full_attention(self, h, seq, w, cos, sin, split, io):
        qn, kn, vv, gate = self._qkv_common(h, seq, w, cos, sin)
        if io is not None:  # LayerIo{k_out, v_out}: post-RoPE K, raw V (native/src/engine.rs:3014-3025)
            io["k"], io["v"] = kn.clone(), vv.clone()
        attn = self._bf(seq, self.heads * self.hd)
        if split:
            from oracle import cpu_oracle as O
            mask = self.torch.from_numpy(O.block_cascade_mask(seq, split)).cuda()
            self.fi.prefill_custom(qn, kn, vv, mask, attn, seq)
        else:
            self.fi.prefill_noncausal(qn, kn, vv, attn, seq)
        self._tap("attn_out", attn)
        return self._gate_and_o(attn, gate, seq, w)

    def _gdn(self, h, seq, w, io):
        nk, nv, dk, dv, cd = self.nk, self.nv, self.dk, self.dv, self.conv_dim
        qkv = self.gemm(h, w["in_qkv"])
        if io is not None:  # last three pre-convolution rows, left-zero-padded (native/src/engine.rs:3348-3361)
            hist = self.torch.zeros(3, cd, dtype=self.torch.bfloat16, device="cuda")
            keep = min(seq, 3)
            hist[3 - keep:] = qkv[seq - keep:]
            io["hist"] = hist
        conv = self._bf(seq, cd)
        self.k.launch("conv1d_silu_tiled_bf16", ((cd + 255) // 256, (seq + CONV_TILE - 1) // CONV_TILE), (256,), 0, [qkv, w["conv"], conv, seq, cd])  # kernels.rs:1698-1722
        z, b, a = self.gemm(h, w["in_z"]), self.gemm(h, w["in_b"]), self.gemm(h, w["in_a"])
        qf, kf, vf = self._f32(seq, nv, dk), self._f32(seq, nv, dk), self._f32(seq, nv, dv)
        g, beta = self._f32(seq, nv), self._f32(seq, nv)
        self.k.launch("gdn_prepare", (seq, nv), (128,), 128 * 4, [conv, b, a, w["A_log"], w["dt_bias"], qf, kf, vf, g, beta, nk, nv, dk, dv])  # kernels.rs:1621-1668
        state = self.torch.zeros(nv, dk, dv, dtype=self.torch.float32, device="cuda")
        core = self._bf(seq, nv * dv)
        if self.gdn_chunked and seq >= GDN_CHUNK_MIN:  # native/src/engine.rs:3505-3560
            smem = (dk * GDN_CHUNK_VC + 2 * GDN_CHUNK_C * dk + 2 * GDN_CHUNK_C * GDN_CHUNK_VC + GDN_CHUNK_C * GDN_CHUNK_C + 4 * GDN_CHUNK_C) * 4
            self.k.launch("gdn_chunked_tc", (dv // GDN_CHUNK_VC, nv), (256,), smem, [qf, kf, vf, g, beta, state, core, seq, nv, dk, dv, GDN_CHUNK_VC])  # kernels.rs:1862-1915
        else:
            self.k.launch("gdn_recurrent", (nv,), (dv,), 0, [qf, kf, vf, g, beta, state, core, seq, nv, dk, dv])  # kernels.rs:1541-1596
        if io is not None:
            io["state"] = state
        self._tap("gdn_recurrent_out", core)
        normed = self._bf(seq, nv * dv)
        self.k.launch("rmsnorm_gated_bf16", (seq * nv,), (128,), 128 * 4, [core, z, w["norm"], normed, dv, self.eps])  # kernels.rs:438-465
        return self.gemm(normed, w["out"])

    def _layer_single(self, x, seq, w, cos, sin, split, io):
        H = self.H
        h = self.rmsnorm(x, w["input_norm"], seq, H)
        mix = self._full_attention(h, seq, w, cos, sin, split, io) if w["full"] else self._gdn(h, seq, w, io)
        x1, h2 = self.add_rmsnorm(x, mix, w["post_norm"], seq, H)
        return self.add(x1, self._mlp(h2, seq, w))

    def _embed(self, ids):  # kernels.rs:1117-1143; the host checks the vocabulary bound first (engine.rs:1364-1390)
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        if len(ids) and int(ids.max()) >= self.cfg.vocab:
            raise ValueError("token id out of range")
        d = self.torch.from_numpy(ids.astype(np.int64)).to(self.torch.int32).cuda()
        out = self._bf(len(ids), self.H)
        self.k.launch("embed_gather_bf16", (len(ids),), (256,), 0, [self.embed, d, out, len(ids), self.H])
        return out

    def capture_state(self, ids) -> RefState:
        seq = len(ids)
        if seq < 2:
            raise ValueError("a state block needs at least two tokens")
        st = RefState(seq, seq, self.cfg.num_layers)
        x = self._embed(ids)
        cos, sin = self.rope_tables(np.arange(seq))
        for i, w in enumerate(self.layers):
            io = {}
            x = self._layer_single(x, seq, w, cos, sin, 0, io)
            if w["full"]:
                st.kv[i] = (io["k"], io["v"])
            else:
                st.gdn_state[i], st.gdn_hist[i] = io["state"], io["hist"]
            self._tap(f"layer{i}", x)
        return st

    def _readout_rows(self, x, last_rows, B):
        """final norm over all rows, gather, bf16 -> f32, F32 GEMM (native/src/engine.rs:4968-4986)."""
        T = x.shape[0]
        h = self.rmsnorm(x, self.final_norm, T, self.H)
        idx = self.torch.tensor(last_rows, dtype=self.torch.int32, device="cuda")
        rows = self._bf(B, self.H)
        self.k.launch("gather_rows_bf16", (B, 16), (256,), 0, [h, idx, rows, B, self.H])  # kernels.rs:2175-2199
        prev = self.torch.backends.cuda.matmul.allow_tf32
        self.torch.backends.cuda.matmul.allow_tf32 = False
        out = self.torch.matmul(rows.float(), self.readout.t())
        self.torch.backends.cuda.matmul.allow_tf32 = prev
        return out.cpu().numpy()

    def decision_logits_split(self, ids, split: int) -> np.ndarray:
        seq = len(ids)
        if split == 0 or split >= seq:
            raise ValueError("block split out of range")
        x = self._embed(ids)
        cos, sin = self.rope_tables(np.arange(seq))
        for w in self.layers:
            x = self._layer_single(x, seq, w, cos, sin, split, None)
        return self._readout_rows(x, [seq - 1], 1)[0]

    # ---- the state-once question pass --------------------------------------------------------------------
    def _full_attention_batch(self, h, offs, lens, w, cos, sin, cache, layer):
        torch = self.torch
        heads, kvh, hd = self.heads, self.kvh, self.hd
        T = int(sum(lens))
        qn, kn, vv, gate = self._qkv_common(h, T, w, cos, sin)
        state_k, state_v = cache.kv[layer]
        S = cache.state_len
        attn = self._bf(T, heads * hd)
        if self.attn_split and S >= T:  # native/src/engine.rs:1908-1962
            state_out, private_out = self._bf(T, heads * hd), self._bf(T, heads * hd)
            state_lse, private_lse = self._f32(T, heads), self._f32(T, heads)
            self.fi.prefill_ext_lse(qn, state_k, state_v, state_out, state_lse, T, S)
            for o, l in zip(offs, lens):
                self.fi.prefill_ext_lse(qn[o:o + l], kn[o:o + l], vv[o:o + l], private_out[o:o + l], private_lse[o:o + l], l, l)
            n = T * heads * hd
            self.k.launch("merge_attn_lse_bf16", ((n + 1023) // 1024,), (1024,), 0, [state_out, state_lse, private_out, private_lse, attn, T, heads, hd])  # kernels.rs:2576-2604 (for_num_elems)
        else:  # native/src/engine.rs:1985-2042
            kv_cap = S + max(lens)
            k_all, v_all = self._bf(kv_cap, kvh * hd), self._bf(kv_cap, kvh * hd)
            k_all[:S].copy_(state_k)
            v_all[:S].copy_(state_v)
            for o, l in zip(offs, lens):
                k_all[S:S + l].copy_(kn[o:o + l])
                v_all[S:S + l].copy_(vv[o:o + l])
                self.fi.prefill_ext(qn[o:o + l], k_all, v_all, attn[o:o + l], l, S + l)
        self._tap("attn_out", attn)
        return self._gate_and_o(attn, gate, T, w)

    def _gdn_batch(self, h, offs, lens, d_offs, d_lens, w, cache, layer):
        torch = self.torch
        nk, nv, dk, dv, cd = self.nk, self.nv, self.dk, self.dv, self.conv_dim
        T, B = int(sum(lens)), len(lens)
        qkv = self.gemm(h, w["in_qkv"])
        conv = self._bf(T, cd)
        self.k.launch("conv1d_silu_seeded_tiled_bf16", ((cd + 255) // 256, (max(lens) + CONV_TILE - 1) // CONV_TILE, B), (256,), 0,
                      [qkv, cache.gdn_hist[layer], w["conv"], conv, d_offs, d_lens, B, cd])  # kernels.rs:2442-2477
        z, b, a = self.gemm(h, w["in_z"]), self.gemm(h, w["in_b"]), self.gemm(h, w["in_a"])
        compact = all(l <= 256 for l in lens)  # native/src/engine.rs:2229-2236, 2349-2354
        qk_heads = nk if compact else nv
        qf, kf, vf = self._f32(T, qk_heads, dk), self._f32(T, qk_heads, dk), self._f32(T, nv, dv)
        g, beta = self._f32(T, nv), self._f32(T, nv)
        args = [conv, b, a, w["A_log"], w["dt_bias"], qf, kf, vf, g, beta, nk, nv, dk, dv]
        core = self._bf(T, nv * dv)
        seed = cache.gdn_state[layer]
        if compact:
            self.k.launch("gdn_prepare_compact_bf16", (T, nv), (128,), 1024, args)  # kernels.rs:2530-2573
            self.k.launch("gdn_recurrent_reg_split_seeded_bf16", (nv * 2, B), (256,), 0,
                          [qf, kf, vf, g, beta, seed, core, d_offs, d_lens, nv, nk, dk, dv, 64, 2])  # kernels.rs:2480-2527
        else:
            self.k.launch("gdn_prepare", (T, nv), (128,), 128 * 4, args)
            if not (self.gdn_chunked and all(l >= GDN_CHUNK_MIN for l in lens)):
                raise NotImplementedError("mixed-length per-sequence GDN fallback (native/src/engine.rs:2463-2560) is not replayed")
            elems = nv * dk * dv
            state = self._f32(B, elems)
            self.k.launch("gdn_seed_broadcast", ((elems + 255) // 256, B), (256,), 0, [seed, state, elems])  # kernels.rs:1508-1539
            smem = (dk * 64 + 2 * GDN_CHUNK_C * dk + 2 * GDN_CHUNK_C * 64 + GDN_CHUNK_C * GDN_CHUNK_C + 4 * GDN_CHUNK_C) * 4
            self.k.launch("gdn_chunked_tc_batched", (dv // 64, nv, B), (256,), smem,
                          [qf, kf, vf, g, beta, state, core, d_offs, d_lens, B, nv, dk, dv, 64])  # kernels.rs:1927-1986
        self._tap("gdn_recurrent_out", core)
        normed = self._bf(T, nv * dv)
        self.k.launch("rmsnorm_gated_bf16", (T * nv,), (128,), 128 * 4, [core, z, w["norm"], normed, dv, self.eps])
        return self.gemm(normed, w["out"])

    def readout_state_once_batch(self, cache: RefState, questions, max_rows: int = 64, max_keys: int = 1 << 18, max_scores: int = 1 << 27) -> np.ndarray:
        """Engine::state_once_batch_rows (native/src/engine.rs:4866-4934): stable sort by length, greedy chunks under the
        row / key / score caps (defaults of :4870-4881), one pass per chunk, rows scattered back to input order."""
        from oracle import cpu_oracle as O
        if not len(questions):
            raise ValueError("empty state-once question batch")
        lens = [len(q) for q in questions]
        if min(lens) == 0:
            raise ValueError("batch item has no tokens")
        n, order, chunk_of = O.plan_chunks(lens, cache.state_len, max_rows, max_keys, max_scores)
        if n <= 1:
            return self._question_pass(cache, questions)
        out = np.zeros((len(questions), self.cfg.readout_rows), dtype=np.float32)
        for ch in range(n):
            idx = [int(i) for i in order if chunk_of[i] == ch]
            out[idx] = self._question_pass(cache, [questions[i] for i in idx])
        return out

    def _question_pass(self, cache: RefState, questions) -> np.ndarray:
        """state_once_batch_rows_inner (native/src/engine.rs:4936-4987)."""
        torch = self.torch
        lens = [len(q) for q in questions]
        offs = [0]
        for l in lens[:-1]:
            offs.append(offs[-1] + l)
        T, B, H = sum(lens), len(lens), self.H
        d_offs = torch.tensor(offs, dtype=torch.int32, device="cuda")
        d_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
        # BatchInfo::positions (native/src/engine.rs:726-734): every question restarts at pos_end
        positions = np.concatenate([cache.pos_end + np.arange(l) for l in lens])
        cos, sin = self.rope_tables(positions)
        x = self._embed(np.concatenate([np.asarray(q, dtype=np.uint32) for q in questions]))
        for i, w in enumerate(self.layers):
            h = self.rmsnorm(x, w["input_norm"], T, H)
            mix = (self._full_attention_batch(h, offs, lens, w, cos, sin, cache, i) if w["full"]
                   else self._gdn_batch(h, offs, lens, d_offs, d_lens, w, cache, i))
            x1, h2 = self.add_rmsnorm(x, mix, w["post_norm"], T, H)
            x = self.add(x1, self._mlp(h2, T, w))
            self._tap(f"layer{i}", x)
        return self._readout_rows(x, [o + l - 1 for o, l in zip(offs, lens)], B)
