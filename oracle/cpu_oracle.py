"""ctypes binding of the CPU oracle (``oracle/decidra_oracle.cpp``).

Test infrastructure only: imported by ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``. The product package never
imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "liboracle.so"


class OrcConfig(C.Structure):
    """Field order mirrors ``orc_config`` in decidra_oracle.cpp."""

    _fields_ = [
        ("num_layers", C.c_int32),
        ("hidden", C.c_int32),
        ("heads", C.c_int32),
        ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("rotary_dim", C.c_int32),
        ("rope_theta", C.c_float),
        ("gdn_k_heads", C.c_int32),
        ("gdn_v_heads", C.c_int32),
        ("gdn_dk", C.c_int32),
        ("gdn_dv", C.c_int32),
        ("conv_kernel", C.c_int32),
        ("intermediate", C.c_int32),
        ("vocab", C.c_int32),
        ("readout_rows", C.c_int32),
        ("rms_eps", C.c_float),
        ("dtype", C.c_int32),
        ("layer_is_full", C.c_uint8 * 256),
    ]


def build(force: bool = False) -> Path:
    """Compile liboracle.so with the Makefile beside this file (g++ only, no GPU)."""
    src = _HERE / "decidra_oracle.cpp"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        L = C.CDLL(str(_LIB_PATH))
        P = C.c_void_p
        fp = C.POINTER(C.c_float)
        L.orc_create.restype = P
        L.orc_create.argtypes = [C.POINTER(OrcConfig), C.c_uint64]
        L.orc_create_lazy.restype = P
        L.orc_create_lazy.argtypes = [C.POINTER(OrcConfig), C.c_uint64]
        L.orc_destroy.argtypes = [P]
        L.orc_state_free.argtypes = [P]
        L.orc_state_len.argtypes = [P]
        L.orc_state_pos_end.argtypes = [P]
        L.orc_tap_enable.argtypes = [P, C.c_int]
        L.orc_tap_size.restype = C.c_int64
        L.orc_tap_size.argtypes = [P, C.c_char_p]
        L.orc_tap_read.argtypes = [P, C.c_char_p, fp]
        L.orc_capture_state.argtypes = [P, C.POINTER(C.c_uint32), C.c_int, C.POINTER(P)]
        L.orc_readout_state_once.argtypes = [P, P, C.POINTER(C.c_uint32), C.POINTER(C.c_int32), C.c_int, fp]
        L.orc_decision_logits_split.argtypes = [P, C.POINTER(C.c_uint32), C.c_int, C.c_int, fp]
        L.orc_state_tensor.restype = C.c_int64
        L.orc_state_tensor.argtypes = [P, C.c_int, C.c_int, fp]
        L.orc_state_zero.argtypes = [P, C.c_int, C.c_int]
        L.orc_gen_tensor.argtypes = [C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_uint64, fp]
        L.orc_k_rb.restype = C.c_float
        L.orc_k_rb.argtypes = [C.c_float]
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _ip(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def _up(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_uint32))


def make_config(**kw) -> OrcConfig:
    c = OrcConfig()
    full = kw.pop("layer_is_full")
    for k, v in kw.items():
        setattr(c, k, v)
    for i, f in enumerate(full):
        c.layer_is_full[i] = int(f)
    return c


def gen_tensor(seed: int, layer: int, kind: int, n: int, bf16: bool, first: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_gen_tensor(seed, layer, kind, int(bf16), first, n, _fp(out))
    return out


class OracleState:
    def __init__(self, handle):
        self.h = handle

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_state_free(self.h)
            self.h = None

    @property
    def state_len(self) -> int:
        return lib().orc_state_len(self.h)

    @property
    def pos_end(self) -> int:
        return lib().orc_state_pos_end(self.h)

    def tensor(self, layer: int, what: int):
        n = lib().orc_state_tensor(self.h, layer, what, None)
        if n < 0:
            return None
        out = np.empty(n, dtype=np.float32)
        lib().orc_state_tensor(self.h, layer, what, _fp(out))
        return out

    def zero(self, layer: int, what: int) -> None:
        lib().orc_state_zero(self.h, layer, what)


class Oracle:
    """CPU restatement of Engine::{capture_state, readout_state_once_batch, decision_logits_split}."""

    def __init__(self, cfg: OrcConfig, seed: int = 0, lazy: bool = False):
        """lazy: generate the weights of a layer when a pass reaches it and drop them after it (deep models)."""
        self.cfg = cfg
        self.h = (lib().orc_create_lazy if lazy else lib().orc_create)(C.byref(cfg), seed)

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_destroy(self.h)
            self.h = None

    def capture_state(self, ids) -> OracleState:
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        out = C.c_void_p()
        rc = lib().orc_capture_state(self.h, _up(ids), len(ids), C.byref(out))
        if rc:
            raise ValueError(f"oracle capture_state failed rc={rc}")
        return OracleState(out)

    def readout_state_once_batch(self, state: OracleState, questions) -> np.ndarray:
        lens = np.array([len(q) for q in questions], dtype=np.int32)
        flat = np.ascontiguousarray(np.concatenate([np.asarray(q, dtype=np.uint32) for q in questions]) if len(questions) else np.zeros(0, np.uint32))
        out = np.empty((len(questions), self.cfg.readout_rows), dtype=np.float32)
        rc = lib().orc_readout_state_once(self.h, state.h, _up(flat), _ip(lens), len(questions), _fp(out))
        if rc:
            raise ValueError(f"oracle readout failed rc={rc}")
        return out

    def decision_logits_split(self, ids, split: int) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        out = np.empty(self.cfg.readout_rows, dtype=np.float32)
        rc = lib().orc_decision_logits_split(self.h, _up(ids), len(ids), split, _fp(out))
        if rc:
            raise ValueError(f"oracle decision_logits_split failed rc={rc}")
        return out

    def set_precision(self, precision: int, fp8_min_rows: int = 0) -> None:
        """precision 2 = FP8 GEMMs in question passes of >= fp8_min_rows rows (default 512)."""
        lib().orc_set_precision(self.h, precision, fp8_min_rows)

    def tap_enable(self, on: bool = True) -> None:
        lib().orc_tap_enable(self.h, int(on))

    def tap(self, name: str):
        n = lib().orc_tap_size(self.h, name.encode())
        if n < 0:
            return None
        out = np.empty(n, dtype=np.float32)
        lib().orc_tap_read(self.h, name.encode(), _fp(out))
        return out


# ----- kernel-level helpers -------------------------------------------------

def rb(x: np.ndarray) -> np.ndarray:
    """Round float32 through bf16 (RNE), vectorised numpy twin of the C helper."""
    x = _f32(x)
    u = x.view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32).reshape(x.shape)


def k_gemm(X, W, bf16: bool) -> np.ndarray:
    X, W = _f32(X), _f32(W)
    T, K = X.shape
    N = W.shape[0]
    out = np.empty((T, N), dtype=np.float32)
    lib().orc_k_gemm(_fp(X), _fp(W), _fp(out), T, N, K, int(bf16))
    return out


def k_quant_fp8_rows(x, clip: float = 1.0):
    """Returns (e4m3 codes uint8 [rows, cols], scales f32 [rows])."""
    x = _f32(x)
    codes = np.empty(x.shape, dtype=np.uint8)
    scales = np.empty(x.shape[0], dtype=np.float32)
    lib().orc_k_quant_fp8_rows(_fp(x), x.shape[0], x.shape[1], C.c_float(clip), codes.ctypes.data_as(C.POINTER(C.c_uint8)), _fp(scales))
    return codes, scales


def e4m3_to_f32(codes) -> np.ndarray:
    lib().orc_k_e4m3_to_f32.restype = C.c_float
    lib().orc_k_e4m3_to_f32.argtypes = [C.c_uint8]
    table = np.array([lib().orc_k_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)
    return table[np.asarray(codes, dtype=np.uint8)]


def k_gemm_fp8(X, W, bf16: bool = True) -> np.ndarray:
    X, W = _f32(X), _f32(W)
    T, K = X.shape
    N = W.shape[0]
    out = np.empty((T, N), dtype=np.float32)
    lib().orc_k_gemm_fp8(_fp(X), _fp(W), _fp(out), T, N, K, int(bf16))
    return out


def k_quant_w4(W):
    """int4 g128 round-to-nearest: (packed uint32 [N, ceil(K/8)], fp16 scales as uint16 [N, ceil(K/128)])."""
    W = _f32(W)
    N, K = W.shape
    packed = np.zeros((N, (K + 7) // 8), dtype=np.uint32)
    scales = np.zeros((N, (K + 127) // 128), dtype=np.uint16)
    lib().orc_k_quant_w4(_fp(W), N, K, packed.ctypes.data_as(C.POINTER(C.c_uint32)), scales.ctypes.data_as(C.POINTER(C.c_uint16)))
    return packed, scales


def k_dequant_w4(packed, scales, K: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    N = packed.shape[0]
    W = np.empty((N, K), dtype=np.float32)
    lib().orc_k_dequant_w4(packed.ctypes.data_as(C.POINTER(C.c_uint32)), scales.ctypes.data_as(C.POINTER(C.c_uint16)), N, K, _fp(W))
    return W


def k_nvfp4_rows(x, global_scale: float = 1.0):
    """NVFP4 round trip of each row: (packed uint8 [rows, K/2], e4m3 scales uint8 [rows, K/16], dequantised f32)."""
    x = _f32(x)
    rows, K = x.shape
    packed = np.zeros((rows, K // 2), dtype=np.uint8)
    scales = np.zeros((rows, K // 16), dtype=np.uint8)
    deq = np.empty((rows, K), dtype=np.float32)
    u8 = C.POINTER(C.c_uint8)
    lib().orc_k_nvfp4_rows(_fp(x), rows, K, C.c_float(global_scale), packed.ctypes.data_as(u8), scales.ctypes.data_as(u8), _fp(deq))
    return packed, scales, deq


def nvfp4_scale_repack(scales: np.ndarray, inner: int) -> np.ndarray:
    """Row-major e4m3 scales [outer, inner/16] -> cuBLASLt 128 x 4 tiles (uint8, padded to whole 128-row blocks)."""
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    outer = scales.shape[0]
    out = np.zeros(((outer + 127) // 128) * (inner // 64) * 512, dtype=np.uint8)
    u8 = C.POINTER(C.c_uint8)
    lib().orc_nvfp4_scale_repack(scales.ctypes.data_as(u8), outer, inner, out.ctypes.data_as(u8))
    return out


def k_rmsnorm(x, w, eps: float, zero_centered: bool, bf16: bool) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().orc_k_rmsnorm(_fp(x), _fp(w), _fp(out), x.shape[0], x.shape[1], C.c_float(eps), int(zero_centered), int(bf16))
    return out


def k_add_rmsnorm(x, mix, w, eps: float, bf16: bool):
    x, mix, w = _f32(x), _f32(mix), _f32(w)
    res, out = np.empty_like(x), np.empty_like(x)
    lib().orc_k_add_rmsnorm(_fp(x), _fp(mix), _fp(w), _fp(res), _fp(out), x.shape[0], x.shape[1], C.c_float(eps), int(bf16))
    return res, out


def k_rmsnorm_gated(x, gate, w, eps: float, bf16: bool) -> np.ndarray:
    x, gate, w = _f32(x), _f32(gate), _f32(w)
    out = np.empty_like(x)
    lib().orc_k_rmsnorm_gated(_fp(x), _fp(gate), _fp(w), _fp(out), x.shape[0], x.shape[1], C.c_float(eps), int(bf16))
    return out


def k_conv1d(x, hist, w, bf16: bool) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    h = None if hist is None else _f32(hist)
    lib().orc_k_conv1d(_fp(x), None if h is None else _fp(h), _fp(w), _fp(out), x.shape[0], x.shape[1], int(bf16))
    return out


def k_gdn_prepare(qkv, b, a, A_log, dt_bias, nk, nv, dk, dv, bf16: bool):
    qkv, b, a, A_log, dt_bias = map(_f32, (qkv, b, a, A_log, dt_bias))
    T = qkv.shape[0]
    qf = np.empty((T, nv, dk), np.float32)
    kf = np.empty((T, nv, dk), np.float32)
    vf = np.empty((T, nv, dv), np.float32)
    g = np.empty((T, nv), np.float32)
    beta = np.empty((T, nv), np.float32)
    lib().orc_k_gdn_prepare(_fp(qkv), _fp(b), _fp(a), _fp(A_log), _fp(dt_bias), _fp(qf), _fp(kf), _fp(vf), _fp(g), _fp(beta), T, nk, nv, dk, dv, int(bf16))
    return qf, kf, vf, g, beta


def k_gdn_recurrent(qf, kf, vf, g, beta, state, bf16: bool):
    qf, kf, vf, g, beta = map(_f32, (qf, kf, vf, g, beta))
    state = _f32(state).copy()
    T, nv, dk = qf.shape
    dv = vf.shape[2]
    out = np.empty((T, nv, dv), np.float32)
    lib().orc_k_gdn_recurrent(_fp(qf), _fp(kf), _fp(vf), _fp(g), _fp(beta), _fp(state), _fp(out), T, nv, dk, dv, int(bf16))
    return out, state


def k_attention(q, k0, v0, k1, v1, bf16: bool) -> np.ndarray:
    q = _f32(q)
    nq, heads, hd = q.shape
    k0, v0 = _f32(k0), _f32(v0)
    kv = k0.shape[1]
    n1 = 0 if k1 is None else k1.shape[0]
    k1 = _f32(k1) if n1 else np.zeros((1, kv, hd), np.float32)
    v1 = _f32(v1) if n1 else np.zeros((1, kv, hd), np.float32)
    out = np.empty_like(q)
    lib().orc_k_attention(_fp(q), nq, _fp(k0), _fp(v0), k0.shape[0], _fp(k1), _fp(v1), n1, _fp(out), heads, kv, hd, int(bf16))
    return out


def k_rope(x, pos, rotary_dim: int, theta: float, bf16: bool) -> np.ndarray:
    x = _f32(x).copy()
    T, nh, hd = x.shape
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    lib().orc_k_rope(_fp(x), nh, T, _ip(pos), hd, rotary_dim, C.c_float(theta), int(bf16))
    return x


def k_rope_tables(rotary_dim: int, theta: float, max_pos: int, bf16: bool):
    half = rotary_dim // 2
    cos_t = np.empty((max_pos, half), np.float32)
    sin_t = np.empty((max_pos, half), np.float32)
    lib().orc_k_rope_tables(rotary_dim, C.c_float(theta), max_pos, int(bf16), _fp(cos_t), _fp(sin_t))
    return cos_t, sin_t


# ----- integer / layout parts ----------------------------------------------

def block_cascade_mask(seq: int, split: int) -> np.ndarray:
    mask = np.zeros((seq * seq + 7) // 8, dtype=np.uint8)
    rc = lib().orc_block_cascade_mask(C.c_int64(seq), C.c_int64(split), mask.ctypes.data_as(C.POINTER(C.c_uint8)))
    if rc:
        raise ValueError(f"block split {split} out of range for {seq} tokens")
    return mask


def pack(lens, pos_start: int):
    lens = np.ascontiguousarray(lens, dtype=np.int32)
    B = len(lens)
    total = int(lens.sum()) if B else 0
    offsets = np.zeros(B + 1, np.int32)
    positions = np.zeros(max(total, 1), np.int32)
    tok_q = np.zeros(max(total, 1), np.int32)
    last = np.zeros(max(B, 1), np.int32)
    rc = lib().orc_pack(_ip(lens), B, pos_start, _ip(offsets), _ip(positions), _ip(tok_q), _ip(last))
    if rc:
        raise ValueError("empty batch" if rc == -3 else "batch item has no tokens")
    return offsets, positions[:total], tok_q[:total], last[:B]


def plan_chunks(lens, state: int, max_rows: int = 64, max_keys: int = 1 << 18, max_scores: int = 1 << 27):
    lens = np.ascontiguousarray(lens, dtype=np.int64)
    B = len(lens)
    order = np.zeros(max(B, 1), np.int32)
    chunk_of = np.zeros(max(B, 1), np.int32)
    n = lib().orc_plan_chunks(lens.ctypes.data_as(C.POINTER(C.c_int64)), B, C.c_int64(state), C.c_int64(max_rows), C.c_int64(max_keys), C.c_int64(max_scores), _ip(order), _ip(chunk_of))
    if n < 0:
        raise ValueError(f"plan_chunks rc={n}")
    return n, order[:B], chunk_of[:B]


def repack_nvfp4_scales(src: np.ndarray, outer: int, inner: int) -> np.ndarray:
    src = np.ascontiguousarray(src, dtype=np.uint8)
    dst = np.zeros((inner // 64) * ((outer + 127) // 128) * 512, dtype=np.uint8)
    lib().orc_repack_nvfp4_scales(src.ctypes.data_as(C.POINTER(C.c_uint8)), C.c_int64(outer), C.c_int64(inner), dst.ctypes.data_as(C.POINTER(C.c_uint8)))
    return dst


KIND = {"choice": 0, "noul": 1, "score": 2}


def decode_answer(logits, count: int, temperature: float, kind: str):
    logits = _f32(logits)
    shares = np.zeros(count, np.float32)
    out2 = np.zeros(2, np.float32)
    rc = lib().orc_decode_answer(_fp(logits), count, C.c_float(temperature), KIND[kind], _fp(shares), _fp(out2))
    if rc:
        raise ValueError("non-finite d3 logits")
    return shares, out2


def set_gemm_variant(v: int) -> None:
    """0: default 8-lane f32 accumulation; 1: double-precision in-order accumulation."""
    lib().orc_set_gemm_variant(v)


def num_threads() -> int:
    return lib().orc_num_threads()


# ---- checkpoint storage formats (numpy integer arithmetic) --------------------------------------------------

def ct_w4_dequant(packed, scale, zp, in_dim: int, group_size: int) -> np.ndarray:
    """compressed-tensors pack-quantized int4 -> bf16-rounded f32 [out, in].

    Restates dequant_w4a16_bf16 (native/kernels/kernels.cu:874-892): packed int32 [out, ceil(in/8)], nibble
    (i & 7) of word (i >> 3); scale f32 values of the bf16 tensor [out, groups]; zp int32 [ceil(out/8), groups],
    nibble (o & 7) of word (o >> 3); w = bf16((q - z) * scale). zp None = symmetric checkpoint, whose loader
    substitutes 0x88888888 words, i.e. z = 8 (native/src/weights.rs:314-320)."""
    packed = np.ascontiguousarray(packed).view(np.uint32)
    out_dim = packed.shape[0]
    i = np.arange(in_dim)
    o = np.arange(out_dim)
    q = ((packed[:, i >> 3] >> (4 * (i & 7)).astype(np.uint32)) & 0xF).astype(np.int32)
    g = i // group_size
    if zp is None:
        z = np.full((out_dim, in_dim), 8, np.int32)
    else:
        zw = np.ascontiguousarray(zp).view(np.uint32)
        z = ((zw[(o >> 3)[:, None], g[None, :]] >> (4 * (o & 7)).astype(np.uint32)[:, None]) & 0xF).astype(np.int32)
    s = _f32(scale)[:, g]
    return rb(((q - z).astype(np.float32) * s).astype(np.float32))


E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def ct_nvfp4_dequant(packed, scales, weight_global: float) -> np.ndarray:
    """compressed-tensors nvfp4-pack-quantized weight -> bf16-rounded f32 [out, in].

    Layout of NvFp4Weight (native/src/weights.rs:36-45, 502-547): packed uint8 [out, in/2], low nibble = even input;
    e4m3 scale per 16 inputs, row-major [out, in/16]; the weight's real value is e2m1 * scale / weight_global, the
    weight factor of alpha = 1 / (weight_global * input_global) in Engine::nvfp4_gemm (native/src/engine.rs:4109)."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out_dim, half = packed.shape
    codes = np.empty((out_dim, half * 2), dtype=np.uint8)
    codes[:, 0::2] = packed & 0xF
    codes[:, 1::2] = packed >> 4
    sd = e4m3_to_f32(scales).astype(np.float32)
    if weight_global > 0:
        sd = (sd / np.float32(weight_global)).astype(np.float32)
    return rb((E2M1[codes] * np.repeat(sd, 16, axis=1)).astype(np.float32))
