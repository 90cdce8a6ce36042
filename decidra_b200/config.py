"""Model and option structs of the C ABI, plus the two benchmark presets (the tiny CPU-runnable hybrid and the d3-turbo shape).

``ModelConfig`` mirrors ``dcd_model_config`` (include/decidra_b200.h), the plain-struct form of
juanqui/decidra's ``Config`` (native/src/config.rs:49-158).
"""
from __future__ import annotations

import ctypes as C


class ModelConfig(C.Structure):
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

    def layer_types(self):
        return [int(self.layer_is_full[i]) for i in range(self.num_layers)]

    def conv_dim(self) -> int:
        return 2 * self.gdn_k_heads * self.gdn_dk + self.gdn_v_heads * self.gdn_dv

    def linear_macs_per_token(self) -> int:
        """Multiply-accumulates of all linear layers for one token (P_lin)."""
        H, I = self.hidden, self.intermediate
        full = H * self.heads * 2 * self.head_dim + 2 * H * self.kv_heads * self.head_dim + self.heads * self.head_dim * H
        vd = self.gdn_v_heads * self.gdn_dv
        gdn = H * self.conv_dim() + H * vd + 2 * H * self.gdn_v_heads + vd * H
        n_full = sum(self.layer_types())
        return self.num_layers * 3 * H * I + n_full * full + (self.num_layers - n_full) * gdn

    def question_flops(self, L: int, S: int) -> float:
        n_full = sum(self.layer_types())
        n_gdn = self.num_layers - n_full
        return (2.0 * self.linear_macs_per_token() * L + n_full * 4.0 * self.heads * self.head_dim * (S + L) * L
                + n_gdn * self.gdn_v_heads * 6.0 * self.gdn_dk * self.gdn_dv * L)

    def capture_flops(self, S: int) -> float:
        n_full = sum(self.layer_types())
        n_gdn = self.num_layers - n_full
        return (2.0 * self.linear_macs_per_token() * S + n_full * 4.0 * self.heads * self.head_dim * S * S
                + n_gdn * self.gdn_v_heads * 6.0 * self.gdn_dk * self.gdn_dv * S)


class Options(C.Structure):
    """Mirrors ``dcd_options``; zero means default."""

    _fields_ = [
        ("precision", C.c_int32),
        ("max_pass_tokens", C.c_int32),
        ("max_rows", C.c_int32),
        ("max_keys", C.c_int64),
        ("max_scores", C.c_int64),
        ("gemm_path", C.c_int32),
        ("attn_path", C.c_int32),
        ("max_positions", C.c_int32),
        ("gdn_path", C.c_int32),
        ("fp8_min_rows", C.c_int32),
        ("nvfp4_scale_copy", C.c_int32),
        ("w4a16_gemm", C.c_int32),
        ("nvfp4_fusion", C.c_int32),
        ("attn_split", C.c_int32),
        ("w4a16_prefetch", C.c_int32),
        ("gdn_overlap", C.c_int32),
    ]


def make_config(*, num_layers, hidden, heads, kv_heads, head_dim, rotary_dim, rope_theta, gdn_k_heads, gdn_v_heads, gdn_dk,
                gdn_dv, intermediate, vocab, readout_rows=255, rms_eps=1e-6, dtype=1, full_attn_interval=4,
                layer_is_full=None, conv_kernel=4) -> ModelConfig:
    c = ModelConfig()
    c.num_layers, c.hidden, c.heads, c.kv_heads, c.head_dim, c.rotary_dim = num_layers, hidden, heads, kv_heads, head_dim, rotary_dim
    c.rope_theta = rope_theta
    c.gdn_k_heads, c.gdn_v_heads, c.gdn_dk, c.gdn_dv, c.conv_kernel = gdn_k_heads, gdn_v_heads, gdn_dk, gdn_dv, conv_kernel
    c.intermediate, c.vocab, c.readout_rows, c.rms_eps, c.dtype = intermediate, vocab, readout_rows, rms_eps, dtype
    if layer_is_full is None:
        layer_is_full = [1 if (i + 1) % full_attn_interval == 0 else 0 for i in range(num_layers)]
    for i, f in enumerate(layer_is_full):
        c.layer_is_full[i] = int(f)
    return c


def tiny_config(dtype: int = 0) -> ModelConfig:
    """The tiny hybrid the reference can run on its CPU scalar path: 4 layers [GDN,GDN,GDN,full], hidden 256, 4q/1kv heads of 64, GDN 2k/4v heads of
    64, SwiGLU 688, vocab 4096, readout [255,256]. partial_rotary_factor 0.25 (as d3-turbo) → rotary_dim 16."""
    return make_config(num_layers=4, hidden=256, heads=4, kv_heads=1, head_dim=64, rotary_dim=16, rope_theta=1e7,
                       gdn_k_heads=2, gdn_v_heads=4, gdn_dk=64, gdn_dv=64, intermediate=688, vocab=4096, dtype=dtype)


def d3_config(num_layers: int = 64, dtype: int = 1, vocab: int = 248320) -> ModelConfig:
    """The d3-turbo shape of the headline benchmark and of the quantised and ragged-stress workloads: 3 GDN : 1 full, hidden 5120, 24q/4kv heads of 256 (rotary 64),
    GDN 16k/48v heads of 128, SwiGLU 17408, vocab 248320, readout [255,5120]."""
    return make_config(num_layers=num_layers, hidden=5120, heads=24, kv_heads=4, head_dim=256, rotary_dim=64, rope_theta=1e7,
                       gdn_k_heads=16, gdn_v_heads=48, gdn_dk=128, gdn_dv=128, intermediate=17408, vocab=vocab, dtype=dtype)
