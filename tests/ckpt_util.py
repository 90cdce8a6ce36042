"""Test helpers: write safetensors files and synthetic model directories (numpy only).

File format (safetensors): u64 little-endian header length, a JSON header {name: {dtype, shape, data_offsets}},
then the tensor bytes back to back."""
import json
import struct
from pathlib import Path

import numpy as np

# tensor kinds of the C ABI (DCD_T_*)
T_EMBED, T_FINAL_NORM, T_READOUT = 0, 1, 2
T_INPUT_NORM, T_POST_NORM, T_GATE, T_UP, T_DOWN = 10, 11, 12, 13, 14
T_Q, T_K, T_V, T_O, T_QNORM, T_KNORM = 20, 21, 22, 23, 24, 25
T_IN_QKV, T_IN_Z, T_IN_B, T_IN_A, T_OUT, T_CONV, T_A_LOG, T_DT_BIAS, T_GNORM = 30, 31, 32, 33, 34, 35, 36, 37, 38


def bf16_bits(x) -> np.ndarray:
    """f32 -> bf16 bit patterns (round to nearest even) as uint16."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_round(x) -> np.ndarray:
    return (bf16_bits(x).astype(np.uint32) << 16).view(np.float32).reshape(np.shape(x))


def write_safetensors(path, tensors, metadata=None, pad_header_to=8):
    """tensors: {name: (dtype string, shape, numpy array holding the raw storage)}."""
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, (dt, shape, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % pad_header_to)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def bf16_entry(x):
    x = np.asarray(x, dtype=np.float32)
    return ("BF16", x.shape, bf16_bits(x))


def f32_entry(x):
    x = np.asarray(x, dtype=np.float32)
    return ("F32", x.shape, x)


def write_config(model_dir, cfg, partial_rotary_factor, nested=True, attention_in="decision"):
    """config.json (+ decision_config.json) for a product ModelConfig."""
    text = {
        "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.heads, "num_key_value_heads": cfg.kv_heads,
        "hidden_size": cfg.hidden, "head_dim": cfg.head_dim, "intermediate_size": cfg.intermediate, "vocab_size": cfg.vocab,
        "rms_norm_eps": float(cfg.rms_eps),
        "layer_types": ["full_attention" if f else "linear_attention" for f in cfg.layer_types()],
        "linear_num_key_heads": cfg.gdn_k_heads, "linear_num_value_heads": cfg.gdn_v_heads,
        "linear_key_head_dim": cfg.gdn_dk, "linear_value_head_dim": cfg.gdn_dv,
        "rope_parameters": {"rope_theta": float(cfg.rope_theta), "partial_rotary_factor": partial_rotary_factor,
                            "mrope_section": [11, 11, 10]},
    }
    top = {"text_config": text} if nested else dict(text)
    if attention_in == "config":
        top["attention_mode"] = "prefix_bidir"
    Path(model_dir, "config.json").write_text(json.dumps(top))
    if attention_in == "decision":
        Path(model_dir, "decision_config.json").write_text(json.dumps({"attention_mode": "prefix_bidir"}))


def _int4_module(rng, out, in_dim, group, symmetric):
    words, groups = (in_dim + 7) // 8, in_dim // group
    packed = rng.integers(0, 2**32, (out, words), dtype=np.uint64).astype(np.uint32).view(np.int32)
    scale = bf16_round(rng.uniform(0.002, 0.006, (out, groups)).astype(np.float32))
    zp = None if symmetric else rng.integers(0, 2**32, ((out + 7) // 8, groups), dtype=np.uint64).astype(np.uint32).view(np.int32)
    return packed, scale, zp


def _nvfp4_module(rng, out, in_dim):
    packed = rng.integers(0, 256, (out, in_dim // 2), dtype=np.uint8)
    # e4m3 codes of positive normal scales below 2 (exponent field 1..7), so that weights stay near 0.05
    scales = (rng.integers(1, 8, (out, in_dim // 16)) << 3 | rng.integers(0, 8, (out, in_dim // 16))).astype(np.uint8)
    return packed, scales, float(rng.uniform(200.0, 4000.0))


def synth_model_dir(model_dir, cfg, oracle, seed=0, prefix="model.language_model.", quant=None, shards=1,
                    partial_rotary_factor=0.25, readout_dtype="F32"):
    """Write a synthetic checkpoint of `cfg` and return {(layer, kind): f32 values} — the logical tensors a
    loader must end up with. quant: None (all BF16), "int4" (groups of 64 and 128, with and without zero points), "int4_sym128"
    (symmetric, group 128) or "nvfp4" (every linear whose input width allows it; the others stay BF16, as a real mixed checkpoint
    does)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    H, I = cfg.hidden, cfg.intermediate
    qcols, kvcols = cfg.heads * 2 * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    kd, vd = cfg.gdn_k_heads * cfg.gdn_dk, cfg.gdn_v_heads * cfg.gdn_dv
    conv_dim = 2 * kd + vd
    tensors, logical = {}, {}

    def normal(shape, std=0.02, shift=0.0):
        return bf16_round((rng.standard_normal(shape) * std + shift).astype(np.float32))

    def plain(name, layer, kind, values, storage="BF16", shape=None):
        values = np.asarray(values, dtype=np.float32)
        logical[(layer, kind)] = values.ravel().copy()
        shape = shape or values.shape
        tensors[name] = ("BF16", shape, bf16_bits(values)) if storage == "BF16" else ("F32", shape, values)

    def linear(module, layer, kind, out, in_dim, n_lin=[0]):
        n_lin[0] += 1
        if quant == "int4_sym128" and in_dim % 128 == 0:
            # symmetric, group 128, scales exact in fp16: the form a W4 engine can keep code for code
            packed, scale, zp = _int4_module(rng, out, in_dim, 128, True)
            tensors[module + ".weight_packed"] = ("I32", packed.shape, packed)
            tensors[module + ".weight_scale"] = ("BF16", scale.shape, bf16_bits(scale))
            tensors[module + ".weight_shape"] = ("I64", (2,), np.array([out, in_dim], dtype=np.int64))
            logical[(layer, kind)] = oracle.ct_w4_dequant(packed, scale, None, in_dim, 128).ravel()
        elif quant == "int4" and in_dim % 64 == 0:
            group = 64 if n_lin[0] % 2 else (128 if in_dim % 128 == 0 else 64)
            symmetric = n_lin[0] % 3 == 0
            packed, scale, zp = _int4_module(rng, out, in_dim, group, symmetric)
            tensors[module + ".weight_packed"] = ("I32", packed.shape, packed)
            tensors[module + ".weight_scale"] = ("BF16", scale.shape, bf16_bits(scale))
            tensors[module + ".weight_shape"] = ("I64", (2,), np.array([out, in_dim], dtype=np.int64))
            if zp is not None:
                tensors[module + ".weight_zero_point"] = ("I32", zp.shape, zp)
            logical[(layer, kind)] = oracle.ct_w4_dequant(packed, scale, zp, in_dim, group).ravel()
        elif quant == "nvfp4" and in_dim % 64 == 0:
            packed, scales, g = _nvfp4_module(rng, out, in_dim)
            tensors[module + ".weight_packed"] = ("U8", packed.shape, packed)
            tensors[module + ".weight_scale"] = ("F8_E4M3", scales.shape, scales)
            tensors[module + ".weight_global_scale"] = ("F32", (1,), np.array([g], dtype=np.float32))
            tensors[module + ".input_global_scale"] = ("F32", (1,), np.array([1.0], dtype=np.float32))
            logical[(layer, kind)] = oracle.ct_nvfp4_dequant(packed, scales, g).ravel()
        else:
            plain(module + ".weight", layer, kind, normal((out, in_dim)))

    P = prefix
    plain(P + "embed_tokens.weight", -1, T_EMBED, normal((cfg.vocab, H)))
    plain(P + "norm.weight", -1, T_FINAL_NORM, normal((H,)))
    for i in range(cfg.num_layers):
        l = f"{P}layers.{i}."
        plain(l + "input_layernorm.weight", i, T_INPUT_NORM, normal((H,)))
        plain(l + "post_attention_layernorm.weight", i, T_POST_NORM, normal((H,)))
        linear(l + "mlp.gate_proj", i, T_GATE, I, H)
        linear(l + "mlp.up_proj", i, T_UP, I, H)
        linear(l + "mlp.down_proj", i, T_DOWN, H, I)
        if cfg.layer_is_full[i]:
            linear(l + "self_attn.q_proj", i, T_Q, qcols, H)
            linear(l + "self_attn.k_proj", i, T_K, kvcols, H)
            linear(l + "self_attn.v_proj", i, T_V, kvcols, H)
            linear(l + "self_attn.o_proj", i, T_O, H, cfg.heads * cfg.head_dim)
            plain(l + "self_attn.q_norm.weight", i, T_QNORM, normal((cfg.head_dim,)))
            plain(l + "self_attn.k_norm.weight", i, T_KNORM, normal((cfg.head_dim,)))
        else:
            linear(l + "linear_attn.in_proj_qkv", i, T_IN_QKV, conv_dim, H)
            linear(l + "linear_attn.in_proj_z", i, T_IN_Z, vd, H)
            linear(l + "linear_attn.in_proj_b", i, T_IN_B, cfg.gdn_v_heads, H)
            linear(l + "linear_attn.in_proj_a", i, T_IN_A, cfg.gdn_v_heads, H)
            linear(l + "linear_attn.out_proj", i, T_OUT, H, vd)
            conv = bf16_round(rng.uniform(-0.5, 0.5, (conv_dim, 4)).astype(np.float32))
            plain(l + "linear_attn.conv1d.weight", i, T_CONV, conv, shape=(conv_dim, 1, 4))  # the HF [C, 1, 4] form
            plain(l + "linear_attn.A_log", i, T_A_LOG, rng.uniform(0, np.log(16.0), cfg.gdn_v_heads).astype(np.float32), storage="F32")
            plain(l + "linear_attn.dt_bias", i, T_DT_BIAS, bf16_round(rng.uniform(-6.9, -2.3, cfg.gdn_v_heads).astype(np.float32)))
            plain(l + "linear_attn.norm.weight", i, T_GNORM, normal((cfg.gdn_dv,), shift=1.0))
    readout = (rng.standard_normal((cfg.readout_rows, H)) * 0.02).astype(np.float32)
    if readout_dtype == "BF16":
        readout = bf16_round(readout)
        write_safetensors(model_dir / "readout.safetensors", {"weight": ("BF16", readout.shape, bf16_bits(readout))})
    else:
        write_safetensors(model_dir / "readout.safetensors", {"weight": ("F32", readout.shape, readout)})
    logical[(-1, T_READOUT)] = readout.ravel().copy()

    names = list(tensors)
    if shards == 1:
        write_safetensors(model_dir / "model.safetensors", tensors, metadata={"format": "pt"})
    else:
        weight_map = {}
        for s in range(shards):
            part = {n: tensors[n] for n in names[s::shards]}
            fn = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
            write_safetensors(model_dir / fn, part, metadata={"format": "pt"})
            weight_map.update({n: fn for n in part})
        (model_dir / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    write_config(model_dir, cfg, partial_rotary_factor)
    return logical
