"""Checkpoint loading on the GPU through the C ABI.

A synthetic model directory (config.json, decision_config.json, safetensors shards, readout.safetensors) is
written with the tiny configuration; the engine built from it must hold, tensor for tensor, the values the
CPU oracle computes from the stored bytes (bit-exact: BF16 copies, int4 and NVFP4 dequantisation are order-free
arithmetic), and must answer bit-identically to an engine that received the same values through the
tensor-by-tensor upload."""
import numpy as np
import pytest

import ckpt_util as U
from conftest import tiny_inputs

pytestmark = pytest.mark.gpu


def _kinds(cfg):
    out = [(-1, U.T_EMBED), (-1, U.T_FINAL_NORM), (-1, U.T_READOUT)]
    for i in range(cfg.num_layers):
        out += [(i, U.T_INPUT_NORM), (i, U.T_POST_NORM), (i, U.T_GATE), (i, U.T_UP), (i, U.T_DOWN)]
        if cfg.layer_is_full[i]:
            out += [(i, k) for k in (U.T_Q, U.T_K, U.T_V, U.T_O, U.T_QNORM, U.T_KNORM)]
        else:
            out += [(i, k) for k in (U.T_IN_QKV, U.T_IN_Z, U.T_IN_B, U.T_IN_A, U.T_OUT, U.T_CONV, U.T_A_LOG, U.T_DT_BIAS, U.T_GNORM)]
    return out


def _options(dcd, **opt):
    o = dcd.Options()
    o.max_pass_tokens = 512
    for k, v in opt.items():
        setattr(o, k, v)
    return o


def _engine_from_logical(dcd, cfg, logical, **opt):
    e = dcd.Engine(cfg, _options(dcd, **opt))
    for (layer, kind) in _kinds(cfg):
        e.load_tensor(layer, kind, logical[(layer, kind)])
    return e


def _answers(e):
    state, questions = tiny_inputs()
    return e.readout_state_once_batch(e.capture_state(state), questions)


@pytest.mark.parametrize("quant,shards,prefix,readout_dtype", [
    (None, 1, "model.language_model.", "F32"),
    (None, 3, "model.", "BF16"),
    ("int4", 2, "language_model.", "F32"),
    ("nvfp4", 1, "", "F32"),
])
def test_engine_from_model_dir_matches_tensor_upload(dcd, oracle, tmp_path, quant, shards, prefix, readout_dtype):
    from decidra_b200 import checkpoint
    cfg = dcd.tiny_config(1)
    logical = U.synth_model_dir(tmp_path, cfg, oracle, seed=3, prefix=prefix, quant=quant, shards=shards, readout_dtype=readout_dtype)
    e = checkpoint.engine_from_dir(tmp_path, _options(dcd))
    c = e.cfg
    assert (c.num_layers, c.hidden, c.heads, c.kv_heads, c.head_dim, c.rotary_dim, c.readout_rows) == (4, 256, 4, 1, 64, 16, 255)
    assert c.layer_types() == cfg.layer_types()
    for (layer, kind) in _kinds(cfg):
        want = logical[(layer, kind)]
        assert e.read_tensor(layer, kind, want.size).tobytes() == want.tobytes(), (layer, kind)
    ref = _engine_from_logical(dcd, cfg, logical)
    got, want = _answers(e), _answers(ref)
    assert np.isfinite(got).all() and np.abs(got).max() > 1e-3
    assert got.tobytes() == want.tobytes()
    e.close(); ref.close()


@pytest.mark.parametrize("precision,quant", [(1, "int4"), (2, None), (3, "nvfp4"), (3, None)])
def test_checkpoint_into_quantised_engines(dcd, oracle, tmp_path, precision, quant):
    """The loaded values take the engine's own precision route: a fused matrix is collected in the bf16 stage and
    quantised once after its last member."""
    from decidra_b200 import checkpoint
    cfg = dcd.tiny_config(1)
    H, I = cfg.hidden, cfg.intermediate
    logical = U.synth_model_dir(tmp_path, cfg, oracle, seed=5, quant=quant)
    e = checkpoint.engine_from_dir(tmp_path, _options(dcd, precision=precision))
    ref = _engine_from_logical(dcd, cfg, logical, precision=precision)
    got = _answers(e)
    assert np.isfinite(got).all() and np.abs(got).max() > 1e-3
    if precision == 1:
        # A fused matrix whose members are all symmetric group-128 int4 is served code for code (reads back as the checkpoint's
        # own dequantisation); every other matrix is quantised once by the engine (reads back as the int4 round trip of the loaded
        # values). Either way a bf16 engine holding the values read back answers with the same bits: only the storage differs.
        shapes = {U.T_GATE: (I, H), U.T_UP: (I, H), U.T_DOWN: (H, I), U.T_Q: (cfg.heads * 2 * cfg.head_dim, H), U.T_K: (cfg.kv_heads * cfg.head_dim, H),
                  U.T_V: (cfg.kv_heads * cfg.head_dim, H), U.T_O: (H, cfg.heads * cfg.head_dim), U.T_IN_QKV: (cfg.conv_dim(), H),
                  U.T_IN_Z: (cfg.gdn_v_heads * cfg.gdn_dv, H), U.T_IN_B: (cfg.gdn_v_heads, H), U.T_IN_A: (cfg.gdn_v_heads, H),
                  U.T_OUT: (H, cfg.gdn_v_heads * cfg.gdn_dv)}
        vals, kept, requantised = dict(logical), 0, 0
        for (layer, kind) in _kinds(cfg):
            if kind not in shapes:
                continue
            n, k = shapes[kind]
            back = e.read_tensor(layer, kind, n * k)
            p, s = oracle.k_quant_w4(logical[(layer, kind)].reshape(n, k))
            if back.tobytes() == logical[(layer, kind)].tobytes():
                kept += 1
            else:
                assert back.tobytes() == oracle.k_dequant_w4(p, s, k).tobytes(), (layer, kind)
                requantised += 1
            vals[(layer, kind)] = back
        print(f"int4 checkpoint on a W4 engine: {kept} tensors served as stored, {requantised} quantised once by the engine")
        assert requantised > 0 and (quant != "int4" or kept > 0)
        same = _engine_from_logical(dcd, cfg, vals)
        assert got.tobytes() == _answers(same).tobytes()
        same.close()
    elif precision == 2:
        # FP8 rows are quantised row by row, so the order of arrival cannot matter
        assert got.tobytes() == _answers(ref).tobytes()
    else:
        # the NVFP4 tensor scale is taken over the whole fused matrix; matrices with one member compare exactly
        for layer, kind, n in [(0, U.T_DOWN, H * I), (3, U.T_O, H * cfg.heads * cfg.head_dim), (1, U.T_OUT, H * cfg.gdn_v_heads * cfg.gdn_dv)]:
            assert e.read_tensor(layer, kind, n).tobytes() == ref.read_tensor(layer, kind, n).tobytes(), (layer, kind)
    if quant is None:
        plain = checkpoint.engine_from_dir(tmp_path, _options(dcd))
        base = _answers(plain)
        err = float(np.abs(got - base).max())
        print(f"precision {precision}: |logits - bf16 engine| max {err:.4g}, |logits| max {np.abs(base).max():.4g}")
        # W4A4 noise on a 4-layer random-init model is of the order of the logits themselves; FP8 stays close
        assert err < (0.25 if precision == 2 else 1.5) * max(1.0, float(np.abs(base).max()))
        plain.close()
    e.close(); ref.close()


def test_w4_engine_serves_the_checkpoints_own_int4_codes(dcd, oracle, tmp_path):
    """A symmetric group-128 int4 checkpoint on a precision-1 engine: nothing is quantised a second time. Every adopted tensor
    reads back as compressed-tensors dequantisation of the stored codes and scales, bit for bit (the reference serves exactly
    those: dequant_w4a16_bf16, native/kernels/kernels.cu:867-892), including groups that contain code 0 (value -8), whose absmax
    re-quantisation would have changed the scale. Members that cannot be adopted (down_proj: input width 688 has no group of
    128, stored as BF16) take the quantise-once route; the answers equal those of an engine fed the same values tensor by tensor
    only where nothing was re-quantised, so they are compared with the bf16 engine on the dequantised weights instead."""
    from decidra_b200 import checkpoint
    cfg = dcd.tiny_config(1)
    H, I = cfg.hidden, cfg.intermediate
    logical = U.synth_model_dir(tmp_path, cfg, oracle, seed=7, quant="int4_sym128")
    e = checkpoint.engine_from_dir(tmp_path, _options(dcd, precision=1))
    adopted = [(0, U.T_GATE, I * H), (0, U.T_UP, I * H), (1, U.T_IN_QKV, cfg.conv_dim() * H), (1, U.T_IN_Z, cfg.gdn_v_heads * cfg.gdn_dv * H),
               (2, U.T_IN_B, cfg.gdn_v_heads * H), (2, U.T_IN_A, cfg.gdn_v_heads * H), (2, U.T_OUT, H * cfg.gdn_v_heads * cfg.gdn_dv),
               (3, U.T_Q, cfg.heads * 2 * cfg.head_dim * H), (3, U.T_K, cfg.kv_heads * cfg.head_dim * H), (3, U.T_V, cfg.kv_heads * cfg.head_dim * H),
               (3, U.T_O, H * cfg.heads * cfg.head_dim)]
    has_code0 = False
    for layer, kind, n in adopted:
        want = logical[(layer, kind)]
        assert e.read_tensor(layer, kind, n).tobytes() == want.tobytes(), (layer, kind)
        has_code0 = has_code0 or bool((want < 0).any())
    assert has_code0
    # down_proj was stored as BF16 (688 = 5 * 128 + 48): quantised once by the engine
    p, s = oracle.k_quant_w4(logical[(0, U.T_DOWN)].reshape(H, I))
    assert e.read_tensor(0, U.T_DOWN, H * I).tobytes() == oracle.k_dequant_w4(p, s, I).tobytes()
    # the same weights on a bf16 engine (down_proj through its int4 round trip) answer identically: the W4 engine only changes storage
    vals = dict(logical)
    for i in range(cfg.num_layers):
        p, s = oracle.k_quant_w4(logical[(i, U.T_DOWN)].reshape(H, I))
        vals[(i, U.T_DOWN)] = oracle.k_dequant_w4(p, s, I).ravel()
    ref = _engine_from_logical(dcd, cfg, vals)
    got, want = _answers(e), _answers(ref)
    assert np.isfinite(got).all() and got.tobytes() == want.tobytes()
    e.close(); ref.close()


def test_typed_upload_equals_f32_upload(dcd, oracle):
    from decidra_b200 import checkpoint
    cfg = dcd.tiny_config(1)
    a = dcd.Engine(cfg, _options(dcd))
    b = dcd.Engine(cfg, _options(dcd))
    a.init_random(1)
    b.init_random(1)
    rng = np.random.default_rng(9)
    H, I = cfg.hidden, cfg.intermediate
    up = U.bf16_round((rng.standard_normal((I, H)) * 0.02).astype(np.float32))
    a.load_tensor(2, U.T_UP, up)
    checkpoint.load_tensor_typed(b, 2, U.T_UP, U.bf16_bits(up), checkpoint.DT_BF16)
    alog = rng.uniform(0, 2.7, cfg.gdn_v_heads).astype(np.float32)
    a.load_tensor(0, U.T_A_LOG, alog)
    checkpoint.load_tensor_typed(b, 0, U.T_A_LOG, alog, checkpoint.DT_F32)
    knorm = U.bf16_round((rng.standard_normal(cfg.head_dim) * 0.02).astype(np.float32))
    a.load_tensor(3, U.T_KNORM, knorm)
    checkpoint.load_tensor_typed(b, 3, U.T_KNORM, knorm.astype(np.float16), checkpoint.DT_F16)
    for layer, kind, n in [(2, U.T_UP, I * H), (2, U.T_GATE, I * H), (0, U.T_A_LOG, cfg.gdn_v_heads)]:
        assert a.read_tensor(layer, kind, n).tobytes() == b.read_tensor(layer, kind, n).tobytes()
    f16_back = U.bf16_round(knorm.astype(np.float16).astype(np.float32))
    assert b.read_tensor(3, U.T_KNORM, cfg.head_dim).tobytes() == f16_back.tobytes()
    with pytest.raises(dcd.EngineError, match="expects"):
        checkpoint.load_tensor_typed(b, 2, U.T_UP, U.bf16_bits(up)[:-1], checkpoint.DT_BF16)
    with pytest.raises(dcd.EngineError, match="F32, F16 or BF16"):
        checkpoint.load_tensor_typed(b, 2, U.T_UP, np.zeros(I * H, dtype=np.int32), checkpoint.DT_I32)
    a.close(); b.close()


def test_loader_errors_name_the_tensor(dcd, oracle, tmp_path):
    from decidra_b200 import checkpoint
    cfg = dcd.tiny_config(1)
    U.synth_model_dir(tmp_path / "ok", cfg, oracle, seed=1)
    # a different width: the engine refuses the shape and says which tensor
    wide = dcd.tiny_config(1)
    wide.intermediate = 704
    e = dcd.Engine(wide, _options(dcd))
    st = checkpoint.Store(tmp_path / "ok")
    with pytest.raises(dcd.EngineError, match=r"layers\.0\.mlp\.gate_proj\.weight: checkpoint shape 688 x 256"):
        checkpoint.load_checkpoint(e, st, tmp_path / "ok" / "readout.safetensors")
    e.close()
    # a checkpoint without one of the tensors
    import json
    src = checkpoint.Store(tmp_path / "ok" / "model.safetensors")
    keep = {}
    dt_name = {checkpoint.DT_F32: "F32", checkpoint.DT_BF16: "BF16"}
    for n in src.names():
        if n.endswith("layers.2.linear_attn.dt_bias"):
            continue
        d, shape, _ = src.info(n)
        keep[n] = (dt_name[d], shape, src.array(n))
    (tmp_path / "cut").mkdir()
    U.write_safetensors(tmp_path / "cut" / "model.safetensors", keep)
    e = dcd.Engine(cfg, _options(dcd))
    with pytest.raises(dcd.EngineError, match=r"layers\.2\.linear_attn\.dt_bias not found"):
        checkpoint.load_checkpoint(e, checkpoint.Store(tmp_path / "cut"), None)
    # no embedding under any known prefix
    U.write_safetensors(tmp_path / "odd.safetensors", {"transformer.wte.weight": ("F32", (1,), np.zeros(1, dtype=np.float32))})
    with pytest.raises(dcd.EngineError, match="could not locate embed_tokens.weight"):
        checkpoint.load_checkpoint(e, checkpoint.Store(tmp_path / "odd.safetensors"), None)
    # wrong readout shape
    U.write_safetensors(tmp_path / "head.safetensors", {"weight": ("F32", (3, cfg.hidden), np.zeros((3, cfg.hidden), dtype=np.float32))})
    with pytest.raises(dcd.EngineError, match="readout.weight is 3 x 256"):
        checkpoint.load_checkpoint(e, st, tmp_path / "head.safetensors")
    e.close()


def test_large_tensor_is_streamed_in_chunks(dcd, oracle):
    """A tensor larger than one staging buffer (32 MiB) goes through several chunks of the ring; rows keep
    their places (also through the gate/up interleave)."""
    from decidra_b200 import checkpoint
    cfg = dcd.make_config(num_layers=1, hidden=1024, heads=4, kv_heads=1, head_dim=64, rotary_dim=16, rope_theta=1e7, gdn_k_heads=2,
                          gdn_v_heads=4, gdn_dk=64, gdn_dv=64, intermediate=8192 * 3, vocab=40000, layer_is_full=[0])
    e = dcd.Engine(cfg, _options(dcd))
    e.init_random(0)
    rng = np.random.default_rng(4)
    H, I = cfg.hidden, cfg.intermediate
    for kind, rows in ((U.T_EMBED, cfg.vocab), (U.T_GATE, I), (U.T_UP, I)):        # 80 MB, 48 MB, 48 MB as bf16
        layer = -1 if kind == U.T_EMBED else 0
        bits = rng.integers(0, 2**16, rows * H, dtype=np.uint16) & np.uint16(0xBF7F)   # finite bf16 patterns
        checkpoint.load_tensor_typed(e, layer, kind, bits, checkpoint.DT_BF16)
        want = (bits.astype(np.uint32) << 16).view(np.float32)
        assert e.read_tensor(layer, kind, rows * H).tobytes() == want.tobytes(), kind
    e.close()
