"""CPU tests of the checkpoint store and config reader (no GPU: these entry points touch no device).

They follow the reference's Store / Config behaviour: directory resolution order (native/src/tensor.rs:62-99),
dtype names (tensor.rs:25-38), the name -> byte-range table, and Config::from_dir defaults and fail-closed
attention_mode handling (native/src/config.rs:49-172, including the fixture of its own unit test, :190-221)."""
import json
import struct

import numpy as np
import pytest

from ckpt_util import bf16_bits, write_safetensors


@pytest.fixture(scope="module")
def ck(dcd):
    from decidra_b200 import checkpoint
    return checkpoint


def _sample(rng):
    return {
        "a.f32": ("F32", (3, 5), rng.standard_normal((3, 5)).astype(np.float32)),
        "b.bf16": ("BF16", (4, 8), bf16_bits(rng.standard_normal((4, 8)))),
        "c.f16": ("F16", (7,), rng.standard_normal(7).astype(np.float16)),
        "d.i32": ("I32", (2, 3), rng.integers(-2**31, 2**31 - 1, (2, 3), dtype=np.int64).astype(np.int32)),
        "e.i64": ("I64", (2,), np.array([17408, 5120], dtype=np.int64)),
        "f.u8": ("U8", (9,), rng.integers(0, 256, 9, dtype=np.uint8)),
        "g.bool": ("BOOL", (4,), np.array([1, 0, 1, 1], dtype=np.uint8)),
        "h.f8": ("F8_E4M3", (2, 16), rng.integers(0, 256, (2, 16), dtype=np.uint8)),
        "i.f8fn": ("F8_E4M3FN", (16,), rng.integers(0, 256, 16, dtype=np.uint8)),
        "scalar": ("F32", (), np.array(3.5, dtype=np.float32)),
        "empty": ("F32", (0, 4), np.zeros((0, 4), dtype=np.float32)),
        "näme \"q\" \\ ☃": ("U8", (1,), np.array([7], dtype=np.uint8)),
    }


def test_single_file_table_and_bytes(ck, tmp_path):
    rng = np.random.default_rng(0)
    tensors = _sample(rng)
    path = tmp_path / "one.safetensors"
    write_safetensors(path, tensors, metadata={"format": "pt", "note": "x"})
    st = ck.Store(path)
    assert len(st) == len(tensors)
    assert sorted(st.names()) == sorted(tensors)
    want_dt = {"F32": ck.DT_F32, "BF16": ck.DT_BF16, "F16": ck.DT_F16, "I32": ck.DT_I32, "I64": ck.DT_I64, "U8": ck.DT_U8,
               "BOOL": ck.DT_U8, "F8_E4M3": ck.DT_F8E4M3, "F8_E4M3FN": ck.DT_F8E4M3}
    for name, (dt, shape, arr) in tensors.items():
        d, s, nbytes = st.info(name)
        assert d == want_dt[dt] and s == tuple(shape) and nbytes == np.asarray(arr).nbytes
        assert st.array(name).tobytes() == np.ascontiguousarray(arr).tobytes()
    assert st.contains("a.f32") and not st.contains("a.f33")
    with pytest.raises(Exception, match="not found"):
        st.info("missing.weight")
    st.close()


def test_reads_files_written_by_the_safetensors_package(ck, tmp_path):
    torch = pytest.importorskip("torch")
    st_torch = pytest.importorskip("safetensors.torch")
    g = torch.Generator().manual_seed(1)
    tensors = {
        "w": torch.randn(6, 10, generator=g).to(torch.bfloat16),
        "x": torch.randn(3, generator=g),
        "n": torch.arange(12, dtype=torch.int32).reshape(3, 4),
        "s": torch.tensor([17408, 5120], dtype=torch.int64),
    }
    path = tmp_path / "pkg.safetensors"
    st_torch.save_file(tensors, str(path), metadata={"format": "pt"})
    st = ck.Store(path)
    assert st.array("w").tobytes() == tensors["w"].view(torch.int16).numpy().tobytes()
    assert np.array_equal(st.array("x"), tensors["x"].numpy())
    assert np.array_equal(st.array("n"), tensors["n"].numpy())
    assert st.array("s").tolist() == [17408, 5120]


def test_directory_resolution_order(ck, tmp_path):
    rng = np.random.default_rng(2)
    one = {"t": ("F32", (2,), np.array([1, 2], dtype=np.float32))}
    # 1. model.safetensors alone wins over other files in the directory
    d1 = tmp_path / "single"
    d1.mkdir()
    write_safetensors(d1 / "model.safetensors", one)
    write_safetensors(d1 / "readout.safetensors", {"weight": ("F32", (1, 2), np.zeros((1, 2), dtype=np.float32))})
    st = ck.Store(d1)
    assert st.names() == ["t"]
    # 2. an index lists the shards; files it does not list are ignored
    d2 = tmp_path / "sharded"
    d2.mkdir()
    write_safetensors(d2 / "model-00001-of-00002.safetensors", {"a": ("F32", (2,), rng.standard_normal(2).astype(np.float32))})
    write_safetensors(d2 / "model-00002-of-00002.safetensors", {"b": ("F32", (3,), rng.standard_normal(3).astype(np.float32))})
    write_safetensors(d2 / "readout.safetensors", {"weight": ("F32", (1, 2), np.zeros((1, 2), dtype=np.float32))})
    (d2 / "model.safetensors.index.json").write_text(json.dumps(
        {"metadata": {"total_size": 20}, "weight_map": {"a": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}}))
    st = ck.Store(d2)
    assert sorted(st.names()) == ["a", "b"]
    # 3. neither: every *.safetensors, sorted by name (a later file overrides an earlier tensor of the same name)
    d3 = tmp_path / "loose"
    d3.mkdir()
    write_safetensors(d3 / "a.safetensors", {"x": ("F32", (1,), np.array([1.0], dtype=np.float32))})
    write_safetensors(d3 / "b.safetensors", {"x": ("F32", (1,), np.array([2.0], dtype=np.float32)), "y": ("U8", (1,), np.array([3], dtype=np.uint8))})
    (d3 / "notes.txt").write_text("ignored")
    st = ck.Store(d3)
    assert sorted(st.names()) == ["x", "y"] and st.array("x")[0] == 2.0
    # 4. nothing to open
    d4 = tmp_path / "none"
    d4.mkdir()
    with pytest.raises(Exception, match="no safetensors files"):
        ck.Store(d4)
    with pytest.raises(Exception, match="opening"):
        ck.Store(tmp_path / "absent.safetensors")


def test_malformed_files_are_rejected(ck, tmp_path):
    good = {"t": ("F32", (2,), np.array([1, 2], dtype=np.float32))}
    p = tmp_path / "f64.safetensors"
    write_safetensors(p, {"t": ("F64", (1,), np.array([1.0]))})
    with pytest.raises(Exception, match="unsupported safetensors dtype F64"):
        ck.Store(p)
    p = tmp_path / "short.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(Exception, match="header length"):
        ck.Store(p)
    p = tmp_path / "tiny.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(Exception, match="not a safetensors file"):
        ck.Store(p)
    p = tmp_path / "badjson.safetensors"
    p.write_bytes(struct.pack("<Q", 8) + b'{"t": [}')
    with pytest.raises(Exception, match="parsing header"):
        ck.Store(p)
    # a byte range that leaves the file, and one that disagrees with dtype x shape
    for offs, what in (([0, 64], "data_offsets"), ([0, 4], "byte range")):
        h = json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": offs}}).encode()
        p = tmp_path / f"range{offs[1]}.safetensors"
        p.write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 8)
        with pytest.raises(Exception, match=what):
            ck.Store(p)
    # a dimension that is not an unsigned integer, and a shape whose element count wraps 64 bits and would then "match" its range
    for shape, tag in (([2.5], "frac"), ([-2], "neg"), (["2"], "str"), ([1 << 62, 4, 2], "wrap"), ([1 << 63, 2], "wrap2")):
        h = json.dumps({"t": {"dtype": "F32", "shape": shape, "data_offsets": [0, 8]}}).encode()
        p = tmp_path / f"shape_{tag}.safetensors"
        p.write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 8)
        with pytest.raises(Exception, match="shape is not a list of unsigned integers"):
            ck.Store(p)
    write_safetensors(tmp_path / "ok.safetensors", good)
    assert ck.Store(tmp_path / "ok.safetensors").array("t").tolist() == [1.0, 2.0]


def _write_cfg(d, config, decision=None):
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps(config))
    if decision is not None:
        (d / "decision_config.json").write_text(json.dumps(decision))


MINIMAL = {"text_config": {"num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "hidden_size": 64,
                           "intermediate_size": 128, "vocab_size": 256, "layer_types": ["linear_attention", "full_attention"]}}


def test_config_minimal_fixture_and_defaults(ck, tmp_path):
    """The configuration of the reference's own Config unit test: two layers, everything else defaulted."""
    _write_cfg(tmp_path / "m", MINIMAL, {"attention_mode": "prefix_bidir"})
    c = ck.config_from_dir(tmp_path / "m")
    assert (c.num_layers, c.heads, c.kv_heads, c.hidden, c.intermediate, c.vocab) == (2, 4, 2, 64, 128, 256)
    assert c.layer_types() == [0, 1]
    assert c.head_dim == 16                       # hidden / heads
    assert c.rotary_dim == 16                     # partial_rotary_factor defaults to 1.0
    assert c.rope_theta == np.float32(1e7) and c.rms_eps == np.float32(1e-6)
    assert (c.gdn_k_heads, c.gdn_v_heads, c.gdn_dk, c.gdn_dv, c.conv_kernel) == (16, 48, 128, 128, 4)
    assert c.dtype == 1 and c.readout_rows == 0


def test_config_d3_shape_flat_and_nested(ck, tmp_path):
    text = {"num_hidden_layers": 64, "num_attention_heads": 24, "num_key_value_heads": 4, "hidden_size": 5120, "head_dim": 256,
            "intermediate_size": 17408, "vocab_size": 248320, "rms_norm_eps": 1e-6,
            "layer_types": (["linear_attention"] * 3 + ["full_attention"]) * 16,
            "linear_num_key_heads": 16, "linear_num_value_heads": 48, "linear_key_head_dim": 128, "linear_value_head_dim": 128,
            "rope_parameters": {"rope_theta": 10000000.0, "partial_rotary_factor": 0.25, "mrope_section": [11, 11, 10]}}
    _write_cfg(tmp_path / "nested", {"text_config": text, "attention_mode": "prefix_bidir"})
    flat = dict(text)
    flat["attention_mode"] = "prefix_bidir"
    del flat["rope_parameters"]
    flat["partial_rotary_factor"] = 0.25          # the fallback location of the factor
    _write_cfg(tmp_path / "flat", flat)
    for d in ("nested", "flat"):
        c = ck.config_from_dir(tmp_path / d)
        assert (c.num_layers, c.hidden, c.heads, c.kv_heads, c.head_dim, c.rotary_dim) == (64, 5120, 24, 4, 256, 64)
        assert c.layer_types() == [0, 0, 0, 1] * 16
        assert (c.intermediate, c.vocab) == (17408, 248320)
    # layer_types shorter than the layer count: the rest are full attention; kv heads default to the head count
    short = {"num_hidden_layers": 3, "num_attention_heads": 2, "hidden_size": 32, "intermediate_size": 64, "vocab_size": 10,
             "layer_types": ["linear_attention"], "attention_mode": "prefix_bidir"}
    _write_cfg(tmp_path / "short", short)
    c = ck.config_from_dir(tmp_path / "short")
    assert c.layer_types() == [0, 1, 1] and c.kv_heads == 2


def test_config_fails_closed(ck, tmp_path):
    _write_cfg(tmp_path / "nomode", MINIMAL)
    with pytest.raises(Exception, match="no attention_mode"):
        ck.config_from_dir(tmp_path / "nomode")
    _write_cfg(tmp_path / "causal", MINIMAL, {"attention_mode": "causal"})
    with pytest.raises(Exception, match="unsupported attention_mode"):
        ck.config_from_dir(tmp_path / "causal")
    conflict = dict(MINIMAL)
    conflict["attention_mode"] = "causal"
    _write_cfg(tmp_path / "conflict", conflict, {"attention_mode": "prefix_bidir"})
    with pytest.raises(Exception, match="conflicts"):
        ck.config_from_dir(tmp_path / "conflict")
    missing = {"text_config": {k: v for k, v in MINIMAL["text_config"].items() if k != "vocab_size"}}
    _write_cfg(tmp_path / "missing", missing, {"attention_mode": "prefix_bidir"})
    with pytest.raises(Exception, match="config missing vocab_size"):
        ck.config_from_dir(tmp_path / "missing")
    # integers that would not survive the narrowing to the engine's 32-bit fields, or make no model
    for key, value, what in (("hidden_size", 1 << 33, "hidden_size outside"), ("vocab_size", 1 << 40, "vocab_size outside"),
                             ("intermediate_size", 0, "intermediate_size outside"), ("num_attention_heads", 1 << 20, "num_attention_heads outside"),
                             ("num_key_value_heads", 3, "not a multiple")):
        bad = {"text_config": dict(MINIMAL["text_config"], **{key: value})}
        _write_cfg(tmp_path / ("bad_" + key), bad, {"attention_mode": "prefix_bidir"})
        with pytest.raises(Exception, match=what):
            ck.config_from_dir(tmp_path / ("bad_" + key))
    (tmp_path / "empty").mkdir()
    with pytest.raises(Exception, match="config.json"):
        ck.config_from_dir(tmp_path / "empty")
