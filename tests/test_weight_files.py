"""Weight-plane shard files (the raw layout the reference's FasterTransformer loader reads) and the oracle's restatement
of the weight quantiser: CPU only."""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _wf():
    spec = importlib.util.spec_from_file_location("weight_files_under_test", ROOT / "abq-llm_b200" / "weight_files.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def test_file_names_and_shapes_follow_the_reference_loader():
    wf = _wf()
    # LlamaDecoderLayerWeight.cc:377-403 with hidden 4096, ffn 11008, w_bits 2, two ranks; sizes there are in 16-bit elements
    assert wf.shard_path("/m", 3, "attention.query_key_value", 1).name == "model.layers.3.attention.query_key_value.weight.1.bin"
    assert wf.shard_path("/m", 0, "mlp.down_proj", 0, "scale").name == "model.layers.0.mlp.down_proj.weight.0.scale.bin"
    hidden, ffn, tp, q, sz = 4096, 11008, 2, 2, 16
    halves = {"attention.query_key_value": (q * hidden) * (3 * hidden // sz // tp), "attention.dense": (q * hidden // tp) * (hidden // sz),
              "mlp.gate_proj": (q * hidden) * (ffn // sz // tp), "mlp.up_proj": (ffn // sz // tp) * (q * hidden),
              "mlp.down_proj": (q * ffn // tp) * (hidden // sz)}
    for name, n_half in halves.items():
        planes, rows, words = wf.shard_shape(name, hidden, ffn, tp, q)
        assert planes * rows * words * 4 == n_half * 2, name
    with pytest.raises(KeyError):
        wf.shard_path("/m", 0, "lm_head", 0)


def test_round_trip_and_size_check(tmp_path, oracle):
    wf = _wf()
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 4, size=(96, 256), dtype=np.int32)
    planes = oracle.pack(codes, 2)
    scale = rng.uniform(0.001, 0.02, size=(96, 2)).astype(np.float16)
    zero = rng.integers(0, 4, size=(96, 2)).astype(np.uint8)
    wf.write_shard(tmp_path, 5, "mlp.up_proj", 1, planes, scale, zero)
    raw = (tmp_path / "model.layers.5.mlp.up_proj.weight.1.bin").read_bytes()
    assert len(raw) == 2 * 96 * 8 * 4 and raw == planes.astype("<u4").tobytes()   # no header, plane-major, little-endian words
    p2, s2, z2 = wf.read_shard(tmp_path, 5, "mlp.up_proj", 1, 2, 96, 256, groups=2)
    assert np.array_equal(p2, planes) and np.array_equal(s2, scale) and np.array_equal(z2, zero)
    assert np.array_equal(oracle.unpack(p2, False), codes)
    with pytest.raises(ValueError):
        wf.read_shard(tmp_path, 5, "mlp.up_proj", 1, 2, 100, 256)       # wrong size is an error, not random data
    with pytest.raises(FileNotFoundError):
        wf.read_shard(tmp_path, 6, "mlp.up_proj", 1, 2, 96, 256)        # so is a missing file
    wf.write_shard(tmp_path, 7, "attention.dense", 0, planes)             # weights only, as the reference ships them
    assert wf.read_shard(tmp_path, 7, "attention.dense", 0, 2, 96, 256)[1:] == (None, None)


def test_split_ranges():
    wf = _wf()
    assert wf.split_ranges(11008, 4, 128) == [(0, 2816), (2816, 5632), (5632, 8320), (8320, 11008)]
    assert wf.split_ranges(4096, 8, 128) == [(i * 512, (i + 1) * 512) for i in range(8)]


@pytest.mark.parametrize("bits,group,symmetric", [(4, None, False), (2, 64, False), (3, 128, False), (8, 128, False), (4, 128, True)])
def test_oracle_weight_quantiser_properties(oracle, bits, group, symmetric):
    """The restated min/max quantiser: codes in range, extremes hit the ends of the range, dequantisation error at most
    half a step (plus the clamp of the 1/2-bit "bit balance" top level), per group."""
    rng = np.random.default_rng(bits)
    w = rng.normal(0, 0.02, size=(32, 512)).astype(np.float16)
    codes, scale, zero = oracle.quantize_weights_minmax(w, bits, group, symmetric)
    assert codes.min() >= 0 and codes.max() <= (1 << bits) - 1
    g = group or 512
    deq = ((codes.reshape(32, -1, g) - zero.reshape(32, -1, 1).astype(np.int32)) * scale.reshape(32, -1, 1).astype(np.float32)).reshape(32, 512)
    step = np.repeat(scale.reshape(32, -1).astype(np.float32), g, axis=1)
    slack = 1.55 if bits <= 2 else 0.55  # the clamped top level of the 1/2-bit rule costs up to one more step
    assert np.all(np.abs(deq - w.astype(np.float32)) <= slack * step + 1e-6)
    if not symmetric:
        assert np.all(codes.reshape(32, -1, g).min(axis=2) == 0)
