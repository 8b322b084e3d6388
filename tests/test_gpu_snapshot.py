"""Snapshot writer (write_snapshot, src/snapshot.rs:86-148): dense Hugging-Face-keyed tensors -> a directory with
model.safetensors + config.json; with a QuantSpec the projections are stored as MLX Q4/Q8 triplets.  The reference's
own checks (tests/snapshot.rs) need real checkpoints; here the round trip is checked on the tiny decoder:
a snapshot reloads through Weights::from_dir + ModelConfig::from_json + from_weights to the same bits as
quantize-on-load, and a dense snapshot to the same bits as the source."""
import json
import struct

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

CFG_JSON = {"model_type": "llama", "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2,
            "head_dim": 64, "intermediate_size": 704, "vocab_size": 1024, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
            "tie_word_embeddings": False}
SHAPE = dict(H.CONFIG0, inter=704)  # the quantization group (64) must divide every input dimension


@pytest.fixture(scope="module")
def env():
    from mlx_llm_b200 import _lib, engine

    ctx = _lib.Context(0)
    yield ctx, engine
    ctx.close()


def _weights(eng, w):
    out = eng.Weights()
    out.add("model.embed_tokens.weight", w["embed"])
    out.add("lm_head.weight", w["lm_head"])
    out.add("model.norm.weight", np.ones(SHAPE["hidden"], np.float32))
    for l, lw in enumerate(w["layers"]):
        names = H.hf_weight_names(l)
        for k, v in lw.items():
            out.add(names[k], v)
        out.add(names["input_ln"], np.ones(SHAPE["hidden"], np.float32))
        out.add(names["post_ln"], np.ones(SHAPE["hidden"], np.float32))
    return out


def _logits(eng, ctx, model, prompts):
    pool = eng.BlockPool(ctx, model, 16, 64, 4, 16)
    caches = [eng.PagedKvCache(pool) for _ in prompts]
    logits, am = model.step(list(zip(prompts, caches)))
    for c in caches:
        c.free()
    pool.free()
    return np.asarray(logits), list(am)


def _read_header(path):
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        return json.loads(f.read(n))


@pytest.mark.parametrize("bits", [4, 8])
def test_quantized_snapshot_round_trip(env, tmp_path, bits):
    ctx, eng = env
    tw = H.tiny_weights(SHAPE)
    src = _weights(eng, tw)
    out_dir = tmp_path / f"snap_q{bits}"
    n = eng.write_snapshot(ctx, src, CFG_JSON, out_dir, eng.QuantSpec(64, bits))
    # 3 non-projection tensors + per layer 2 norms + 7 projections x 3
    assert n == 3 + 2 * (2 + 7 * 3)
    cfg_text = (out_dir / "config.json").read_text()
    cfg = json.loads(cfg_text)
    assert cfg["quantization"] == {"group_size": 64, "bits": bits} and cfg["hidden_size"] == 256
    hdr = _read_header(out_dir / "model.safetensors")
    q = hdr["model.layers.0.self_attn.q_proj.weight"]
    assert q["dtype"] == "U32" and q["shape"] == [256, 256 * bits // 32]
    assert hdr["model.layers.1.mlp.down_proj.scales"] == {"dtype": "BF16", "shape": [256, 704 // 64],
                                                          "data_offsets": hdr["model.layers.1.mlp.down_proj.scales"]["data_offsets"]}
    assert hdr["model.embed_tokens.weight"]["dtype"] == "F32"  # written through unchanged
    # reload as a stored-triplet snapshot and compare with quantize-on-load from the dense source
    stored = eng.Weights.from_dir(out_dir)
    assert stored.contains("model.layers.0.mlp.up_proj.biases")
    m_stored = eng.CausalLm.from_weights(ctx, stored, "", eng.model_config_from_json(cfg_text))
    m_onload = eng.CausalLm.from_weights(ctx, src, "", eng.model_config_from_json(json.dumps(CFG_JSON)), eng.QuantSpec(64, bits))
    assert m_stored.is_quantized() and m_onload.is_quantized()
    prompts = H.config0_prompts()
    l1, a1 = _logits(eng, ctx, m_stored, prompts)
    l2, a2 = _logits(eng, ctx, m_onload, prompts)
    assert np.array_equal(l1, l2) and a1 == a2
    # a second quantization of the already quantized snapshot is refused, as a config error
    with pytest.raises(Exception) as ei:
        eng.write_snapshot(ctx, src, cfg_text, tmp_path / "again", eng.QuantSpec(64, bits))
    assert "already quantized" in str(ei.value)
    for m in (m_stored, m_onload):
        m.free()
    stored.free()
    src.free()


def test_dense_snapshot_is_bit_identical(env, tmp_path):
    ctx, eng = env
    tw = H.tiny_weights(SHAPE)
    src = _weights(eng, tw)
    out_dir = tmp_path / "snap_dense"
    n = eng.write_snapshot(ctx, src, CFG_JSON, out_dir)
    assert n == 3 + 2 * (2 + 7)
    assert "quantization" not in json.loads((out_dir / "config.json").read_text())
    back = eng.Weights.from_dir(out_dir)
    cfg = eng.model_config_from_json(json.dumps(CFG_JSON))
    m1 = eng.CausalLm.from_weights(ctx, src, "", cfg)
    m2 = eng.CausalLm.from_weights(ctx, back, "", cfg)
    prompts = H.config0_prompts()
    l1, a1 = _logits(eng, ctx, m1, prompts)
    l2, a2 = _logits(eng, ctx, m2, prompts)
    assert np.array_equal(l1, l2) and a1 == a2
    for m in (m1, m2):
        m.free()
    back.free()
    src.free()
