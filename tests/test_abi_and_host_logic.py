"""CPU-side checks: the C-ABI library loads and exports every symbol include/b200llm.h declares, the
host-only entry points (config parsing, weights container, RoPE tables) behave like the reference,
and the product fails loudly without a GPU instead of falling back to anything."""
import ctypes as C
import json
import os
import re
import struct

import numpy as np
import pytest

from tests import helpers as H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from mlx_llm_b200 import _lib, build

    build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200llm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text)) - {"b2_event_cb"})


def test_library_exports_every_declared_symbol(lib):
    names = declared_symbols()
    assert len(names) > 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in b200llm.h but not exported: {missing}"


def test_no_torch_and_no_oracle_in_the_product():
    """The shipped library links only the CUDA runtime, and the package never imports the oracle."""
    import subprocess

    from mlx_llm_b200 import _lib

    out = subprocess.run(["ldd", _lib.LIB_PATH], capture_output=True, text=True).stdout
    names = [line.split()[0] for line in out.splitlines() if line.strip()]  # library names only: load addresses are random hex
    assert not any("torch" in n or "c10" in n for n in names), names
    pkg = os.path.join(ROOT, "mlx_llm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower() or f == "build.py", f"{f} mentions the oracle"


def test_fails_loudly_without_a_gpu(lib):
    from mlx_llm_b200 import _lib

    if _lib.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(_lib.B2Error) as e:
        _lib.Context(0)
    assert e.value.code == -1


def test_model_config_from_json_llama31(lib):  # config.rs:608-632
    from mlx_llm_b200 import engine as eng

    c = eng.model_config_from_json(dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                                        num_key_value_heads=8, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0,
                                        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                                          original_max_position_embeddings=8192)))
    assert (c.hidden_size, c.head_dim, c.num_kv_heads, c.num_heads // c.num_kv_heads) == (4096, 128, 8, 4)
    assert c.rope_kind == 1 and c.rope_factor == 8.0 and c.rope_original_context == 8192.0 and c.qk_norm == 0


def test_model_config_defaults_and_errors(lib):  # config.rs:634-660, :870-884
    from mlx_llm_b200 import engine as eng
    from mlx_llm_b200._lib import B2Error

    c = eng.model_config_from_json(dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, vocab_size=32))
    assert c.head_dim == 16 and c.num_kv_heads == 4 and c.rope_kind == 0
    assert abs(c.rms_norm_eps - 1e-5) < 1e-12 and c.rope_theta == 500000.0 and c.tie_word_embeddings == 0
    with pytest.raises(B2Error) as e:
        eng.model_config_from_json(dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, vocab_size=32))
    assert e.value.code == -4 and "intermediate_size" in str(e.value)
    q = eng.model_config_from_json(dict(architectures=["Qwen3ForCausalLM"], hidden_size=1024, intermediate_size=3072,
                                        num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                                        vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=True,
                                        max_position_embeddings=40960))
    assert q.qk_norm == 1 and q.head_dim == 128 and q.tie_word_embeddings == 1 and q.rope_kind == 0
    qz = eng.model_config_from_json(dict(model_type="llama", hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                         num_attention_heads=4, vocab_size=32, quantization=dict(group_size=64, bits=4)))
    assert (qz.quant_bits, qz.quant_group) == (4, 64)
    bare = eng.model_config_from_json(dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                           vocab_size=32, rope_scaling=dict(factor=4.0)))
    assert bare.rope_kind == 1 and bare.rope_factor == 4.0 and bare.rope_high_freq_factor == 4.0  # a bare factor block is llama3
    yarn = eng.model_config_from_json(dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                           vocab_size=32, rope_scaling=dict(type="yarn", factor=4.0)))
    assert yarn.rope_kind == 0
    for arch in ("Gemma2ForCausalLM", "DeepseekV2ForCausalLM", "Qwen3VLForConditionalGeneration", "Phi3ForCausalLM", "FooBar"):
        with pytest.raises(B2Error) as e:
            eng.model_config_from_json(dict(architectures=[arch], hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                            num_attention_heads=4, vocab_size=32))
        assert e.value.code == -5
    with pytest.raises(B2Error):
        eng.model_config_from_json("{not json")


def test_rope_host_functions_match_oracle(lib):
    from mlx_llm_b200 import kernels as K
    from oracle import oracle as orc

    for hd, theta, kind in [(64, 10000.0, 0), (128, 500000.0, 1), (128, 1000000.0, 0)]:
        inv = K.rope_inv_freq(hd, theta, kind, 8.0, 1.0, 4.0, 8192.0)
        assert np.array_equal(inv, orc.rope_inv_freq(hd, theta, kind, 8.0, 1.0, 4.0, 8192.0))
        cos, sin = K.rope_tables(inv, 512)
        oc, os_ = orc.rope_cos_sin(inv, np.arange(512, dtype=np.int32))
        assert np.array_equal(cos, oc[:, : hd // 2]) and np.array_equal(sin, os_[:, : hd // 2])


def write_safetensors(path, tensors):
    header, blobs, off = {}, [], 0
    for name, (dtype, arr) in tensors.items():
        b = np.ascontiguousarray(arr).tobytes()
        header[name] = dict(dtype=dtype, shape=list(arr.shape), data_offsets=[off, off + len(b)])
        blobs.append(b)
        off += len(b)
    header["__metadata__"] = {"format": "pt"}
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def test_weights_from_safetensors_file_and_dir(lib, tmp_path):  # weights.rs:100-131
    from mlx_llm_b200 import engine as eng
    from mlx_llm_b200._lib import B2Error

    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = H.f32_to_bf16_np(np.ones((2, 2), np.float32))
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {"model.a.weight": ("F32", a)})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {"model.b.weight": ("BF16", b), "x.packed": ("U32", np.zeros(4, np.uint32))})
    w = eng.Weights.from_dir(tmp_path)
    assert w.contains("model.a.weight") and w.contains("model.b.weight") and w.contains("x.packed") and not w.contains("nope")
    w.free()
    w1 = eng.Weights.from_file(tmp_path / "model-00001-of-00002.safetensors")
    assert w1.contains("model.a.weight") and not w1.contains("model.b.weight")
    w1.free()
    with pytest.raises(B2Error) as e:
        eng.Weights.from_dir(tmp_path / "missing")
    assert e.value.code == -3
    (tmp_path / "empty").mkdir()
    with pytest.raises(B2Error):
        eng.Weights.from_dir(tmp_path / "empty")
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(B2Error):
        eng.Weights.from_file(bad)
    w2 = eng.Weights()
    w2.add("t", a)
    assert w2.contains("t")
    w2.free()


def test_page_policy_oracle_is_self_consistent():
    """The numpy restatement of the page allocator: page 0 first, most recently freed first."""
    from oracle import batch_meta as bm

    pool = bm.PagePool(8, 16)
    a, b = bm.SeqPages(pool, 0), bm.SeqPages(pool, 1)
    assert a.reserve(17) == [(0, 0, 0), (0, 1, 1)]
    a.commit(17)
    assert b.reserve(1) == [(1, 0, 2)]
    b.commit(1)
    assert a.reserve(15) == [] and a.reserve(16) == [(0, 2, 3)]
    b.free()
    c = bm.SeqPages(pool, 1)
    assert c.reserve(1) == [(1, 0, 2)]
    bt = np.zeros((2, 4), np.int32)
    meta = bm.build_batch_metadata([0, 1], [16, 1], [17, 0], [0, 1], bt, [(0, 0, 0), (0, 1, 1), (0, 2, 3), (1, 0, 2)], 64, 64, 16)
    assert meta["cu_seqlens"].tolist() == [0, 16, 17] and meta["context_lens"].tolist() == [33, 1]
    assert meta["slot_mapping"][:2].tolist() == [1 * 16 + 1, 1 * 16 + 2] and meta["slot_mapping"][15] == 3 * 16 + 0
    assert meta["slot_mapping"][16] == 2 * 16 and meta["logit_rows"].tolist() == [16] and meta["dec_ctx"].tolist() == [1]
    assert meta["pf_seq"].tolist() == [0] and meta["counts"].tolist() == [1, 1, 1, 1, 0, 17]


def test_ngram_proposer_matches_its_restatement(lib):
    """b2_ngram_propose (host code, no GPU) against oracle/policies.py on random small-alphabet histories."""
    from mlx_llm_b200 import engine as eng
    from oracle import policies as pol

    rng = np.random.default_rng(0)
    for _ in range(300):
        h = rng.integers(0, 4, size=int(rng.integers(0, 40))).tolist()
        n, k = int(rng.integers(1, 5)), int(rng.integers(0, 7))
        assert eng.ngram_propose(h, n, k) == pol.ngram_propose(h, n, k), (h, n, k)
    assert eng.ngram_propose([1, 2, 3, 9, 1, 2, 3], 3, 4) == [9, 1, 2, 3]      # longest n-gram first, copy to the end
    assert eng.ngram_propose([7, 1, 2, 8, 1, 2, 5, 1, 2], 2, 1) == [5]           # the most recent earlier occurrence
    assert eng.ngram_propose([1, 2, 3], 3, 2) == []


def test_prefix_policy_restatement():
    """The host policy of the prefix cache: longest stored prefix, whole-prompt cap, LRU, subsumed entries."""
    from oracle import policies as pol

    p = pol.PrefixPolicy(2)
    assert p.lookup([1, 2, 3, 4]) == 0
    p.store([1, 2, 3, 4, 9], 4)
    assert p.lookup([1, 2, 3, 7]) == 3 and p.lookup([1, 2, 3, 4]) == 3      # whole-prompt match keeps one token to compute
    assert p.lookup([1, 2, 3, 4, 9, 9]) == 4                                 # never beyond the stored KV
    p.store([5, 6], 1)
    p.store([1, 2, 3, 4, 9, 9, 9], 6)                                         # subsumes the first entry
    assert [e["tokens"] for e in p.entries] == [[5, 6], [1, 2, 3, 4, 9, 9, 9]]
    p.store([8], 0)
    assert [e["tokens"] for e in p.entries] == [[1, 2, 3, 4, 9, 9, 9], [8]]  # [5, 6] was the least recently used
    assert p.stats == dict(lookups=4, hits=3, reused_prefix_tokens=10, computed_prefill_tokens=8)
