"""Shared builders for the test suite: seeded inputs and the tiny random-init decoder of
configuration 0 (2 layers, hidden 256, 4 q / 2 kv heads, head_dim 64, SwiGLU 688, vocab 1024)."""
import numpy as np

INC = np.uint64(0x9E3779B97F4A7C15)


def splitmix_stream(seed, n):
    """First n outputs of SplitMix64(seed) (src/primitives/sampler.rs:36-61), vectorised."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + (np.arange(1, n + 1, dtype=np.uint64)) * INC
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def splitmix_f32(seed, n):
    return ((splitmix_stream(seed, n) >> np.uint64(40)).astype(np.float32)) / np.float32(1 << 24)


class NormalStream:
    """N(0,1) draws from one SplitMix64 stream via Box-Muller, two uniforms per value, in draw order."""

    def __init__(self, seed):
        self.seed = seed
        self.used = 0

    def normal(self, n):
        u = splitmix_f32(self.seed, self.used + 2 * n)[self.used:]
        self.used += 2 * n
        u1 = np.maximum(u[0::2].astype(np.float64), 2.0 ** -25)
        u2 = u[1::2].astype(np.float64)
        return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)


CONFIG0 = dict(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, inter=688, vocab=1024, eps=1e-5, theta=10000.0,
               rope_kind=0, rope_factor=1.0, rope_low=1.0, rope_high=4.0, rope_orig=8192.0, qk_norm=0, quant_bits=0, group=64,
               f32_mode=0)
CONFIG0_PROMPT_LENS = [17, 33, 64, 129]


def tiny_weights(cfg=CONFIG0, seed=0, std=0.02):
    """Weights ~ N(0, std) drawn from SplitMix64(seed) in the order: embed, lm_head, then per layer
    q, k, v, o, gate, up, down.  Norm weights are ones."""
    ns = NormalStream(seed)
    H, qd, kvd, I, V = cfg["hidden"], cfg["heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"], cfg["inter"], cfg["vocab"]
    w = {"embed": (ns.normal(V * H) * std).reshape(V, H), "lm_head": (ns.normal(V * H) * std).reshape(V, H), "layers": []}
    shapes = dict(q=(qd, H), k=(kvd, H), v=(kvd, H), o=(H, qd), gate=(I, H), up=(I, H), down=(H, I))
    for _ in range(cfg["layers"]):
        w["layers"].append({k: (ns.normal(s[0] * s[1]) * std).reshape(s) for k, s in shapes.items()})
    return w


def config0_prompts(seed=1, vocab=1024, lens=CONFIG0_PROMPT_LENS):
    u = splitmix_f32(seed, sum(lens))
    ids = np.minimum((u * vocab).astype(np.int32), vocab - 1)
    out, o = [], 0
    for n in lens:
        out.append(ids[o:o + n].copy())
        o += n
    return out


def build_oracle_model(orc, cfg=CONFIG0, weights=None, quant_bits=0):
    """Load the tiny weights into an oracle model; quant_bits quantizes the projections on load."""
    weights = weights or tiny_weights(cfg)
    m = orc.Model(**cfg)
    m.set_dense(0, "embed", weights["embed"])
    m.set_dense(0, "lm_head", weights["lm_head"])
    m.set_norm(0, "norm", np.ones(cfg["hidden"], np.float32))
    for l, lw in enumerate(weights["layers"]):
        for k, v in lw.items():
            m.set_dense(l, k, v)
            if quant_bits:
                m.quantize_projection(l, k, quant_bits)
        m.set_norm(l, "input_ln", np.ones(cfg["hidden"], np.float32))
        m.set_norm(l, "post_ln", np.ones(cfg["hidden"], np.float32))
        if cfg.get("qk_norm"):
            m.set_norm(l, "q_norm", np.ones(cfg["head_dim"], np.float32))
            m.set_norm(l, "k_norm", np.ones(cfg["head_dim"], np.float32))
    return m


def lcg_randf(n, seed):
    """The reference attention tests' input generator (src/primitives/attention.rs:312-322)."""
    out = np.empty(n, np.float32)
    s = seed & 0xFFFFFFFFFFFFFFFF
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = np.float32(np.float32(s >> 40) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)
    return out


def f32_to_bf16_np(x):
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16), numpy only."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> np.uint64(16)) & np.uint64(1)
    return ((u + np.uint64(0x7FFF) + lsb) >> np.uint64(16)).astype(np.uint16)


def bf16_to_f32_np(h):
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def make_paged_case(seed, ctx_lens, hq, hkv, hd, page, q_lens=None, pool_factor=2):
    """Seeded paged-KV case: N(0,1) q/K/V in bf16, pool of pool_factor x the needed pages, block
    tables drawn from a random permutation of the physical pages (BASELINE configuration 1)."""
    rng = np.random.default_rng(seed)
    ctx_lens = np.asarray(ctx_lens, np.int32)
    n = ctx_lens.size
    q_lens = np.ones(n, np.int32) if q_lens is None else np.asarray(q_lens, np.int32)
    pages_per = (ctx_lens + page - 1) // page
    total = int(pages_per.sum())
    pool_pages = max(1, pool_factor * total)
    perm = rng.permutation(pool_pages).astype(np.int32)
    max_blocks = int(max(1, pages_per.max()))
    bt = np.zeros((n, max_blocks), np.int32)
    o = 0
    for i in range(n):
        bt[i, : pages_per[i]] = perm[o:o + pages_per[i]]
        o += pages_per[i]
    kpool = f32_to_bf16_np(rng.standard_normal((pool_pages, hkv, page, hd), dtype=np.float32))
    vpool = f32_to_bf16_np(rng.standard_normal((pool_pages, hkv, page, hd), dtype=np.float32))
    T = int(q_lens.sum())
    q = f32_to_bf16_np(rng.standard_normal((T, hq, hd), dtype=np.float32))
    cu = np.zeros(n + 1, np.int32)
    cu[1:] = np.cumsum(q_lens)
    return dict(q=q, kpool=kpool, vpool=vpool, block_tables=bt, ctx_lens=ctx_lens, cu_seqlens=cu, max_blocks=max_blocks,
                pool_pages=pool_pages, hq=hq, hkv=hkv, hd=hd, page=page, scale=float(hd) ** -0.5)


def hf_weight_names(layer):
    p = f"model.layers.{layer}."
    return dict(q=p + "self_attn.q_proj.weight", k=p + "self_attn.k_proj.weight", v=p + "self_attn.v_proj.weight",
                o=p + "self_attn.o_proj.weight", gate=p + "mlp.gate_proj.weight", up=p + "mlp.up_proj.weight",
                down=p + "mlp.down_proj.weight", input_ln=p + "input_layernorm.weight",
                post_ln=p + "post_attention_layernorm.weight", q_norm=p + "self_attn.q_norm.weight",
                k_norm=p + "self_attn.k_norm.weight")


def engine_config(eng, cfg=CONFIG0, quant_bits=0):
    return eng.model_config(compute_f32=cfg.get("f32_mode", 0), num_layers=cfg["layers"], hidden_size=cfg["hidden"], num_heads=cfg["heads"], num_kv_heads=cfg["kv_heads"],
                            head_dim=cfg["head_dim"], intermediate_size=cfg["inter"], vocab_size=cfg["vocab"], rms_norm_eps=cfg["eps"],
                            rope_theta=cfg["theta"], rope_kind=cfg["rope_kind"], rope_factor=cfg["rope_factor"],
                            rope_low_freq_factor=cfg["rope_low"], rope_high_freq_factor=cfg["rope_high"],
                            rope_original_context=cfg["rope_orig"], qk_norm=cfg.get("qk_norm", 0), quant_bits=quant_bits,
                            quant_group=64 if quant_bits else 0)


def build_engine_model(eng, ctx, cfg=CONFIG0, weights=None, quant=None, tp=None):
    """The same tiny weights as build_oracle_model, handed to the engine as f32 host tensors under
    the Hugging Face key names CausalLm::from_weights reads (src/models/llama.rs:122-181, :245-281)."""
    weights = weights or tiny_weights(cfg)
    w = eng.Weights()
    w.add("model.embed_tokens.weight", weights["embed"])
    w.add("lm_head.weight", weights["lm_head"])
    w.add("model.norm.weight", np.ones(cfg["hidden"], np.float32))
    for l, lw in enumerate(weights["layers"]):
        names = hf_weight_names(l)
        for k, v in lw.items():
            w.add(names[k], v)
        w.add(names["input_ln"], np.ones(cfg["hidden"], np.float32))
        w.add(names["post_ln"], np.ones(cfg["hidden"], np.float32))
        if cfg.get("qk_norm"):
            w.add(names["q_norm"], np.ones(cfg["head_dim"], np.float32))
            w.add(names["k_norm"], np.ones(cfg["head_dim"], np.float32))
    m = eng.CausalLm.from_weights(ctx, w, "", engine_config(eng, cfg), quant, tp=tp)
    w.free()
    return m


def bf16_ulp_diff(a, b):
    """Distance in bf16 ulps between two uint16 bf16 arrays (same-sign finite values)."""
    def key(h):
        h = h.astype(np.int32)
        return np.where(h & 0x8000, 0x8000 - (h & 0x7FFF), 0x8000 + (h & 0x7FFF))
    return np.abs(key(np.asarray(a)) - key(np.asarray(b)))


def close_bf16_out(got_bf16, ref_f32, abs_tol=2e-3):
    """Parity rule for a bf16 output whose unrounded (f32-accumulated) value must lie within `abs_tol` of the
    reference.  Rounding to bf16 is monotonic, so such an output can only be a bf16 number between
    bf16(ref - abs_tol) and bf16(ref + abs_tol): exactly that interval is accepted, nothing wider.  Returns
    (ok, worst absolute difference between the rounded output and the reference)."""
    got = bf16_to_f32_np(got_bf16)
    ref = np.asarray(ref_f32, np.float32)
    tol = np.float32(abs_tol)
    lo = bf16_to_f32_np(f32_to_bf16_np(ref - tol))
    hi = bf16_to_f32_np(f32_to_bf16_np(ref + tol))
    ok = np.isfinite(got) & (got >= lo) & (got <= hi)
    return bool(ok.all()), float(np.abs(got - ref).max())


def weights_crc(w):
    """Checksum of the tiny model's weights (detects a libm that draws different Box-Muller values)."""
    import zlib

    crc = zlib.crc32(np.ascontiguousarray(w["embed"]).tobytes())
    crc = zlib.crc32(np.ascontiguousarray(w["lm_head"]).tobytes(), crc)
    for lw in w["layers"]:
        for k in ("q", "k", "v", "o", "gate", "up", "down"):
            crc = zlib.crc32(np.ascontiguousarray(lw[k]).tobytes(), crc)
    return int(crc)
