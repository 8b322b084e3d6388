"""Seeded synthetic serving workloads and model shapes of the benchmark configurations.

Llama-3-8B-architecture continuous batching (BASELINE configuration 3): 2048 requests, Poisson
arrivals at 50 req/s, prompt lengths lognormal with median 512 (sigma 1.0 — not given by the
configuration, chosen here) clipped to [16, 8192], output lengths uniform in [64, 512], prompt token
ids uniform over the vocabulary.  No public dataset is involved.
"""
import numpy as np

LLAMA3_8B = dict(num_layers=32, hidden_size=4096, num_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=14336,
                 vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0, rope_kind=1, rope_factor=8.0, rope_low_freq_factor=1.0,
                 rope_high_freq_factor=4.0, rope_original_context=8192.0, qk_norm=0)
QWEN3_32B = dict(num_layers=64, hidden_size=5120, num_heads=64, num_kv_heads=8, head_dim=128, intermediate_size=25600,
                 vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1000000.0, rope_kind=0, rope_factor=1.0, rope_low_freq_factor=1.0,
                 rope_high_freq_factor=4.0, rope_original_context=8192.0, qk_norm=1)
# a 4-layer cut of the 8B shape for quick checks (same per-layer kernels and tile shapes)
LLAMA3_8B_4L = dict(LLAMA3_8B, num_layers=4)


def serving_requests(n=2048, seed=0, rate=50.0, vocab=128256, median_prompt=512, sigma=1.0, min_prompt=16, max_prompt=8192,
                     min_out=64, max_out=512, poisson=True):
    """Returns (prompts [list of int32 arrays], max_new [n], arrival_s [n])."""
    rng = np.random.default_rng(seed)
    plen = np.clip(np.rint(np.exp(rng.normal(np.log(median_prompt), sigma, size=n))), min_prompt, max_prompt).astype(np.int64)
    out = rng.integers(min_out, max_out + 1, size=n).astype(np.int64)
    arrival = np.cumsum(rng.exponential(1.0 / rate, size=n)) if poisson else np.zeros(n)
    prompts = [rng.integers(0, vocab, size=int(p), dtype=np.int32) for p in plen]
    return prompts, out, arrival


def long_context_requests(n=512, seed=0, vocab=151936, min_prompt=1024, max_prompt=32768, max_new=256):
    """BASELINE configuration 4: n sequences, prompt lengths uniform in [min_prompt, max_prompt], max_new outputs each,
    all present at time 0.  Returns (prompts, max_new [n], arrival_s [n])."""
    rng = np.random.default_rng(seed)
    plen = rng.integers(min_prompt, max_prompt + 1, size=n)
    prompts = [rng.integers(0, vocab, size=int(p), dtype=np.int32) for p in plen]
    return prompts, np.full(n, max_new, np.int64), np.zeros(n)


def projection_params(cfg):
    """Weights every token is multiplied with in the projections (per token: 2 flops each)."""
    h, qd, kvd, i = cfg["hidden_size"], cfg["num_heads"] * cfg["head_dim"], cfg["num_kv_heads"] * cfg["head_dim"], cfg["intermediate_size"]
    return cfg["num_layers"] * (h * (qd + 2 * kvd) + qd * h + 3 * h * i)


def step_weight_bytes(cfg, bits):
    """Bytes of weights one decode step streams: projections (quantized: bits/8 + 4 bytes per 64-group)
    plus the bf16 lm_head."""
    p = projection_params(cfg)
    per = bits / 8.0 + 4.0 / 64.0 if bits else 2.0
    return p * per + cfg["vocab_size"] * cfg["hidden_size"] * 2


def kv_bytes_per_token(cfg):
    return cfg["num_layers"] * 2 * cfg["num_kv_heads"] * cfg["head_dim"] * 2
