"""Generates tests/golden/config0.json: the CPU oracle's greedy token streams, block-id table and
per-step top-2 margins for BASELINE configuration 0 (tiny random-init Llama decoder, seed 0, 4
sequences with prompt lengths 17/33/64/129, page 16, 32 greedy tokens each), in the bf16 arithmetic the
reference computes in and in f32.

The reference itself (Rust + MLX) cannot run here and ships no stored token goldens, so this fixture
pins the oracle's own output against accidental change; the block-id table is additionally the one
derived by hand from the reference's freeze-on-fill rule.

    python tests/golden/gen_config0.py
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from oracle import oracle as orc  # noqa: E402
from tests import helpers as H  # noqa: E402


def main():
    w = H.tiny_weights()
    m = H.build_oracle_model(orc, weights=w)
    prompts = H.config0_prompts()
    out = m.generate_continuous(prompts, [32] * 4)
    margins = []
    for p, toks in zip(prompts, out["tokens"]):
        c = orc.Cache(2, block_size=16)
        _, lf = m.forward([(p, c, 0)])
        row = []
        for t in toks:
            s = np.sort(lf[0])
            row.append(round(float(s[-1] - s[-2]), 6))
            _, lf = m.forward([([t], c, c.offset())])
        margins.append(row)
    # the same model evaluated in f32 (BASELINE configuration 0 as worded): the streams the engine's compute_f32 mode must
    # reproduce token for token
    m32 = H.build_oracle_model(orc, cfg=dict(H.CONFIG0, f32_mode=1), weights=w)
    out32 = m32.generate_continuous(prompts, [32] * 4)
    doc = dict(config=H.CONFIG0, prompt_lens=H.CONFIG0_PROMPT_LENS, weights_crc=H.weights_crc(w),
               prompts=[p.tolist() for p in prompts], tokens=out["tokens"], block_ids=out["block_ids"], pool=out["pool"],
               top2_f32_margins=margins, tokens_f32=out32["tokens"])
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config0.json")
    with open(path, "w") as f:
        json.dump(doc, f, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    main()
