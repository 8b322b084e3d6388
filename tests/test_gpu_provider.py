"""The serving form of the continuous-batching loop (b2_continuous_open / _submit / _halt / _result) and the TextLlm
provider mirror on top of it, on the GPU: requests that join while others decode produce exactly the tokens of the
single-sequence loop (generate, src/decode/stream.rs:113-121), a halted request ends with the reason it was given, and
concurrent `generate` calls of the provider (src/provider.rs:567-918, text path) share one batch."""
import threading

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    from mlx_llm_b200 import _lib, engine

    ctx = _lib.Context(0)
    cfg = dict(H.CONFIG0, f32_mode=1)  # f32: batched and single-sequence runs give identical tokens
    model = H.build_engine_model(engine, ctx, cfg=cfg)
    yield ctx, engine, model
    model.free()
    ctx.close()


def test_submissions_join_a_running_batch(env):
    ctx, eng, model = env
    prompts = [p.tolist() for p in H.config0_prompts()]
    want = [eng.generate(model, p, max_new_tokens=n).tokens for p, n in zip(prompts, (24, 9, 17, 30))]
    events = {}
    se = eng.ServingEngine(model, eng.ContinuousConfig(max_batch=3, block_size=16, exactness=eng.THROUGHPUT, prefill_chunk_tokens=32,
                                                       max_pages=64, max_blocks_per_seq=16),
                           on_event=lambda rid, ev: events.setdefault(rid, []).append(ev))
    assert se.step(1) is True                                     # idle: nothing submitted yet
    ids = [se.submit(eng.BatchRequest(prompts[0], 24))]
    for _ in range(5):
        se.step(1)
    ids.append(se.submit(eng.BatchRequest(prompts[1], 9)))       # joins while request 0 decodes
    ids.append(se.submit(eng.BatchRequest(prompts[2], 17)))
    ids.append(se.submit(eng.BatchRequest(prompts[3], 30)))      # waits: max_batch is 3
    steps = 0
    while not se.step(1):
        steps += 1
        assert steps < 500
    for rid, w in zip(ids, want):
        out = se.result(rid)
        assert out.tokens == w and out.finish_reason == 1
        toks = [e[1] for e in events[rid] if e[0] == "token"]
        assert toks == w and events[rid][-1] == ("done", 1, len(w))
    # a request that cannot fit a block-table row is refused at submission, the engine stays usable
    with pytest.raises(Exception):
        se.submit(eng.BatchRequest(prompts[3], 1000))
    rid = se.submit(eng.BatchRequest(prompts[1], 5))
    while not se.step(1):
        pass
    assert se.result(rid).tokens == want[1][:5]
    se.free()


def test_halt_ends_one_request_and_leaves_the_others(env):
    ctx, eng, model = env
    prompts = [p.tolist() for p in H.config0_prompts()]
    want = eng.generate(model, prompts[2], max_new_tokens=20).tokens
    events = {}
    se = eng.ServingEngine(model, eng.ContinuousConfig(max_batch=4, block_size=16, exactness=eng.THROUGHPUT, prefill_chunk_tokens=64,
                                                       max_pages=64, max_blocks_per_seq=16),
                           on_event=lambda rid, ev: events.setdefault(rid, []).append(ev))
    a = se.submit(eng.BatchRequest(prompts[0], 200))
    b = se.submit(eng.BatchRequest(prompts[2], 20))
    c = se.submit(eng.BatchRequest(prompts[1], 200))
    for _ in range(6):
        se.step(1)
    se.halt(a, 3)   # a stop string matched
    se.halt(c, 2)   # the client went away
    while not se.step(1):
        pass
    assert se.result(a).finish_reason == 3 and events[a][-1][:2] == ("done", 3)
    assert se.result(c).finish_reason == 2 and events[c][-1][:2] == ("done", 2)
    assert 0 < len(se.result(a).tokens) < 200
    assert se.result(b).tokens == want and se.result(b).finish_reason == 1
    se.free()


class IdTokenizer:
    """Token ids 0..1023 <-> characters of a private alphabet (one character per id)."""

    BASE = 0x4E00

    def encode(self, text):
        return [ord(ch) - self.BASE for ch in text]

    def decode(self, ids):
        return "".join(chr(self.BASE + int(i)) for i in ids)


def test_provider_batches_concurrent_generate_calls(env):
    ctx, eng, model = env
    from mlx_llm_b200 import provider as prov

    tok = IdTokenizer()
    prompts = [p.tolist() for p in H.config0_prompts()]
    lens = (20, 12, 16, 25)
    want = [eng.generate(model, p, max_new_tokens=n).tokens for p, n in zip(prompts, lens)]
    p = prov.LlamaProvider(model, tok, config=eng.ContinuousConfig(max_batch=4, block_size=16, exactness=eng.THROUGHPUT,
                                                                    prefill_chunk_tokens=64, max_pages=128, max_blocks_per_seq=16))
    outs, evs = [None] * 4, [[] for _ in range(4)]

    def run(i):
        req = prov.TextLlmRequest([{"role": "user", "content": tok.decode(prompts[i])}], max_new_tokens=lens[i])
        outs[i] = p.generate(req, evs[i].append)

    threads = [threading.Thread(target=run, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    for i in range(4):
        assert outs[i] is not None, "generate did not return"
        assert tok.encode(outs[i].text) == want[i]
        assert outs[i].finish_reason == "length" and outs[i].usage == prov.Usage(len(prompts[i]), lens[i])
        assert [e[1] for e in evs[i][:-1]] == want[i] and evs[i][-1][0] == "done"
    # a stop string: the text of request 0 up to (not including) its 8th and 9th generated characters
    stop = tok.decode(want[0][7:9])
    out = p.complete(prov.TextLlmRequest([{"role": "user", "content": tok.decode(prompts[0])}], max_new_tokens=20, stop=[stop]))
    first = tok.decode(want[0]).find(stop)
    assert out.finish_reason == "stopped" and out.text == tok.decode(want[0])[:first]
    p.close()
