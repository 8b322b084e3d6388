"""Host logic of the TextLlm provider mirror (mlx_llm_b200/provider.py) with the serving engine replaced by a
host-side fake: stop strings over streamed text, event order, cancel, validation, concurrent callers.  The
reference behaviour these follow: src/provider.rs:567-918 (validate, pre-inference cancel :585-587, incremental
detokenisation :748-760, stop strings :659-667 and the flushed tail :884-896, Done with usage :905-912)."""
import threading

import pytest

from mlx_llm_b200 import engine as eng
from mlx_llm_b200 import provider as prov


class ByteTokenizer:
    def encode(self, text):
        return list(text.encode("utf-8"))

    def decode(self, ids):
        return bytes(int(i) % 256 for i in ids).decode("utf-8", errors="ignore")


class FakeServingEngine:
    """Generates, for a request whose prompt is P, the bytes of SCRIPT[P] one per step and per running request."""

    SCRIPT = {}

    def __init__(self, model, config, on_event=None):
        self.on_event = on_event
        self.reqs = []   # [prompt text, max_new, produced, finish]

    def submit(self, r):
        text = bytes(r.prompt_ids).decode()
        self.reqs.append([self.SCRIPT[text].encode(), r.max_new_tokens, 0, -1])
        return len(self.reqs) - 1

    def halt(self, rid, reason=2):
        r = self.reqs[rid]
        if r[3] == -1:
            r[3] = -reason - 10  # pending: reported at the next step, like the engine does

    def step(self, n=1):
        busy = False
        for rid, r in enumerate(self.reqs):
            if r[3] <= -10:
                r[3] = -(r[3] + 10)
                self.on_event(rid, ("done", r[3], r[2]))
                continue
            if r[3] != -1:
                continue
            busy = True
            self.on_event(rid, ("token", r[0][r[2]], r[2]))
            r[2] += 1
            if r[2] >= r[1] or r[2] >= len(r[0]):
                r[3] = 1
                self.on_event(rid, ("done", 1, r[2]))
        return not busy

    def free(self):
        pass


@pytest.fixture
def provider(monkeypatch):
    monkeypatch.setattr(eng, "ServingEngine", FakeServingEngine)
    p = prov.LlamaProvider(model=None, tokenizer=ByteTokenizer())
    yield p
    p.close()


def test_stop_matcher_holds_back_partial_prefixes():
    m = prov.StopMatcher(["END", "\n\n"])
    out = "".join(m.push(p) for p in ["hello E", "N", "D world"])
    assert out == "hello " and m.stopped and m.flush() == ""
    m = prov.StopMatcher(["STOP"])
    out = "".join(m.push(p) for p in ["abc ST", "OX def"]) + m.flush()
    assert out == "abc STOX def" and not m.stopped
    m = prov.StopMatcher(["ab"])
    assert m.push("xa") == "x" and m.flush() == "a"          # the held tail is real output when nothing matched
    assert prov.StopMatcher([]).push("anything") == "anything"


def test_generate_streams_text_then_done(provider):
    FakeServingEngine.SCRIPT = {"say hi": "hello world, this is text"}
    events = []
    out = provider.generate(prov.TextLlmRequest([{"role": "user", "content": "say hi"}], max_new_tokens=11), events.append)
    assert out.text == "hello world" and out.finish_reason == "length"
    assert out.usage == prov.Usage(prompt_tokens=6, generated_tokens=11)
    assert [e[0] for e in events] == ["token"] * 11 + ["done"]
    assert [e[3] for e in events[:-1]] == list(range(11))          # gap-free emit index
    assert "".join(e[2] for e in events[:-1]) == "hello world"
    assert events[-1] == ("done", "length", out.usage)


def test_stop_string_trims_and_halts(provider):
    FakeServingEngine.SCRIPT = {"q": "answer: 42\n\nand more that must not appear" + " ..." * 20000}
    out = provider.generate(prov.TextLlmRequest([{"role": "user", "content": "q"}], max_new_tokens=80000, stop=["\n\n"]))
    assert out.text == "answer: 42" and out.finish_reason == "stopped"
    assert out.usage.generated_tokens < 80000   # the request was halted: the batch did not run it to its budget


def test_unfinished_stop_prefix_is_flushed(provider):
    FakeServingEngine.SCRIPT = {"q": "ends with a half stop EN"}
    out = provider.generate(prov.TextLlmRequest([{"role": "user", "content": "q"}], max_new_tokens=200, stop=["END"]))
    assert out.text == "ends with a half stop EN" and out.finish_reason == "length"


def test_cancel_before_and_during(provider):
    FakeServingEngine.SCRIPT = {"q": "x" * 5000}
    flag = threading.Event()
    flag.set()
    with pytest.raises(prov.Canceled):
        provider.generate(prov.TextLlmRequest([{"role": "user", "content": "q"}], cancel=flag))
    flag = threading.Event()
    seen = []

    def on_event(ev):
        seen.append(ev)
        if len(seen) == 20:
            flag.set()

    out = provider.generate(prov.TextLlmRequest([{"role": "user", "content": "q"}], max_new_tokens=5000, cancel=flag), on_event)
    assert out.finish_reason == "cancelled" and 20 <= out.usage.generated_tokens < 5000
    assert seen[-1][0] == "done"


def test_validate_rejects_sampling_and_empty(provider):
    with pytest.raises(prov.Unsupported):
        provider.generate(prov.TextLlmRequest([{"role": "user", "content": "q"}], temperature=0.7))
    with pytest.raises(prov.Unsupported):
        provider.generate(prov.TextLlmRequest([]))
    assert provider.descriptor().backend == "b200"


def test_concurrent_callers_share_the_engine(provider):
    FakeServingEngine.SCRIPT = {f"p{i}": f"reply number {i} " * (i + 1) for i in range(8)}
    outs = [None] * 8

    def run(i):
        outs[i] = provider.complete(prov.TextLlmRequest([{"role": "user", "content": f"p{i}"}], max_new_tokens=1000))

    threads = [threading.Thread(target=run, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=30)
    for i in range(8):
        assert outs[i] is not None and outs[i].text == f"reply number {i} " * (i + 1)
