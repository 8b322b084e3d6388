"""CPU restatements of the host policies around the decode loop -- TEST INFRASTRUCTURE ONLY.

* ngram_propose / generate_prompt_lookup: prompt-lookup speculative decoding (src/decode/speculative.rs:73-171) over
  the oracle's forward.  The verify forward is run one position at a time: in the oracle every row of a forward is
  computed independently, so that equals the packed forward bit for bit.
* PrefixPolicy: what PrefixCache::seed_for / store (src/decode/prefix.rs:92-131) decide, without any tensor: which stored
  sequence a prompt reuses, how much, what is evicted, and the PrefixStats that result.
core_llm::speculative::ngram_propose and core_llm::prefix::PrefixIndex themselves are not part of the reference tree
(parity unpinned): both are restated from the reference's description of them and from their call sites.
"""
import numpy as np


def ngram_propose(history, max_ngram, k):
    """Up to k tokens that followed the most recent earlier occurrence of the trailing n-gram, n = max_ngram .. 1."""
    h = list(history)
    if k <= 0 or len(h) < 2:
        return []
    for n in range(min(max_ngram, len(h) - 1), 0, -1):
        pat = h[len(h) - n:]
        for i in range(len(h) - n - 1, -1, -1):
            if h[i:i + n] == pat:
                return h[i + n:i + n + k]
    return []


def _argmax(row):
    return int(np.argmax(row))  # first maximum: ties go to the lowest index (src/primitives/sampler.rs:221-241)


def generate_prompt_lookup(model, cache, prompt, max_new, max_ngram=3, num_draft=4, stop=()):
    """Returns (tokens, finish_reason, dict(forwards, proposed, accepted)).  finish: 0 stop token, 1 max tokens."""
    stats = dict(forwards=0, proposed=0, accepted=0)
    gen = []
    if max_new == 0:
        return gen, 1, stats
    lg, _ = model.forward([(list(prompt), cache, 0)])
    stats["forwards"] += 1
    history = list(prompt)
    cur = _argmax(lg[0])
    if cur in stop:
        return gen, 0, stats
    gen.append(cur)
    history.append(cur)
    while len(gen) < max_new:
        remaining = max_new - len(gen)
        k_cap = min(num_draft, max(remaining - 1, 0))
        drafts = ngram_propose(history, max_ngram, k_cap) if k_cap else []
        stats["proposed"] += len(drafts)
        verify = [cur] + drafts
        base = cache.offset()
        target = []
        for t in verify:  # one packed forward in the reference; row by row here (identical in the oracle)
            lg, _ = model.forward([([t], cache, cache.offset())])
            target.append(_argmax(lg[0]))
        stats["forwards"] += 1
        accepted = 0
        while accepted < len(drafts) and target[accepted] == drafts[accepted]:
            accepted += 1
        stats["accepted"] += accepted
        cache.truncate(base + 1 + accepted)
        for t in drafts[:accepted] + [target[accepted]]:
            if t in stop:
                return gen, 0, stats
            gen.append(t)
            history.append(t)
            cur = t
            if len(gen) >= max_new:
                return gen, 1, stats
    return gen, 1, stats


class PrefixPolicy:
    """Longest-prefix lookup with least-recently-used eviction over stored token sequences."""

    def __init__(self, capacity):
        self.capacity = capacity
        self.entries = []  # dicts: tokens, kv_len (positions whose KV is stored), used
        self.clock = 0
        self.stats = dict(lookups=0, hits=0, reused_prefix_tokens=0, computed_prefill_tokens=0)

    def lookup(self, prompt):
        """Number of prompt positions reused (0 on a miss); refreshes the matched entry."""
        self.stats["lookups"] += 1
        best, best_len = None, 0
        for e in self.entries:
            lim = min(len(e["tokens"]), len(prompt), e["kv_len"])
            common = 0
            while common < lim and e["tokens"][common] == prompt[common]:
                common += 1
            common = min(common, len(prompt) - 1)
            if common > best_len or (common == best_len and common > 0 and e["used"] > best["used"]):
                best, best_len = e, common
        if best is not None and best_len > 0:
            self.clock += 1
            best["used"] = self.clock
            self.stats["hits"] += 1
            self.stats["reused_prefix_tokens"] += best_len
        self.stats["computed_prefill_tokens"] += len(prompt) - best_len
        return best_len

    def store(self, tokens, kv_len):
        tokens = list(tokens)
        self.entries = [e for e in self.entries if not (len(e["tokens"]) <= len(tokens) and e["tokens"] == tokens[:len(e["tokens"])])]
        self.clock += 1
        self.entries.append(dict(tokens=tokens, kv_len=kv_len, used=self.clock))
        while len(self.entries) > self.capacity:
            self.entries.remove(min(self.entries, key=lambda e: e["used"]))
