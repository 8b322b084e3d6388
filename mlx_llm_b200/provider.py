"""Host-side mirror of the reference's `core_llm::TextLlm` provider for the text-only path, routed through ONE
continuous-batching engine so that concurrent `generate` calls share a batch.

Reference: `impl TextLlm for LlamaProvider` (src/provider.rs:567-918): validate -> pre-inference cancel -> render the
chat template -> tokenize -> run the decode loop with the stop tokens -> incremental detokenisation of the running
sequence (re-decode, emit the new suffix, provider.rs:748-760) -> stop strings matched in the decoded text, not in the
token ids (provider.rs:659-667; a hit trims the text and halts the loop with `Stopped`) -> `Token{id, text, index,
channel}` events, then exactly one `Done{finish_reason, usage}` -> `TextLlmOutput{text, usage, finish_reason}`.
The reference runs `generate_with` per request (provider.rs:838-846), one sequence at a time; here every call becomes a
request of a shared serving engine (`b2_continuous_open` / `_submit` / `_halt`), which is what SceneWorks' server would
need to batch across connections.

Not mirrored (out of this path's scope): vision inputs, the thinking and tool-call segmenters, JSON constraints,
stochastic sampling (the device path is greedy: other settings are rejected by `validate`).  The tokenizer and the chat
template are the caller's: anything with `encode(text) -> ids` / `decode(ids) -> text`, and a callable
`template(messages) -> prompt text`.  `core_llm`'s types are not vendored in the reference; the names below follow the
fields `provider.rs` uses.
"""
import queue
import threading
from dataclasses import dataclass, field
from typing import Callable, List, Optional

from . import engine as eng

FINISH_NAMES = {eng_code: name for eng_code, name in ((0, "stop_token"), (1, "length"), (2, "cancelled"), (3, "stopped"))}


class ProviderError(Exception):
    pass


class Canceled(ProviderError):
    """Typed pre-inference cancel (provider.rs:585-587)."""


class Unsupported(ProviderError):
    pass


@dataclass
class Capabilities:  # TextLlmCapabilities (provider.rs:926-940)
    max_context_tokens: int = 0      # 0: not limited by the provider (the page pool decides)
    max_new_tokens: int = 0
    supports_system_prompt: bool = True
    supports_streaming: bool = True
    supports_sampling: bool = False  # greedy only on the device path


@dataclass
class TextLlmDescriptor:  # provider.rs:921-945
    id: str = "b200-llama"
    family: str = "llama"
    backend: str = "b200"
    capabilities: Capabilities = field(default_factory=Capabilities)


@dataclass
class TextLlmRequest:
    messages: List[dict]                       # [{"role": ..., "content": ...}]
    max_new_tokens: int = 256
    stop: List[str] = field(default_factory=list)
    temperature: float = 0.0
    seed: Optional[int] = None
    cancel: Optional[threading.Event] = None   # CancelFlag: set by another thread


@dataclass
class Usage:
    prompt_tokens: int
    generated_tokens: int


@dataclass
class TextLlmOutput:
    text: str
    usage: Usage
    finish_reason: str


class StopMatcher:
    """Stop strings over streamed text (`core_llm`'s StopMatcher as provider.rs:659-667 and :600-617 use it): text is
    released as soon as it can no longer be the beginning of a stop string; on a hit everything before the stop string
    is released, the stop string and what follows are dropped, and `stopped` is set."""

    def __init__(self, stops):
        self.stops = [s for s in stops if s]
        self.held = ""
        self.stopped = False

    def __bool__(self):
        return bool(self.stops)

    def push(self, text):
        if self.stopped:
            return ""
        if not self.stops:
            return text
        buf = self.held + text
        hit = min((i for i in (buf.find(s) for s in self.stops) if i >= 0), default=-1)
        if hit >= 0:
            self.stopped = True
            self.held = ""
            return buf[:hit]
        keep = 0  # longest suffix of buf that is a proper prefix of some stop string
        for s in self.stops:
            for k in range(min(len(s) - 1, len(buf)), 0, -1):
                if buf.endswith(s[:k]):
                    keep = max(keep, k)
                    break
        self.held = buf[len(buf) - keep:] if keep else ""
        return buf[:len(buf) - keep] if keep else buf

    def flush(self):
        out, self.held = self.held, ""
        return "" if self.stopped else out


class LlamaProvider:
    """`TextLlm` over a shared continuous-batching engine.  `generate` may be called from many threads at once; a
    single serving thread owns the engine (one context, one thread) and steps it while anything is in flight."""

    def __init__(self, model, tokenizer, template: Optional[Callable[[List[dict]], str]] = None, stop_tokens=(),
                 config: Optional[eng.ContinuousConfig] = None, descriptor: Optional[TextLlmDescriptor] = None):
        self.model = model
        self.tokenizer = tokenizer
        self.template = template or (lambda messages: "".join(m.get("content", "") for m in messages))
        self.stop_tokens = list(stop_tokens)
        self.config = config or eng.ContinuousConfig(max_batch=64, block_size=16, exactness=eng.THROUGHPUT, prefill_chunk_tokens=512,
                                                     max_pages=4096, max_blocks_per_seq=512)
        self._descriptor = descriptor or TextLlmDescriptor()
        self._submit_q = queue.Queue()   # (BatchRequest, per-request event queue)
        self._halt_q = queue.Queue()     # (request id, reason)
        self._streams = {}               # request id -> per-request event queue (serving thread only)
        self._wake = threading.Event()
        self._closing = False
        self._fatal = None
        self._thread = threading.Thread(target=self._serve, name="b200-serving", daemon=True)
        self._thread.start()

    # ---- the serving thread ---------------------------------------------------------------------------
    def _serve(self):
        try:
            engine = eng.ServingEngine(self.model, self.config, on_event=self._on_engine_event)
        except Exception as e:  # report to every caller instead of dying silently
            self._fatal = e
            return
        try:
            idle = True
            while not self._closing:
                if idle and self._submit_q.empty() and self._halt_q.empty():
                    self._wake.wait(0.05)
                    self._wake.clear()
                while True:
                    try:
                        breq, stream = self._submit_q.get_nowait()
                    except queue.Empty:
                        break
                    try:
                        rid = engine.submit(breq)
                        self._streams[rid] = stream
                        stream.put(("id", rid))
                    except Exception as e:
                        stream.put(("error", e))
                while True:
                    try:
                        rid, reason = self._halt_q.get_nowait()
                    except queue.Empty:
                        break
                    engine.halt(rid, reason)
                idle = engine.step(1)
        except Exception as e:
            self._fatal = e
            for stream in self._streams.values():
                stream.put(("error", e))
        finally:
            engine.free()

    def _on_engine_event(self, rid, event):
        stream = self._streams.get(rid)
        if stream is None:
            return
        stream.put(event)
        if event[0] == "done":
            del self._streams[rid]

    def close(self):
        self._closing = True
        self._wake.set()
        self._thread.join(timeout=30)

    # ---- TextLlm ------------------------------------------------------------------------------------------
    def descriptor(self) -> TextLlmDescriptor:
        return self._descriptor

    def validate(self, req: TextLlmRequest):
        cap = self._descriptor.capabilities
        if not req.messages:
            raise Unsupported("request has no messages")
        if req.temperature > 0 and not cap.supports_sampling:
            raise Unsupported("only greedy sampling (temperature 0) runs on the device path")
        if cap.max_new_tokens and req.max_new_tokens > cap.max_new_tokens:
            raise Unsupported(f"max_new_tokens {req.max_new_tokens} exceeds the provider's {cap.max_new_tokens}")
        if not cap.supports_system_prompt and any(m.get("role") == "system" for m in req.messages):
            raise Unsupported("system prompts are not supported")

    def generate(self, req: TextLlmRequest, on_event: Optional[Callable[[tuple], None]] = None) -> TextLlmOutput:
        """Events: ("token", id, text, index) per released piece of text, then one ("done", finish_reason, Usage)."""
        self.validate(req)
        if req.cancel is not None and req.cancel.is_set():
            raise Canceled("canceled before inference")
        if self._fatal:
            raise ProviderError(f"the serving engine is down: {self._fatal}")
        prompt = self.template(req.messages)
        prompt_ids = [int(t) for t in self.tokenizer.encode(prompt)]
        cap = self._descriptor.capabilities
        if cap.max_context_tokens and len(prompt_ids) + req.max_new_tokens > cap.max_context_tokens:
            raise Unsupported("prompt + max_new_tokens exceeds the provider's context")
        stream = queue.Queue()
        self._submit_q.put((eng.BatchRequest(prompt_ids, req.max_new_tokens, list(self.stop_tokens)), stream))
        self._wake.set()
        matcher = StopMatcher(req.stop)
        acc, shown, streamed, emit_index, last_id = [], 0, [], 0, 0
        rid, halted, finish, generated = None, False, None, 0

        def emit(text, tok):
            nonlocal emit_index
            if text:
                streamed.append(text)
                if on_event:
                    on_event(("token", tok, text, emit_index))
                emit_index += 1

        while finish is None:
            try:
                ev = stream.get(timeout=0.05)
            except queue.Empty:
                if self._fatal:
                    raise ProviderError(f"the serving engine is down: {self._fatal}")
                if rid is not None and not halted and req.cancel is not None and req.cancel.is_set():
                    self._halt_q.put((rid, 2))  # Done{Cancelled} follows
                    self._wake.set()
                    halted = True
                continue
            if ev[0] == "id":
                rid = ev[1]
            elif ev[0] == "error":
                raise ev[1] if isinstance(ev[1], Exception) else ProviderError(str(ev[1]))
            elif ev[0] == "token":
                if halted:
                    continue  # tokens the batch produced between the stop hit and the halt taking effect
                last_id = ev[1]
                acc.append(ev[1])
                text = self.tokenizer.decode(acc)
                if len(text) > shown:
                    delta, shown = text[shown:], len(text)
                    emit(matcher.push(delta), last_id)
                    if matcher.stopped:
                        self._halt_q.put((rid, 3))  # Done{Stopped} follows
                        self._wake.set()
                        halted = True
                if not halted and req.cancel is not None and req.cancel.is_set():
                    self._halt_q.put((rid, 2))
                    self._wake.set()
                    halted = True
            elif ev[0] == "done":
                finish, generated = ev[1], ev[2]
        if not matcher.stopped:
            emit(matcher.flush(), last_id)  # a partial stop prefix that never completed is real output
        usage = Usage(len(prompt_ids), generated)
        # a stop string decides the reason even when the batch finished the request before the halt reached it
        reason = "stopped" if matcher.stopped else FINISH_NAMES.get(finish, str(finish))
        if on_event:
            on_event(("done", reason, usage))
        return TextLlmOutput("".join(streamed), usage, reason)

    def complete(self, req: TextLlmRequest) -> TextLlmOutput:
        """`TextLlm::complete`: generate without a listener."""
        return self.generate(req, None)
