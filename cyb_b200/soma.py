"""Host-side mirror of the interface cyb drives its local mind through.

cyb's shell spawns `soma_kernel::Soma` once (shell/src/worlds/soma_bridge.rs:65),
sends questions with `ask_on(question, context, catalog)` (:144-146), drains
`poll()` once per frame (:242) and reacts to the events Waking, Thinking,
Prefill{done,total}, Delta, Answer{question, answer, concepts, tokens, tok_per_s,
tok_in_s, tok_out_s}, Error and ModelChanged (:244-339); `use_model(path)`
switches weights (shell/src/worlds/models/mod.rs:386).  Asks are served one at a
time on the mind's own thread (:49-52).  soma-kernel itself is not part of the
cyb checkout, so this module restates that contract over the engine's executor:
prompt assembly, chunked prefill with progress, token streaming and the three
rates.  The tokenizer of the real runtime is not available; text is mapped to
byte tokens (one token per UTF-8 byte), which any model with vocab >= 256 accepts.
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional


# ---- events (names and fields as cyb matches on them) ----------------------
@dataclass
class Waking:
    pass


@dataclass
class Thinking:
    pass


@dataclass
class Prefill:
    done: int
    total: int


@dataclass
class Delta:
    text: str


@dataclass
class Answer:
    question: str
    answer: str
    concepts: List[str]
    tokens: int
    tok_per_s: float
    tok_in_s: float
    tok_out_s: float


@dataclass
class Error:
    message: str


@dataclass
class ModelChanged:
    path: str


@dataclass
class SomaConfig:
    max_new_tokens: int = 64
    prefill_chunk: int = 128      # tokens per Prefill progress event
    stop_token: Optional[int] = None
    model_path: Optional[str] = None


@dataclass
class MindStatus:
    """What the mind runs and how its answers went: the running means cyb keeps per answer
    (`MindStatus::push_speed`, shell/src/worlds/models/mod.rs:36-52; fed from the Answer event,
    shell/src/worlds/soma_bridge.rs:303-305; cleared of its last rate when the model changes,
    models/mod.rs:386-394)."""
    model: Optional[str] = None
    last_tok_per_s: Optional[float] = None
    avg_tok_in_s: float = 0.0
    avg_tok_out_s: float = 0.0
    n_speed: int = 0

    def push_speed(self, tok_in_s: float, tok_out_s: float) -> None:
        n = float(self.n_speed)
        self.n_speed += 1
        k = float(self.n_speed)
        self.avg_tok_in_s = (self.avg_tok_in_s * n + tok_in_s) / k
        self.avg_tok_out_s = (self.avg_tok_out_s * n + tok_out_s) / k

    def observe(self, event) -> None:
        """Feed every polled event through here to keep the status current."""
        if isinstance(event, Answer):
            self.last_tok_per_s = event.tok_per_s
            self.push_speed(event.tok_in_s, event.tok_out_s)
        elif isinstance(event, ModelChanged):
            self.model = event.path
            self.last_tok_per_s = None


def model_file_engine(ctx, max_seq: int = 2048):
    """Engine factory over `.model` containers: `factory(path)` reads the container's config, creates a
    decoder of that shape on `ctx` and loads the file into it (what `use_model(path)` followed by
    the next ask amounts to; weights are held until the next switch)."""
    from cyb_b200 import qeng

    def factory(path):
        if path is None:
            raise ValueError("no model chosen (SomaConfig.model_path / use_model)")
        mc, _ = qeng.model_file_config(path, ctx)
        dec = ctx.decoder(layers=mc.layers, d_model=mc.d_model, ffn=mc.ffn, heads=mc.heads, kv_heads=mc.kv_heads,
                          vocab=mc.vocab, head_dim=mc.head_dim, rms_eps=mc.rms_eps, rope_base=mc.rope_base,
                          max_batch=1, max_seq=max_seq)
        dec.load_file(path)
        return dec
    return factory


def encode(text: str) -> List[int]:
    return list(text.encode("utf-8"))


def decode(tokens) -> str:
    return bytes(int(t) & 0xFF for t in tokens).decode("utf-8", errors="replace")


def concepts_of(question: str, answer: str) -> List[str]:
    """Content words shared vocabulary of an exchange (lower-cased, de-duplicated, in order)."""
    seen, out = set(), []
    for w in (question + " " + answer).lower().replace("?", " ").replace(".", " ").replace(",", " ").split():
        if len(w) > 3 and w not in seen:
            seen.add(w)
            out.append(w)
    return out[:8]


def assemble_prompt(question: str, context: List[str], catalog: str) -> str:
    """Standing prompt: command catalog, recalled exchanges (at most 3, clipped to 400 chars as the
    caller does, soma_bridge.rs:165-171), then the question."""
    parts = []
    if catalog:
        parts.append("commands: " + catalog)
    for c in context[:3]:
        parts.append("recall: " + c[:400])
    parts.append("q: " + question)
    parts.append("a:")
    return "\n".join(parts)


class Soma:
    """`Soma.spawn(config, engine_factory)` starts the mind thread.  `engine_factory(path)` returns an
    object with reset(batch), prefill(tokens[1,T]) and decode(steps) -> tokens[1,steps] (the
    engine's Decoder has exactly these), created lazily on the first ask ("waking")."""

    def __init__(self, config: SomaConfig, engine_factory: Callable[[Optional[str]], object]):
        self.config = config
        self._factory = engine_factory
        self._engine = None
        self._asks: "queue.Queue" = queue.Queue()
        self._events: "queue.Queue" = queue.Queue()
        self._model_path = config.model_path
        self._stop = False
        self._thread = threading.Thread(target=self._run, name="soma", daemon=True)
        self._thread.start()

    @classmethod
    def spawn(cls, config: SomaConfig, engine_factory) -> "Soma":
        return cls(config, engine_factory)

    # ---- the caller's side ---------------------------------------------------
    def ask_on(self, question: str, context: List[str], catalog: str) -> None:
        self._asks.put(("ask", question, list(context), catalog))

    def use_model(self, path: str) -> None:
        self._asks.put(("model", path))

    def poll(self):
        try:
            return self._events.get_nowait()
        except queue.Empty:
            return None

    def shutdown(self, timeout: float = 10.0) -> None:
        self._stop = True
        self._asks.put(("stop",))
        self._thread.join(timeout)

    # ---- the mind's thread ---------------------------------------------------
    def _run(self):
        while not self._stop:
            item = self._asks.get()
            try:
                if item[0] == "stop":
                    return
                if item[0] == "model":
                    if self._engine is not None and hasattr(self._engine, "free"):
                        self._engine.free()  # the old weights go before the new ones are mapped
                    self._engine = None  # reload lazily
                    self._model_path = item[1]
                    self._events.put(ModelChanged(item[1]))
                else:
                    self._answer(*item[1:])
            except Exception as e:  # the queue moves on (soma_bridge.rs:322-333)
                self._events.put(Error(str(e)))

    def _answer(self, question, context, catalog):
        import numpy as np
        cfg = self.config
        if self._engine is None:
            self._events.put(Waking())
            self._engine = self._factory(self._model_path)
        self._events.put(Thinking())
        toks = encode(assemble_prompt(question, context, catalog))
        eng = self._engine
        eng.reset(1)
        t0 = time.perf_counter()
        done = 0
        while done < len(toks):
            chunk = toks[done:done + cfg.prefill_chunk]
            eng.prefill(np.asarray([chunk], dtype=np.int32))
            done += len(chunk)
            self._events.put(Prefill(done, len(toks)))
        t_in = time.perf_counter() - t0
        out, t1 = [], time.perf_counter()
        for _ in range(cfg.max_new_tokens):
            tok = int(eng.decode(1)[0][0])
            if cfg.stop_token is not None and tok == cfg.stop_token:
                break
            out.append(tok)
            self._events.put(Delta(decode([tok])))
        t_out = time.perf_counter() - t1
        answer = decode(out)
        n = len(out)
        self._events.put(Answer(question=question, answer=answer, concepts=concepts_of(question, answer), tokens=n,
                                tok_per_s=(len(toks) + n) / max(t_in + t_out, 1e-9),
                                tok_in_s=len(toks) / max(t_in, 1e-9), tok_out_s=n / max(t_out, 1e-9)))
