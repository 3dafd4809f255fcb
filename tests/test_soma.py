"""The host loop that mirrors soma-kernel's contract (events, serial asks, chunked prefill,
error isolation), on CPU with a fake engine."""
import time

import numpy as np

from cyb_b200 import soma


class FakeEngine:
    def __init__(self, path, script=b" 42."):
        self.path, self.script, self.calls = path, script, []

    def reset(self, batch):
        self.calls.append(("reset", batch))
        self.i = 0

    def prefill(self, tokens):
        self.calls.append(("prefill", tokens.shape[1]))

    def decode(self, steps):
        t = self.script[self.i % len(self.script)]
        self.i += 1
        return np.array([[t]], np.int32)


def _drain(s, until, timeout=10.0):
    evs, t0 = [], time.time()
    while time.time() - t0 < timeout:
        e = s.poll()
        if e is None:
            time.sleep(0.005)
            continue
        evs.append(e)
        if isinstance(e, until):
            return evs
    raise AssertionError("timeout; got %r" % evs)


def test_event_sequence_and_rates():
    made = []
    s = soma.Soma.spawn(soma.SomaConfig(max_new_tokens=4, prefill_chunk=16), lambda p: made.append(FakeEngine(p)) or made[-1])
    s.ask_on("what is six times seven?", ["earlier: numbers " * 40], "ls cd ask")
    evs = _drain(s, soma.Answer)
    kinds = [type(e).__name__ for e in evs]
    assert kinds[0] == "Waking" and kinds[1] == "Thinking" and kinds[-1] == "Answer"
    pre = [e for e in evs if isinstance(e, soma.Prefill)]
    assert pre[-1].done == pre[-1].total and all(a.done < b.done for a, b in zip(pre, pre[1:]))
    assert "".join(e.text for e in evs if isinstance(e, soma.Delta)) == " 42."
    a = evs[-1]
    assert a.answer == " 42." and a.tokens == 4 and a.tok_in_s > 0 and a.tok_out_s > 0 and a.tok_per_s > 0
    assert "seven" in a.concepts
    # recalled context is clipped to 400 characters
    assert sum(n for k, n in made[0].calls if k == "prefill") == len(soma.encode(soma.assemble_prompt(
        "what is six times seven?", ["earlier: numbers " * 40], "ls cd ask")))
    # second ask: no second waking, asks are serial
    s.ask_on("again?", [], "")
    evs = _drain(s, soma.Answer)
    assert "Waking" not in [type(e).__name__ for e in evs] and len(made) == 1
    s.shutdown()


def test_errors_do_not_stop_the_queue_and_model_switch():
    class Broken(FakeEngine):
        def prefill(self, tokens):
            raise RuntimeError("device lost")
    engines = []

    def factory(path):
        engines.append(Broken(path) if path == "bad.model" else FakeEngine(path))
        return engines[-1]
    s = soma.Soma.spawn(soma.SomaConfig(max_new_tokens=2, model_path="bad.model"), factory)
    s.ask_on("q1", [], "")
    evs = _drain(s, soma.Error)
    assert "device lost" in evs[-1].message
    s.use_model("good.model")
    assert isinstance(_drain(s, soma.ModelChanged)[-1], soma.ModelChanged)
    s.ask_on("q2", [], "")
    evs = _drain(s, soma.Answer)
    assert evs[-1].question == "q2" and engines[-1].path == "good.model"
    s.shutdown()
