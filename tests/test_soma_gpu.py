"""The soma host loop over the real executor: spawn -> ask_on -> Waking, Thinking, Prefill{done,
total}, Delta..., Answer{tok_in_s, tok_out_s} (shell/src/worlds/soma_bridge.rs:244-313), with the
mind's weights coming from a `.model` container, a model switch, and the running rate means."""
import os
import time

import numpy as np
import pytest

from oracle import ref

import model_file_writer as mfw

pytestmark = pytest.mark.gpu


def _drain(s, until, timeout=60.0):
    evs, t0 = [], time.time()
    while time.time() - t0 < timeout:
        e = s.poll()
        if e is None:
            time.sleep(0.002)
            continue
        evs.append(e)
        if isinstance(e, until):
            return evs
    raise AssertionError("timeout; got %r" % evs)


def test_soma_loop_on_the_engine(ctx, tmp_path):
    from cyb_b200 import soma
    cfg = ref.DecoderConfig(layers=2, d=256, ffn=512, heads=4, kv_heads=2, vocab=320)
    paths = []
    for seed in (5, 6):
        W = ref.make_decoder_weights(cfg, seed=seed)
        p = os.path.join(tmp_path, "mind%d.model" % seed)
        mfw.write_model(p, cfg, W)
        paths.append((p, W))
    status = soma.MindStatus(model=paths[0][0])
    s = soma.Soma.spawn(soma.SomaConfig(max_new_tokens=6, prefill_chunk=300, model_path=paths[0][0]),
                        soma.model_file_engine(ctx, max_seq=1024))
    # prompt of > 600 byte tokens: chunks of 300 rows take the tensor-core prompt path, the rest the decode kernels
    question = "what is six times seven?"
    context = ["earlier: " + "numbers and words " * 30, "before that: " + "more words " * 20]
    s.ask_on(question, context, "ls cd ask")
    evs = _drain(s, (soma.Answer, soma.Error))
    for e in evs:
        status.observe(e)
    kinds = [type(e).__name__ for e in evs]
    assert kinds[0] == "Waking" and kinds[1] == "Thinking" and kinds[-1] == "Answer", kinds
    pre = [e for e in evs if isinstance(e, soma.Prefill)]
    prompt = soma.encode(soma.assemble_prompt(question, context, "ls cd ask"))
    assert len(prompt) > 600 and len(pre) == -(-len(prompt) // 300)
    assert pre[-1].done == pre[-1].total == len(prompt)
    ans = evs[-1]
    deltas = [e for e in evs if isinstance(e, soma.Delta)]
    assert ans.tokens == len(deltas) == 6 and ans.question == question
    assert ans.tok_in_s > 0 and ans.tok_out_s > 0 and ans.tok_per_s > 0
    # the streamed tokens are the teacher's greedy continuation of the same prompt (chunked prefill
    # of 300 + 300 + rest rows: the first two chunks on the bf16 tensor-core path, so compare with a
    # second, single-shot run of the engine rather than with the exact teacher)
    dec = soma.model_file_engine(ctx, max_seq=1024)(paths[0][0])
    dec.reset(1)
    for c0 in range(0, len(prompt), 300):
        dec.prefill(np.asarray([prompt[c0:c0 + 300]], np.int32))
    want = dec.decode(6)[0]
    dec.free()
    assert soma.decode(want) == ans.answer
    assert status.n_speed == 1 and status.avg_tok_out_s == ans.tok_out_s and status.last_tok_per_s == ans.tok_per_s
    # a short ask stays entirely on the decode kernels; the mind does not wake again
    s.ask_on("and seven times six?", [], "")
    evs2 = _drain(s, (soma.Answer, soma.Error))
    for e in evs2:
        status.observe(e)
    assert [type(e).__name__ for e in evs2][0] == "Thinking" and isinstance(evs2[-1], soma.Answer)
    short = soma.encode(soma.assemble_prompt("and seven times six?", [], ""))
    teacher = ref.Decoder(cfg, paths[0][1])
    want2, _ = teacher.generate(np.asarray([short], np.int32), 6)
    assert evs2[-1].answer == soma.decode(want2[0])
    assert status.n_speed == 2 and abs(status.avg_tok_in_s - (ans.tok_in_s + evs2[-1].tok_in_s) / 2) < 1e-6 * status.avg_tok_in_s
    # switching the model: ModelChanged now, Waking on the next question, other weights -> other answer
    s.use_model(paths[1][0])
    evs3 = _drain(s, soma.ModelChanged)
    status.observe(evs3[-1])
    assert status.model == paths[1][0] and status.last_tok_per_s is None
    s.ask_on("and seven times six?", [], "")
    evs4 = _drain(s, (soma.Answer, soma.Error))
    assert [type(e).__name__ for e in evs4][0] == "Waking" and isinstance(evs4[-1], soma.Answer)
    want4, _ = ref.Decoder(cfg, paths[1][1]).generate(np.asarray([short], np.int32), 6)
    assert evs4[-1].answer == soma.decode(want4[0])
    # a missing file is an Error event; the queue moves on
    s.use_model(os.path.join(tmp_path, "absent.model"))
    _drain(s, soma.ModelChanged)
    s.ask_on("anyone there?", [], "")
    assert isinstance(_drain(s, (soma.Answer, soma.Error))[-1], soma.Error)
    s.shutdown()
    ctx.device_status()
