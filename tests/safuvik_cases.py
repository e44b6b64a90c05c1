"""Test bodies for the Safuvik decoder that run the same way on the CPU stand-in of the kernel layer and on
the GPU: each takes ``make_engine(cfg_dict, tensors, **kw)`` and a tolerance (a fraction of the largest
reference value), and compares the engine with the plain implementation in float64."""
from __future__ import annotations

import copy

import torch

import plain_safuvik as plain
from safuvik_tiny import CONFIGS, make_tensors, tokens_for, run_cut, rel_err, parallel_layer, _left
from rbitnet_b200.engine.step import StepEntry


def reference(cfg, tensors, tokens):
    return plain.forward(cfg, tensors, tokens, torch.float64)


def whole_and_layers(make_engine, name, tol, n=150):
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=11)
    toks = tokens_for(cfg, n, 5)
    eng = make_engine(cfg, tensors)
    got = run_cut(eng, toks, [])
    assert rel_err(got, reference(cfg, tensors, toks)) <= tol


def prefill_against_decoding(make_engine, name, tol, n=90, prompt=37):
    """A prompt in one step and the rest token by token, and everything token by token, against the whole."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=12)
    toks = tokens_for(cfg, n, 6)
    ref = reference(cfg, tensors, toks)
    eng = make_engine(cfg, tensors)
    assert rel_err(run_cut(eng, toks, list(range(prompt, n))), ref) <= tol
    assert rel_err(run_cut(eng, toks, list(range(1, n))), ref) <= tol


def portions(make_engine, name, tol, n=140):
    """Portions of 2 tokens, of a page, of odd sizes, and a last portion of one token."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=13)
    toks = tokens_for(cfg, n, 7)
    ref = reference(cfg, tensors, toks)
    eng = make_engine(cfg, tensors)
    for cuts in (list(range(2, n, 2)), [64, 128], [3, 8, 9, 63, 65, 127, n - 1], [1, 2, 4, 70]):
        assert rel_err(run_cut(eng, toks, cuts), ref) <= tol, cuts


def batches_against_alone(make_engine, name, tol, lengths=(1, 2, 75, 9, 131), decode=12):
    """Unequal prompts in one step, then decoded together, the shorter requests ending earlier; the slots
    of those that ended are used again by a second batch.  Against each request alone (plain model)."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=14)
    eng = make_engine(cfg, tensors, max_tokens=64 * 8)
    for round_ in range(2):
        reqs = [tokens_for(cfg, n + (decode if i % 2 else decode // 2), 20 + 10 * round_ + i) for i, n in enumerate(lengths)]
        refs = [reference(cfg, tensors, r) for r in reqs]
        slots = [eng.new_sequence() for _ in reqs]
        got = [[] for _ in reqs]
        out = eng.step([StepEntry(s, r[:n], list(range(n))) for s, r, n in zip(slots, reqs, lengths)])
        at = 0
        for i, n in enumerate(lengths):
            got[i].append(out[at:at + n])
            at += n
        fed = list(lengths)
        live = list(range(len(reqs)))
        while live:
            out = eng.step([StepEntry(slots[i], [reqs[i][fed[i]]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                fed[i] += 1
            for i in [i for i in live if fed[i] == len(reqs[i])]:
                eng.end_sequence(slots[i])
                live.remove(i)
        for i in range(len(reqs)):
            assert rel_err(torch.cat(got[i]).float().cpu(), refs[i]) <= tol, (round_, i)


def slots_and_pages_used_again(make_engine, name, tol):
    """A cache of three pages: every sequence gets the pages and the state slot the one before gave back."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=15)
    eng = make_engine(cfg, tensors, max_tokens=64 * 3)
    for k, n in enumerate((130, 70, 150, 5, 129)):
        toks = tokens_for(cfg, n, 40 + k)
        got = run_cut(eng, toks, [n // 2, n - 3, n - 2, n - 1])
        assert rel_err(got, reference(cfg, tensors, toks)) <= tol, k


def long_decoding(make_engine, name, tol, n=200, prompt=3):
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=16)
    toks = tokens_for(cfg, n, 8)
    eng = make_engine(cfg, tensors)
    assert rel_err(run_cut(eng, toks, list(range(prompt, n))), reference(cfg, tensors, toks)) <= tol


def first_tokens(make_engine, name, tol):
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=17)
    eng = make_engine(cfg, tensors)
    for n in (1, 2, 3, 4):
        toks = tokens_for(cfg, n, 50 + n)
        ref = reference(cfg, tensors, toks)
        assert rel_err(run_cut(eng, toks, []), ref) <= tol
        assert rel_err(run_cut(eng, toks, list(range(1, n))), ref) <= tol


def _attention_only(window, dim=16, vdim=8, heads=2, kv=1, rot=8):
    """One parallel layer, no feed-forward, ordinary residual; the tests silence the recurrent branch."""
    return {"architecture": "Safuvik", "vocab": 40, "width": 32, "norm": {"eps": 1e-5},
            "layers": [parallel_layer(_left(heads, kv, dim, vdim, window, rot, None, base=100.0, scale=2.0), 16, 2, 3, None)]}


def window_edges(make_engine, tol, window, n, cuts):
    """With the recurrent branch silenced, the logits at position i depend on tokens i-window+1 .. i and
    on nothing else: changing the token just outside the window must leave them as they were, changing the
    one just inside must move them.  Scores are made sharp so that one key far back would show."""
    cfg = _attention_only(window)
    tensors = make_tensors(cfg, seed=18, spread=10.0)
    tensors["l0.mix.right.out"] = torch.zeros_like(tensors["l0.mix.right.out"])
    toks = tokens_for(cfg, n, 9)
    eng = make_engine(cfg, tensors)
    base = run_cut(eng, toks, cuts)
    assert rel_err(base, reference(cfg, tensors, toks)) <= tol
    most_moved = 0.0
    for i in sorted({n - 1, n - 2, window + 1, min(n - 1, 2 * window), min(n - 1, 64 + window - 1), min(n - 1, 64 + window)}):
        if i - window < 0:
            continue
        outside, inside = list(toks), list(toks)
        outside[i - window] = (toks[i - window] + 7) % cfg["vocab"]
        inside[i - window + 1] = (toks[i - window + 1] + 7) % cfg["vocab"]
        scale = float(base[i].abs().max())
        moved_out = float((run_cut(eng, outside, cuts)[i] - base[i]).abs().max()) / scale
        moved_in = float((run_cut(eng, inside, cuts)[i] - base[i]).abs().max()) / scale
        assert moved_out <= 1e-6, (i, moved_out)          # nothing of it may enter: the same arithmetic on the same values
        most_moved = max(most_moved, moved_in)
    assert most_moved > 0.01, most_moved                  # and what is inside does enter


def far_token_moves_the_logits(make_engine, name, tol, n=180):
    """The recurrent layers forget slowly here: changing the FIRST token must move the last logits, in the
    engine as in the plain model, whether the sequence came whole or was decoded through the state."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=19, long_memory=True)
    toks = tokens_for(cfg, n, 10)
    other = [(toks[0] + 3) % cfg["vocab"]] + toks[1:]
    ref_a, ref_b = reference(cfg, tensors, toks)[-1], reference(cfg, tensors, other)[-1]
    moved = float((ref_a - ref_b).abs().max() / ref_a.abs().max())
    assert moved > 20 * tol, f"the configuration forgets too fast for this test ({moved})"
    eng = make_engine(cfg, tensors)
    for cuts in ([], list(range(100, n))):
        a, b = run_cut(eng, toks, cuts)[-1], run_cut(eng, other, cuts)[-1]
        assert rel_err(a[None], ref_a[None]) <= tol and rel_err(b[None], ref_b[None]) <= tol


def greedy_generation(make_engine, name, prompts=(7, 1, 30), new=24):
    """``Engine.generate`` (scheduler, batches, the captured decode step where there is one) against a
    greedy loop over the plain model."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=21)
    eng = make_engine(cfg, tensors, graphs=True)
    ps = [tokens_for(cfg, n, 60 + i) for i, n in enumerate(prompts)]
    results = eng.generate(ps, max_tokens=new, temperature=0.0, stop_ids=[])
    for p, r in zip(ps, results):
        seq = list(p)
        for step, tok in enumerate(r.tokens):
            logits = reference(cfg, tensors, seq)[-1]
            best = int(torch.argmax(logits))
            if best != tok:
                # a tie within rounding is not a fault; anything else is
                top = torch.topk(logits, 2).values
                assert float(top[0] - logits[tok]) <= 1e-4 * float(logits.abs().max()), (step, best, tok)
            seq.append(tok)
        assert len(r.tokens) == new
