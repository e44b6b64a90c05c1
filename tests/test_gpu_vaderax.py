"""The Vaderax decoder on the GPU: the package's kernels against the plain implementation (whole models in both
dtypes, the same cases as on the CPU), and each new kernel alone against the plain functions."""
import math

import numpy as np
import pytest
import torch

import plain_vaderax as plain
import vaderax_cases as cases
from safuvik_tiny import tokens_for, rel_err
from vaderax_tiny import CONFIGS, make_tensors
from rbitnet_b200.config import config_from_dict

pytestmark = pytest.mark.gpu

# Fractions of the largest reference value.  float32: the weights are scaled up so that faults show, which amplifies
# rounding.  bfloat16: operands of the products, q/k/v, the cache, the attention's P and the experts' inner rows are
# rounded to 8 bits.
TOL = {"float32": 2e-4, "bfloat16": 6e-2}
# whole models: measured in bfloat16 on these configurations with matrices spread by 4, the median position differs by
# 0.3 to 0.9 %, nine of ten by less than 2.3 %, and single positions where a router's choice fell the other way by up to 15 %
BAND = {"float32": cases.Band(2e-4), "bfloat16": cases.Band(6e-2, spikes=0.1, spread=4.0)}
DTYPES = ["float32", "bfloat16"]


def engine_maker(dtype):
    from rbitnet_b200.engine import Engine

    def make(cfg, tensors, max_tokens=64 * 16, graphs=False, **kw):
        return Engine(config_from_dict(cfg), dict(tensors), dtype=dtype, max_tokens=max_tokens, max_seq=1024,
                      use_graphs=graphs, **kw)
    return make


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole(name, dtype):
    cases.whole(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_prefill_against_decoding(name, dtype):
    cases.prefill_against_decoding(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "D"])
def test_portions(name, dtype):
    cases.portions(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_batches(name, dtype):
    cases.batches_against_alone(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_slots_and_pages_used_again(name, dtype):
    cases.slots_and_pages_used_again(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "E"])
def test_long_decoding(name, dtype):
    cases.long_decoding(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens(name, dtype):
    cases.first_tokens(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("conv", [1, 3])
def test_far_token_through_the_state(conv):
    # float32 only: what the first token of 180 leaves in the last logits is of the size of bfloat16's rounding
    cases.far_token_moves_the_logits(engine_maker("float32"), cases.delta_only(conv), TOL["float32"], least=10.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,far,cuts", [(300, 2, []), (300, 63, [250] + list(range(290, 300))), (200, 64, list(range(1, 200))),
                                        (700, 0, [64, 128, 699]), (130, 127, [129])])
def test_one_far_key(n, far, cuts, dtype):
    cases.one_far_key_stands_out(engine_maker(dtype), TOL[dtype], n, far, cuts, last_only=dtype == "bfloat16")


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_greedy_generation_through_captured_steps(name):
    cases.greedy_generation(engine_maker("float32"), name)


def test_captured_step_in_bfloat16():
    """The captured decode step (padding rows, state saved around the trial run) against the plain model."""
    from rbitnet_b200.engine.step import StepEntry
    cfg = CONFIGS["A"]
    tensors = make_tensors(cfg, 23)
    eng = engine_maker("bfloat16")(cfg, tensors, graphs=True)
    reqs = [tokens_for(cfg, n, 70 + n) for n in (20, 9, 33)]
    slots = [eng.new_sequence() for _ in reqs]
    eng.step([StepEntry(s, r[:-6], []) for s, r in zip(slots, reqs)])
    got = [[] for _ in reqs]
    for k in range(6, 0, -1):
        out = eng.step([StepEntry(s, [r[-k]], [0]) for s, r in zip(slots, reqs)], captured=True)
        for i in range(len(reqs)):
            got[i].append(out[i:i + 1])
    for i, r in enumerate(reqs):
        assert rel_err(torch.cat(got[i]).float().cpu(), plain.forward(cfg, tensors, r)[-6:]) <= TOL["bfloat16"]


# ---------------------------------------------------------------- kernels alone
def _ops(dtype):
    from rbitnet_b200.kernels.ops import CudaOps
    return CudaOps(dtype)


def _meta(ops, runs):
    """runs: (slot, start, n) per sequence."""
    from rbitnet_b200.engine.step import SeqChunk, build_meta
    chunks, at = [], 0
    for slot, start, n in runs:
        chunks.append(SeqChunk(slot, start, n, at))
        at += n
    return build_meta(chunks, np.zeros(at, dtype=np.int32), np.zeros(0, dtype=np.int32), ops.device)


@pytest.mark.parametrize("T,E", [(1, 64), (7, 100), (300, 1000), (3, 4100), (5, 7)])
def test_layer_norm_kernel(T, E):
    ops = _ops(torch.float32)
    g = torch.Generator().manual_seed(E)
    x = torch.randn(T, E, generator=g, dtype=torch.float64) * 3 + 5          # a mean far from zero
    w, b = torch.randn(E, generator=g, dtype=torch.float64), torch.randn(E, generator=g, dtype=torch.float64)
    got = ops.layernorm(x.float().cuda(), w.float().cuda(), b.float().cuda(), 1e-5)
    assert rel_err(got.cpu(), plain.layer_norm(x, w, b, 1e-5)) <= 1e-5
    got = ops.layernorm(x.float().cuda(), w.float().cuda(), None, 1e-5)
    assert rel_err(got.cpu(), plain.layer_norm(x, w, 0.0, 1e-5)) <= 1e-5


@pytest.mark.parametrize("n_experts,identity,top,groups", [(16, 4, 4, (4, 3)), (5, 0, 1, None), (3, 3, 3, (3, 3)), (60, 4, 6, (8, 3)),
                                                           (7, 2, 2, (3, 1)), (2, 0, 2, None), (130, 30, 8, (40, 5))])
@pytest.mark.parametrize("T,K", [(50, 48), (333, 100), (7, 70)])
def test_router_kernel(n_experts, identity, top, groups, T, K):
    """Scores, the choice among the kept groups by score plus correction, weights without it; corrections large
    enough to change the choice, and negative choice scores in whole groups.  Few tokens (a block per token) and many
    (the router's sums as a tiled product), inner sizes that are and are not multiples of 4."""
    ops = _ops(torch.float32)
    g = torch.Generator().manual_seed(n_experts * 10 + top)
    n = n_experts + identity
    h = torch.randn(T, K, generator=g).double()
    w = {"router": torch.randn(n, K, generator=g).double() * 0.3, "correction": torch.randn(n, generator=g).double() * 0.2 - 0.3}
    r = {"experts": n_experts, "identity": identity, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    want_ids, want_w = plain.route(h, r, w)
    ids, weights = ops.route(h.float().cuda(), w["router"].float().cuda(), w["correction"].float().cuda(), top,
                             groups[0] if groups else 0, groups[1] if groups else 0)
    ids, weights = ids.cpu().long(), weights.cpu().double()
    for t in range(T):
        assert sorted(ids[t].tolist()) == sorted(want_ids[t].tolist()), t
        order = torch.argsort(ids[t]), torch.argsort(want_ids[t])
        assert float((weights[t][order[0]] - want_w[t][order[1]]).abs().max()) <= 3e-6
    # the correction decides: without it other experts are chosen somewhere
    other, _ = plain.route(h, r, {"router": w["router"], "correction": torch.zeros(n, dtype=torch.float64)})
    assert any(sorted(other[t].tolist()) != sorted(want_ids[t].tolist()) for t in range(T)) or top == n or T < 50


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,F,n_experts,identity,top", [(1, 64, 40, 6, 2, 2), (3, 64, 40, 6, 2, 4), (70, 64, 24, 3, 0, 1),
                                                          (300, 128, 72, 16, 4, 4), (45, 100, 36, 4, 1, 2), (9, 64, 44, 2, 6, 3),
                                                          (2500, 64, 32, 5, 0, 2), (33, 64, 40, 0, 3, 2)])
def test_routed_experts(dtype, T, E, F, n_experts, identity, top):
    """Few pairs and many, tiles of every size, experts without any token, identity experts, a width and an inner
    size that the tensor-core products refuse."""
    from rbitnet_b200.parts.feed_forward import RoutedExperts
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(T + E)
    part = RoutedExperts(E, F, n_experts, top, n_identity=identity)
    w = {k: (torch.randn(*shape, generator=g) * (0.5 if len(shape) > 1 else 0.1)).to(torch.bfloat16).double()
         for k, (shape, _) in part.weight_shapes().items()}
    if n_experts > 2:
        w["correction"][1] = -10.0            # an expert that nobody chooses
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    h = torch.randn(T, E, generator=g).to(torch.bfloat16).double()
    mlp = {"router": {"experts": n_experts, "identity": identity, "top": top}}
    want = plain.routed_ff(h, mlp, w)

    class Ctx:
        pass
    ctx = Ctx()
    ctx.ops = ops
    got = part.forward(ctx, h.to(dtype).cuda())
    assert rel_err(got.cpu(), want) <= (1e-5 if dtype == torch.float32 else 2e-2)
    x = torch.randn(T, E, generator=g).float().cuda()
    before = x.clone()
    part.forward(ctx, h.to(dtype).cuda(), accumulate_into=x)
    assert rel_err((x - before).cpu(), want) <= (1e-5 if dtype == torch.float32 else 2e-2)
    ops.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [5, 100, 400])
def test_dense_feed_forward(dtype, T):
    from rbitnet_b200.parts.feed_forward import Dense
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(T)
    E, F = 64, 88
    part = Dense(E, F)
    w = {k: (torch.randn(*shape, generator=g) * 0.4).to(torch.bfloat16).double() for k, (shape, _) in part.weight_shapes().items()}
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    h = torch.randn(T, E, generator=g).to(torch.bfloat16).double()

    class Ctx:
        pass
    ctx = Ctx()
    ctx.ops = ops
    assert rel_err(part.forward(ctx, h.to(dtype).cuda()).cpu(), plain.dense_ff(h, w)) <= (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("chunks,one_launch", [(True, True), (False, False), (True, False)])
@pytest.mark.parametrize("H,G,D,Dv,K", [(4, 2, 16, 24, 3), (1, 1, 40, 8, 1), (6, 3, 32, 64, 4), (2, 2, 128, 64, 2), (3, 1, 100, 33, 5),
                                        (2, 1, 8, 130, 2), (1, 1, 300, 20, 3), (2, 2, 600, 8, 2), (2, 1, 30, 16, 2)])
def test_gated_delta_kernels(H, G, D, Dv, K, chunks, one_launch):
    """Whole runs, portions and single tokens through the state and the convolution's ring; key sizes that one to
    thirty-two lanes hold; decays near one, so that the memory of the first tokens is still there at the end.  Runs of
    several tokens in chunks of 32 (a run of 100 tokens ends inside its fourth chunk) and token by token; single tokens
    in the one kernel of a decode step and in the kernels of a prompt."""
    from rbitnet_b200.parts.delta import GatedDeltaRule
    ops = _ops(torch.float32)
    ops.delta_in_chunks = chunks
    ops.fuse_delta_step = one_launch
    g = torch.Generator().manual_seed(H * 1000 + D)
    E, T = 32, 100
    part = GatedDeltaRule(E, H, G, D, Dv, K, norm_eps=1e-5)
    w = {k: torch.randn(*shape, generator=g, dtype=torch.float64) * (0.3 if len(shape) > 1 and not k.endswith("conv") else 1.0)
         for k, (shape, _) in part.weight_shapes().items()}
    w["A_log"] = w["A_log"] - 3.0
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    h = torch.randn(T, E, generator=g, dtype=torch.float64)
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv}
    want = plain.delta_mixer(h, m, w, 1e-5)

    class Ctx:
        def state_view(self, entry):
            return state
    for cuts in ([0, T], [0, 1, 2, 20, 36, 37, T], list(range(T + 1)), [0, 32, 33, 97, T], [0, 64, T]):
        state = {k: torch.zeros((3, *n.shape), device="cuda") for k, n in part.state_need().items()}
        outs = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            ctx = Ctx()
            ctx.ops = ops
            ctx.meta = _meta(ops, [(1, a, b - a)])
            outs.append(part.forward(ctx, h[a:b].float().cuda(), 0))
        assert rel_err(torch.cat(outs).cpu(), want) <= 2e-4, cuts
        assert float(state["S"][0].abs().max()) == 0.0 and float(state["S"][2].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Kh,D,Dv,rot", [(4, 2, 32, 16, 8), (2, 2, 16, 40, 16), (3, 1, 24, 24, 0), (4, 2, 64, 64, 32), (2, 1, 128, 96, 64),
                                           (1, 1, 200, 8, 2)])
def test_attention_part(dtype, H, Kh, D, Dv, rot):
    """The attention with its rotation in pairs (i, i + dims/2), the norm per head after it and the gate per value,
    through the paged cache: whole, in portions across a page border, and token by token."""
    from rbitnet_b200.cache import SequenceCache
    from rbitnet_b200.parts.attention import Attention
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(H * 100 + D)
    E, T = 64, 90
    position = {"kind": "rotary", "params": {"head_dim": D, "theta": 30.0, "pairing": "half", "rot_dim": rot}} if rot else None
    part = Attention(E, H, Kh, D, position=position, scale=0.4, value_dim=Dv, qk_norm="head", norm_eps=1e-5, value_gate=True)
    w = {k: (torch.randn(*shape, generator=g) * 0.3).to(torch.bfloat16).double() for k, (shape, _) in part.weight_shapes().items()}
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    h = torch.randn(T, E, generator=g).to(torch.bfloat16).double()
    m = {"heads": H, "kv_heads": Kh, "dim": D, "vdim": Dv, "scale": 0.4}
    if rot:
        m["rot"] = {"base": 30.0, "dims": rot}
    want = plain.attention(h, m, w, 1e-5)
    for cuts in ([0, T], [0, 60, 64, 65, T], [0, 50] + list(range(51, T + 1))):
        cache = SequenceCache({0: part.cache_need()}, {}, {}, 64 * 4, 1024, dtype, ops.device)
        cache.alloc()
        slot = cache.alloc()

        class Ctx:
            def cache_view(self, entry):
                return cache.view(0)
        outs = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            cache.reserve(slot, b - a)
            cache.upload_tables()
            ctx = Ctx()
            ctx.ops = ops
            ctx.meta = _meta(ops, [(slot, a, b - a)])
            outs.append(part.forward(ctx, h[a:b].to(dtype).cuda(), 0))
            cache.advance(slot, b - a)
        assert rel_err(torch.cat(outs).cpu(), want) <= (2e-5 if dtype == torch.float32 else 3e-2), cuts
    ops.check_errors()
