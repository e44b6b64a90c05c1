"""The Safuvik decoder on the GPU: the package's kernels against the plain implementation (whole models
in both dtypes, the same cases as on the CPU), and each new kernel alone against the plain functions."""
import math

import numpy as np
import pytest
import torch

import plain_safuvik as plain
import safuvik_cases as cases
from safuvik_tiny import CONFIGS, make_tensors, tokens_for, run_cut, rel_err
from rbitnet_b200.config import config_from_dict

pytestmark = pytest.mark.gpu

# Fractions of the largest reference value.  float32: the weights are scaled up so that faults show, which
# amplifies rounding (the plain model in float32 differs from itself in float64 by 2e-5 on them).
# bfloat16: operands of the products, q/k/v, the cache and the attention's P are rounded to 8 bits;
# measured 0.6 to 1.9 % on these configurations.
TOL = {"float32": 2e-4, "bfloat16": 5e-2}
DTYPES = ["float32", "bfloat16"]


def tol(dtype, name=""):
    """Configuration D is matrix memories only, with gates capped at 20: a memory's output is divided by |n . q|, which
    is a difference of a few products at the first tokens, and the bfloat16 rounding of the layer's input rows moves
    such an output by up to 9 % of the largest logit (measured, the same request alone or in a batch; in float32 the same
    positions are right to 6e-6).  The band for it in bfloat16 is 12 %; a lost state or a wrong slot moves the
    logits by more than that, and the float32 run of the same case keeps the tight band."""
    if name == "D" and dtype == "bfloat16":
        return 0.12
    # F (three layers, sharp scores over keys of 64 and 128): one position of 90 differs by 2.4 % whole and 5.2 % decoded
    # (the other 89 by 0.4 to 1.6 %, both ways; float32 2e-5 everywhere), so its band is 8 %
    if name == "F" and dtype == "bfloat16":
        return 0.08
    return TOL[dtype]


def engine_maker(dtype):
    from rbitnet_b200.engine import Engine

    def make(cfg, tensors, max_tokens=64 * 16, graphs=False, **kw):
        return Engine(config_from_dict(cfg), dict(tensors), dtype=dtype, max_tokens=max_tokens, max_seq=1024,
                      use_graphs=graphs, **kw)
    return make


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_whole(name, dtype):
    cases.whole_and_layers(engine_maker(dtype), name, tol(dtype, name))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_prefill_against_decoding(name, dtype):
    cases.prefill_against_decoding(engine_maker(dtype), name, tol(dtype, name))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "F"])
def test_portions(name, dtype):
    cases.portions(engine_maker(dtype), name, tol(dtype, name))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_batches(name, dtype):
    cases.batches_against_alone(engine_maker(dtype), name, tol(dtype, name))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_slots_and_pages_used_again(name, dtype):
    cases.slots_and_pages_used_again(engine_maker(dtype), name, TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding(name, dtype):
    cases.long_decoding(engine_maker(dtype), name, TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens(name, dtype):
    cases.first_tokens(engine_maker(dtype), name, TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,n,cuts", [(5, 30, [11, 25, 26, 27, 28, 29]), (64, 150, [100] + list(range(140, 150))),
                                           (65, 140, []), (9, 80, list(range(60, 80)))])
def test_window_edges(window, n, cuts, dtype):
    cases.window_edges(engine_maker(dtype), TOL[dtype] * (3 if dtype == "bfloat16" else 1), window, n, cuts)


@pytest.mark.parametrize("name", ["A", "B"])
def test_far_token(name):
    # float32 only: the first token of 180 moves the last logits by about 1 %, which is bfloat16's rounding
    cases.far_token_moves_the_logits(engine_maker("float32"), name, TOL["float32"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,Kh,D,Dv,window", [(4, 1, 128, 80, 75), (2, 2, 16, 40, 70), (4, 2, 64, 64, 64), (3, 1, 24, 24, 5),
                                              (2, 1, 96, 32, 129)])
def test_one_key_stands_out_at_the_window_edge(H, Kh, D, Dv, window, dtype):
    """Keys and queries are made by hand: every score is 0 but one key's, which is far above.  Its value
    row alone carries a 1 in the first column.  Just inside the window the output's first column is near
    1, just outside it is 0: for a prompt in one step, in two portions, and token by token; with pages of
    64 the edges fall inside pages and on their borders.  No norm, no rotation: the mask and the cache alone."""
    from rbitnet_b200.cache import SequenceCache
    from rbitnet_b200.kernels.ops import CudaOps
    from rbitnet_b200.parts.base import CacheNeed
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    ops = CudaOps(dt)
    Dc = ops.cache_head_width(D, Dv)
    n = 2 * window + 70
    for special in (n - window, n - window - 1, 63, 64):
        for cuts in ([0, n], [0, n - window + 3, n], [0, n - 20] + list(range(n - 19, n + 1))):
            cache = SequenceCache({0: CacheNeed(Kh, Dc, window)}, {}, {}, 64 * 8, 1024, dt, ops.device)
            cache.alloc()
            slot = cache.alloc()
            proj = torch.zeros(n, (H + Kh) * D + Kh * Dv)
            proj[:, 0:H * D:D] = 6.0                        # every query: 6 in its first value
            proj[special, H * D:(H + Kh) * D:D] = 6.0       # one key: 6 there too, the others 0
            proj[special, (H + Kh) * D::Dv] = 1.0           # and its value row is marked
            outs = []
            for a, b in zip(cuts[:-1], cuts[1:]):
                cache.reserve(slot, b - a)
                cache.upload_tables()
                meta = _meta(ops, [(slot, a, b - a)])
                view = cache.view(0)
                q = ops.norm_rotate_append(proj[a:b].to(dt).cuda().contiguous(), None, meta, view, H, D, Dv, None, None, 1e-6)
                att = ops.attention(q, meta, view, H, 1.0, window)
                outs.append(ops.head_gate(att, None, None, H, Dv, Dc).float().cpu())
                cache.advance(slot, b - a)
            got = torch.cat(outs).view(n, H, Dv)[:, :, 0]
            for i in range(special, n):
                seen = i - special < window
                share = math.exp(36.0) / (math.exp(36.0) + min(i + 1, window) - 1)
                want = share if seen else 0.0
                assert float((got[i] - want).abs().max()) <= 1e-2, (special, cuts[:3], i, got[i], want)
            ops.check_errors()


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
@pytest.fixture(scope="module")
def ops32():
    from rbitnet_b200.kernels.ops import CudaOps
    return CudaOps(torch.float32)


def _meta(ops, runs):
    """runs: (slot, start, n) per sequence."""
    from rbitnet_b200.engine.step import SeqChunk, build_meta
    chunks, at = [], 0
    for slot, start, n in runs:
        chunks.append(SeqChunk(slot, start, n, at))
        at += n
    return build_meta(chunks, np.zeros(at, dtype=np.int32), np.zeros(0, dtype=np.int32), ops.device)


@pytest.mark.parametrize("s,E,n_y", [(4, 96, 2), (1, 64, 1), (3, 1000, 2), (8, 40, 1), (5, 50, 2), (6, 64, 1), (16, 33, 3), (2, 4100, 1)])
def test_stream_step_fused_against_pieces_and_plain(ops32, s, E, n_y):
    g = torch.Generator().manual_seed(s * 100 + E)
    T = 7
    X = torch.randn(s, T, E, generator=g, dtype=torch.float64)
    ys = [torch.randn(T, E, generator=g, dtype=torch.float64) * 3 for _ in range(n_y)]
    ws = [torch.randn(E, generator=g, dtype=torch.float64) for _ in range(n_y)]
    mix, w_out, w_in = (torch.randn(s, s, generator=g, dtype=torch.float64), torch.randn(s, generator=g, dtype=torch.float64),
                        torch.randn(s, generator=g, dtype=torch.float64))
    nw, eps = torch.randn(E, generator=g, dtype=torch.float64), 1e-5
    y = sum(plain.rms(a, eps) * w for a, w in zip(ys, ws)) / n_y if n_y > 1 else ys[0]
    X2 = plain.hyper_write(X, mix, w_out, y)
    h_ref = plain.rms(plain.hyper_read(X2, w_in), eps) * nw
    dev = lambda t: t.float().cuda().contiguous()
    packed = lambda Z: dev(Z.permute(1, 0, 2).reshape(T, s * E))
    xa = packed(X)
    h = ops32.stream_step(xa, s, results=[dev(a) for a in ys], result_norms=[dev(w) for w in ws] if n_y > 1 else None,
                          norm_eps=eps, write=(dev(mix), dev(w_out)), read=(dev(w_in), dev(nw), eps))
    assert rel_err(xa.cpu(), packed(X2).cpu()) <= 1e-5 and rel_err(h.cpu(), h_ref) <= 1e-5
    xb = packed(X)
    yb = ops32.normed_mean([dev(a) for a in ys], [dev(w) for w in ws], eps) if n_y > 1 else dev(ys[0])
    ops32.stream_step(xb, s, results=[yb], write=(dev(mix), dev(w_out)))
    hb = ops32.stream_step(xb, s, read=(dev(w_in), dev(nw), eps))
    assert torch.equal(xa, xb) or rel_err(xb.cpu(), xa.cpu()) <= 1e-6
    assert rel_err(hb.cpu(), h.cpu()) <= 1e-6
    assert rel_err(ops32.streams_sum(xa, s).cpu(), X2.sum(0)) <= 1e-5
    assert torch.equal(ops32.streams_expand(dev(ys[0]), s), dev(ys[0]).repeat(1, s))


@pytest.mark.parametrize("H,D,Dv", [(2, 16, 24), (1, 40, 8), (3, 100, 33), (2, 128, 64), (1, 8, 130), (1, 200, 40), (2, 256, 24), (1, 300, 20)])
def test_matrix_memory_kernel(ops32, H, D, Dv):
    """Whole runs, portions and single tokens through the state, sizes that one to four lanes hold."""
    from rbitnet_b200.parts.recurrent import MatrixMemory
    g = torch.Generator().manual_seed(H * 1000 + D)
    E, T = 32, 45
    part = MatrixMemory(E, H, D, Dv, gate_cap=6.0, norm_eps=1e-5)
    w = {k: torch.randn(*shape, generator=g, dtype=torch.float64) * (0.3 if len(shape) > 1 else 1.0)
         for k, (shape, _) in part.weight_shapes().items()}
    w["f.b"] = w["f.b"] + 3.0
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops32)
    h = torch.randn(T, E, generator=g, dtype=torch.float64)
    p = {"heads": H, "dim": D, "vdim": Dv, "gate_cap": 6.0}
    want = plain.matrix_memory(w, p, h, 1e-5)

    class Ctx:
        ops = ops32
        def state_view(self, entry):
            return state
    for cuts in ([0, T], [0, 1, 2, 20, 36, 37, T], list(range(T + 1))):
        state = {k: torch.zeros((3, *n.shape), device="cuda") for k, n in part.state_need().items()}
        outs = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            ctx = Ctx()
            ctx.meta = _meta(ops32, [(1, a, b - a)])
            outs.append(part.forward(ctx, h[a:b].float().cuda(), 0))
        assert rel_err(torch.cat(outs).cpu(), want) <= 2e-4, cuts
        assert float(state["C"][0].abs().max()) == 0.0 and float(state["C"][2].abs().max()) == 0.0


@pytest.mark.parametrize("W,B,K", [(48, 3, 3), (32, 1, 2), (200, 5, 4), (24, 2, 1)])
def test_gated_recurrence_kernels(ops32, W, B, K):
    from rbitnet_b200.parts.recurrent import GatedLinearRecurrence
    g = torch.Generator().manual_seed(W + K)
    E, T = 40, 50
    part = GatedLinearRecurrence(E, W, B, K)
    w = {k: torch.randn(*shape, generator=g, dtype=torch.float64) * (0.3 if k in ("x", "y", "o", "ra", "ri") else 1.0)
         for k, (shape, _) in part.weight_shapes().items()}
    w["lam"] = w["lam"] - 3.0
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops32)
    h = torch.randn(T, E, generator=g, dtype=torch.float64)
    want = plain.gated_recurrence(w, {"width": W, "blocks": B}, h)

    class Ctx:
        ops = ops32
        def state_view(self, entry):
            return state
    # single rows take one fused kernel (convolution, gates, recurrence); with it switched off, the kernels of a prompt
    for cuts, fused in (([0, T], True), ([0, 1, 2, 3, 4, 30, T - 1, T], True), (list(range(T + 1)), True),
                        (list(range(T + 1)), False), ([0, 2, 3, 40, 41, T], False)):
        ops32.fuse_recurrent_step = fused
        state = {k: torch.zeros((2, *n.shape), device="cuda") for k, n in part.state_need().items()}
        outs = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            ctx = Ctx()
            ctx.meta = _meta(ops32, [(1, a, b - a)])
            outs.append(part.forward(ctx, h[a:b].float().cuda(), 0))
        ops32.fuse_recurrent_step = True
        assert rel_err(torch.cat(outs).cpu(), want) <= 2e-4, (cuts, fused)


@pytest.mark.parametrize("T,fused", [(19, True), (19, False), (300, True), (700, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_limited_gated_activation(dtype, T, fused):
    """In the tensor-core product's epilogue (bfloat16: tiles of 16 to 256 tokens) and as a kernel of its own."""
    from rbitnet_b200.kernels.ops import CudaOps
    from rbitnet_b200.parts.feed_forward import GatedDense
    ops = CudaOps(dtype)
    ops.fuse_gated_act = fused
    g = torch.Generator().manual_seed(5)
    E, F = 64, 88
    part = GatedDense(E, F, "swish_limited", limit=0.8)
    w = {k: (torch.randn(*shape, generator=g) * 0.4).to(torch.bfloat16).double() for k, (shape, _) in part.weight_shapes().items()}
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    h = torch.randn(T, E, generator=g).to(torch.bfloat16).double()
    want = plain.clamped_feed_forward(w, {"limit": 0.8}, h)

    class Ctx:
        pass
    ctx = Ctx()
    ctx.ops = ops
    got = part.forward(ctx, h.to(dtype).cuda())
    assert rel_err(got.cpu(), want) <= (1e-5 if dtype == torch.float32 else 2e-2)
    # the limit is in use: without it the result differs
    assert rel_err(plain.clamped_feed_forward(w, {"limit": 100.0}, h), want) > 0.05
