"""Lulenex in the engine against the plain implementation: each mechanism's kernels alone (with weights or inputs made so that a key just
inside or just outside a block of positions, a far key, a lost state row or a left-out sink shows), then whole models under every way
of cutting the work (in true 32-bit and in bfloat16), pages and slots that are used again, and greedy generation through the engine's
entry point and scheduler."""
from __future__ import annotations

import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_lulenex as P
import tiny_lulenex as tl
import traces

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOLERANCE = {"float32": 1e-4, "bfloat16": 6e-2}   # of the largest |logit| of the sequence
BF16_MEDIAN = 1.5e-2


@pytest.fixture(scope="module")
def rt16():
    from inference_bench_b200.engine.runtime import Runtime
    return Runtime(DEV, dtype="bfloat16")


@pytest.fixture(scope="module")
def ldirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("lulenex")
    return {name: tl.write_model(name, root / name) for name in tl.CONFIGS}


@pytest.fixture(scope="module")
def rt32():
    from inference_bench_b200.engine.runtime import Runtime
    return Runtime(DEV, dtype="float32")


def _f32(t):
    return t.to(DEV, torch.float32).contiguous()


def _ctx(rt, runs, slots=None):
    """A step's context for segments given as (first position, tokens)."""
    from inference_bench_b200.engine.context import Segment, build_context
    return build_context(rt, [Segment(i, (slots[i] if slots else i), p0, [0] * n, []) for i, (p0, n) in enumerate(runs)])


PLAN = [[("a", 1), ("b", 2)], [("a", 1), ("b", 1)], [("a", 2)], [("a", 7), ("b", 6)], [("c", 1), ("a", 3)], [("c", 2), ("a", 9)], [("c", 11)], [("c", 1)], [("c", 1)]]
LENS = {"a": 23, "b": 9, "c": 16}     # b ends after the fourth step; c takes its slot, zeroed


def _walk(rt, zero_slot, step_fn):
    """Runs PLAN: three requests in two slots (c uses b's again), portions of 1, 2 and more tokens beside one another."""
    slot, at = {"a": 0, "b": 1, "c": 1}, {r: 0 for r in LENS}
    for step in PLAN:
        if step[0][0] == "c" and at["c"] == 0:
            zero_slot(1)
        ctx = _ctx(rt, [(at[r], n) for r, n in step], [slot[r] for r, _ in step])
        step_fn(ctx, step, dict(at))
        for r, n in step:
            at[r] += n
    assert at == LENS


# ------------------------------------------------------------------------------------------ attention in blocks of positions with a sink, a gate and a scale
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,page,block,extra", [
    (4, 2, 64, 16, 48, 24), (8, 1, 128, 16, 100, 0), (2, 2, 128, 64, 64, 8), (6, 3, 64, 8, 130, 40), (4, 4, 64, 32, 1000, 0), (3, 1, 64, 16, 1, 5),
    (4, 2, 32, 16, 24, 4), (5, 5, 24, 8, 13, 0), (16, 1, 64, 64, 200, 16)])
def test_attention_in_blocks_of_positions_with_sink_gate_and_scale(rt32, rt16, dtype, heads, kv_heads, dim, page, block, extra):
    """Prompt portions that cross edges of blocks and of pages, the first tokens of a sequence and single decoded tokens right before, at
    and after an edge, all of one request on shuffled pages. One key stands out for one query (they share a large entry): the first key of
    the query's block (inside) and the last of the block before (outside), a query's own position, a key far back in a long block. The
    heads are the first columns of a wider output buffer, gated by one sigmoid a head and scaled; bfloat16 heads of 64 and 128 run on
    the tensor-core kernels, the rest on the generic one."""
    from inference_bench_b200.kernels import attention
    from inference_bench_b200.kernels.ops import KvLayerView
    rt = rt32 if dtype == torch.float32 else rt16
    n_ctx, scale, out_scale = 420, 0.35, 0.7
    g = torch.Generator().manual_seed(heads * dim + page + block)
    e1 = (300 // block) * block                      # a block's first position at or below 300
    runs = [(130, 150), (0, 7), (max(e1 - 1, 0), 1), (e1, 1), (min(e1 + 1, n_ctx - 1), 1), (410, 1), (2 * page - 2, 4), (330, 70)]
    positions = [p0 + i for p0, n in runs for i in range(n)]
    T = len(positions)
    n_pages = -(-n_ctx // page)
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    k, v = torch.randn((n_ctx, kv_heads, dim), generator=g), torch.randn((n_ctx, kv_heads, dim), generator=g)
    q = torch.randn((n_ctx, heads, dim), generator=g) * 0.3
    lo = lambda p: p - p % block
    needles = [(e1, e1, 0), (e1 + 3, lo(e1 + 3), 1 % heads), (e1 + 2, lo(e1 + 2) - 1, 2 % heads), (270, lo(270), 0), (271, lo(271) - 1, 1 % heads),
               (410, lo(410), 0), (409, 5, 1 % heads), (2 * page, 2 * page - 1, 0), (399, 331, 0)]
    for i, (qp, key, head) in enumerate(needles):
        if not 0 <= key < n_ctx or not 0 <= qp < n_ctx:
            continue
        col = (i * 5) % dim
        k[key, head // (heads // kv_heads), col] = 5.0
        q[qp, head, col] = 30.0
    k, v, q = k.to(dtype).float(), v.to(dtype).float(), q.to(dtype).float()
    sink = torch.randn((heads,), generator=g) * 2.0
    gate_parts = torch.randn((2, T, heads + 3), generator=g)
    pool = torch.zeros((2, n_pages + 3, 2, kv_heads, page, dim), dtype=dtype, device=DEV)
    for j in range(n_ctx):
        pool[1, perm[j // page], 0, :, j % page] = k[j].to(dtype)
        pool[1, perm[j // page], 1, :, j % page] = v[j].to(dtype)
    want = P.sink_softmax_in_blocks(q.double(), k.double(), v.double(), torch.arange(n_ctx), scale, block, sink.double())[positions]
    want = want * torch.sigmoid(gate_parts.double().sum(0)[:, 3:])[:, :, None] * out_scale
    ctx = _ctx(rt, runs)
    table = perm.to(torch.int32).reshape(1, -1).repeat(len(runs), 1).contiguous().to(DEV)
    view = KvLayerView(pool, 1, table)
    qd = q[positions].reshape(T, heads * dim).to(DEV, dtype).contiguous()
    out = torch.full((T, heads * dim + extra), 7.0, dtype=dtype, device=DEV)
    attention.paged_attention(ctx, qd, view, heads, None, scale, sink=True, chunk=block, sink_values=_f32(sink), gate=(_f32(gate_parts), 3), out_scale=out_scale, out=out)
    got = out[:, :heads * dim].float().cpu().double().view(T, heads, dim)
    assert (out[:, heads * dim:] == 7.0).all()                     # the columns beyond the heads belong to someone else
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    err = (got - want).abs().amax(dim=(1, 2))
    assert err.max().item() < tol, f"positions {[positions[i] for i in torch.nonzero(err >= tol).flatten().tolist()]} differ by up to {err.max().item():.2e}"
    rt.check_status()



# ------------------------------------------------------------------------------------------ norm with one number, token shift and its state
@pytest.mark.parametrize("H", [48, 80, 132, 1022, 4096])
def test_norm_and_token_shift_over_portions(rt32, H):
    """Every row equals the plain norm and shift of the whole sequence, however the rows are cut; steps of single tokens also run the
    one-kernel form, which gives the same rows and the same state. The contribution added before the norm has a bias."""
    from inference_bench_b200.kernels import ops
    g = torch.Generator().manual_seed(H)
    x = {r: torch.randn((n, H), generator=g) * 3 + 1 for r, n in LENS.items()}
    delta = {r: torch.randn((2, n, H), generator=g) for r, n in LENS.items()}
    gain, mix, bias, eps = torch.tensor(1.3), torch.rand((H,), generator=g), torch.randn((H,), generator=g), 1e-5
    want = {r: P.token_shift(P.scalar_norm(x[r].double() + delta[r].double().sum(0) + bias.double(), gain, eps), mix) for r in LENS}
    w = _f32(gain.reshape(1).expand(H))
    state = torch.zeros((3, H), device=DEV)

    def step_fn(ctx, step, at):
        xs = torch.cat([x[r][at[r]:at[r] + n] for r, n in step]).to(DEV).contiguous()
        ds = torch.cat([delta[r][:, at[r]:at[r] + n] for r, n in step], dim=1).to(DEV).contiguous()
        ops.add_bias_rows(ds[0], _f32(bias))
        T = xs.shape[0]
        single = None
        if all(n == 1 for _, n in step):
            x1, st1, single = xs.clone(), state.clone(), torch.empty((T, H), device=DEV)
            ds1 = ds.clone()
            ops.add_rmsnorm_ext(x1, ds1, w, eps, single, shift=(_f32(mix), st1, ctx.seg_slot))
        normed = torch.empty((T, H), device=DEV)
        ops.add_rmsnorm(xs, ds, w, normed, eps)
        for dt, tol in ((torch.bfloat16, 3e-2), (torch.float32, 3e-5)):
            saved = state.clone()
            out = torch.empty((T, H), dtype=dt, device=DEV)
            ops.token_shift_rows(normed, _f32(mix), state, ctx.seg_of_token, ctx.seg_start, ctx.seg_slot, out)
            if dt != torch.float32:
                state.copy_(saved)
            o = 0
            for r, n in step:
                err = (out[o:o + n].cpu().double() - want[r][at[r]:at[r] + n]).abs().max().item()
                assert err < tol * max(1.0, want[r].abs().max().item()), f"request {r} rows {at[r]}..{at[r] + n}: {err}"
                o += n
        if single is not None:
            assert torch.allclose(single, out, atol=1e-5) and torch.allclose(st1, state, atol=1e-5) and torch.allclose(x1, xs, atol=1e-6)

    _walk(rt32, lambda s: state[s].zero_(), step_fn)
    rt32.check_status()


def test_norm_with_a_bias_xielu_gated_norm_and_loop_entry(rt32):
    from inference_bench_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    T, H, I = 19, 72, 50
    x, delta, bias, w = torch.randn((T, H), generator=g), torch.randn((3, T, H), generator=g), torch.randn((H,), generator=g), torch.rand((H,), generator=g) + 0.5
    xd, out = _f32(x), torch.empty((T, H), device=DEV)
    ops.add_rmsnorm_ext(xd, _f32(delta), _f32(w), 1e-6, out, bias=_f32(bias))
    v = x.double() + delta.double().sum(0) + bias.double()
    assert torch.allclose(xd.cpu().double(), v, atol=1e-5)
    assert torch.allclose(out.cpu().double(), P.rms_unit(v, 1e-6) * w.double(), atol=2e-5)
    # xIELU on both sides of zero, with large arguments and both signs of p and q
    for pq in ([0.3, -0.2], [-2.0, 3.0], [5.0, -5.0]):
        z = torch.randn((2, T, I), generator=g) * 3
        z[0, 0, :5] = torch.tensor([0.0, -1e-6, 1e-6, 30.0, -30.0])
        z[1, 0, :5] = 0.0
        act = torch.empty((T, I), device=DEV)
        ops.xielu_rows(_f32(z), _f32(torch.tensor(pq)), act)
        want = P.xielu(z.double().sum(0), torch.tensor(pq, dtype=torch.float64))
        assert torch.allclose(act.cpu().double(), want, rtol=2e-5, atol=2e-5)
    # the norm over all heads with a sigmoid gate, written into columns of a wider buffer
    o, gate = torch.randn((T, H), generator=g) * 5, torch.randn((2, T, H + 9), generator=g)
    buf = torch.full((T, H + 24), 7.0, device=DEV)
    ops.gated_rmsnorm(_f32(o), _f32(w), 1e-5, _f32(gate), 4, 0.7, buf, 16)
    want = 0.7 * P.rms_unit(o.double(), 1e-5) * w.double() * torch.sigmoid(gate.double().sum(0)[:, 4:4 + H])
    assert torch.allclose(buf[:, 16:16 + H].cpu().double(), want, atol=2e-5)
    assert float((buf[:, :16] - 7).abs().max()) == 0 and float((buf[:, 16 + H:] - 7).abs().max()) == 0
    # the entry of a pass: [x + pending | x0] packed, x reset to the pass's vector
    x0, step = torch.randn((T, H), generator=g), torch.randn((H,), generator=g)
    xd, packed = _f32(x), torch.empty((T, 2 * H), device=DEV)
    ops.loop_pack(xd, _f32(delta), _f32(x0), _f32(step), packed)
    assert torch.allclose(packed.cpu().double(), torch.cat([x.double() + delta.double().sum(0), x0.double()], 1), atol=1e-5)
    assert torch.equal(xd.cpu(), step.expand(T, H))
    rt32.check_status()


# ------------------------------------------------------------------------------------------ the selective scan with its convolution
@pytest.mark.parametrize("T,N,K", [(1, 4096, 64), (8, 4224, 1024), (5, 200, 72), (17, 136, 264), (64, 5000, 520), (100, 4096, 136), (128, 130, 64),
                                   (8, 256, 2048), (129, 520, 264), (300, 1000, 1024), (700, 8192, 256), (2048, 384, 512), (2300, 1100, 72)])
def test_product_with_xielu_in_its_epilogue(rt16, T, N, K):
    """The up projection with the activation applied to the float32 accumulators in the tensor-core kernels (one CTA a tile for few
    tokens, CTA pairs for many; sizes that end inside a tile), against float64, and against the product followed by the row-wise
    kernel; both signs of the activation's two numbers."""
    from inference_bench_b200.kernels import gemm_tcgen05 as G
    from inference_bench_b200.kernels import lib as L
    from inference_bench_b200.kernels import ops
    g = torch.Generator().manual_seed(T + N + K)
    x = (torch.randn(T, K, generator=g) * 0.7).to(torch.bfloat16).to(DEV)
    lw = rt16.matrix((torch.randn(N, K, generator=g) * (2.0 / math.sqrt(K))).to(torch.bfloat16))
    for pq in ((0.8, -0.4), (-1.5, 2.0)):
        pq_dev = _f32(torch.tensor(pq))
        called = []
        real = L.call
        L.call = lambda name, *a: (called.append(name), real(name, *a))[1]
        try:
            act = rt16.up_xielu(x, lw, pq_dev)
        finally:
            L.call = real
        if G.xielu_in_epilogue(T, N, K, rt16.sm_count):
            assert called in (["ib_gemm_xielu_tcgen05"], ["ib_gemm_xielu_tcgen05_2cta"])
            assert called == ["ib_gemm_xielu_tcgen05"] if T <= 128 else T < 2048 or called == ["ib_gemm_xielu_tcgen05_2cta"]
        else:
            assert (T, N, K) == (8, 256, 2048) and called[-1] == "ib_xielu_rows"
        want = P.xielu(x.cpu().double() @ lw.weight.cpu().double().T, torch.tensor(pq, dtype=torch.float64))
        assert ((act.cpu().double() - want).abs() <= 2.0 ** -8 * want.abs() + 2e-5 * want.abs().max()).all()
        z = rt16.linear(x, lw)
        rows = torch.empty((T, N), dtype=torch.bfloat16, device=DEV)
        ops.xielu_rows(z, pq_dev, rows)
        assert ((act.float() - rows.float()).abs() <= 2.0 ** -7 * rows.float().abs() + 1e-6).all()
    rt16.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inner,N,R,taps", [(96, 5, 3, 4), (60, 17, 1, 1), (128, 40, 4, 3), (72, 16, 8, 2), (40, 150, 2, 5), (36, 1, 2, 2)])
def test_selective_scan_over_portions_and_slots(dtype, inner, N, R, taps):
    """The mixer as a part, its state slots by hand: portions of 1, 2 and more tokens (fewer than taps - 1 among them) of three requests
    in two slots equal the plain scan of each whole sequence."""
    from inference_bench_b200.cache.manager import StateView
    from inference_bench_b200.engine.runtime import Runtime
    from inference_bench_b200.parts.scan import SelectiveScan
    rt = Runtime(DEV, dtype=dtype)
    W = 64
    cfg = {"width": W, "vocab": 8, "layers": [{"type": "mamba1", "mixer": {"inner": inner, "state": N, "dt_rank": R, "conv": taps}, "mlp": None}]}
    w = {n[len("l0."):]: t for n, t in tl.tensors(cfg, inner + N).items() if n.startswith("l0.mix")}
    part = SelectiveScan("mix", W, inner, N, R, taps)
    part.bind({n: t.to(DEV) for n, t in w.items()}, rt)
    g = torch.Generator().manual_seed(N)
    h = {r: torch.randn((n, W), generator=g).to(torch.bfloat16) for r, n in LENS.items()}
    want = {r: P.selective_scan_mixer(h[r].double(), w, "mix", cfg["layers"][0]["mixer"]) for r in LENS}
    state, conv = torch.zeros((3, inner, N), device=DEV), torch.zeros((3, max(taps - 1, 1), inner), device=DEV)
    tol = 3e-5 if dtype == "float32" else 4e-2

    def step_fn(ctx, step, at):
        hs = torch.cat([h[r][at[r]:at[r] + n] for r, n in step]).to(DEV, rt.act_dtype).contiguous()
        out = part.forward(ctx, hs, (StateView(state), StateView(conv))).sum(0).cpu().double()
        o = 0
        for r, n in step:
            err = (out[o:o + n] - want[r][at[r]:at[r] + n]).abs().max().item() / want[r].abs().max().item()
            assert err < tol, f"request {r} rows {at[r]}..{at[r] + n}: {err}"
            o += n

    def zero(s):
        state[s].zero_(), conv[s].zero_()

    _walk(rt, zero, step_fn)
    rt.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inner,N,R,taps", [(96, 5, 3, 4), (128, 40, 4, 3), (40, 150, 2, 1), (200, 16, 8, 5)])
def test_selective_scan_long_portions_in_chunks(dtype, inner, N, R, taps):
    """Portions longer than a chunk of the scan (walked chunk by chunk, side by side) beside short ones and single tokens, starting from a
    zero state and from a state that earlier portions left, with lengths just below, at and above a multiple of the chunk; the slot of a
    finished request is used again. Every row equals the plain scan of the whole sequence."""
    from inference_bench_b200.cache.manager import StateView
    from inference_bench_b200.engine.runtime import Runtime
    from inference_bench_b200.kernels.ops import RECURRENCE_CHUNK as C
    from inference_bench_b200.parts.scan import SelectiveScan
    rt = Runtime(DEV, dtype=dtype)
    W = 48
    mixer = {"inner": inner, "state": N, "dt_rank": R, "conv": taps}
    cfg = {"width": W, "vocab": 8, "layers": [{"type": "mamba1", "mixer": mixer, "mlp": None}]}
    w = {n[len("l0."):]: t for n, t in tl.tensors(cfg, 3 * inner + N).items() if n.startswith("l0.mix")}
    part = SelectiveScan("mix", W, inner, N, R, taps)
    part.bind({n: t.to(DEV) for n, t in w.items()}, rt)
    plan = [[("a", 2 * C + 2), ("b", 3)], [("a", 1), ("b", C + 1)], [("a", 3 * C), ("b", 1)], [("c", C), ("a", 1)], [("c", 4 * C - 1), ("a", C + 7)], [("c", 1)]]
    lens = {}
    for step in plan:
        for r, n in step:
            lens[r] = lens.get(r, 0) + n
    g = torch.Generator().manual_seed(N + taps)
    h = {r: torch.randn((n, W), generator=g).to(torch.bfloat16) for r, n in lens.items()}
    want = {r: P.selective_scan_mixer(h[r].double(), w, "mix", mixer) for r in lens}
    state, conv = torch.zeros((2, inner, N), device=DEV), torch.zeros((2, max(taps - 1, 1), inner), device=DEV)
    slot, at = {"a": 0, "b": 1, "c": 1}, {r: 0 for r in lens}
    tol = 3e-5 if dtype == "float32" else 4e-2
    for step in plan:
        if step[0][0] == "c" and at["c"] == 0:
            state[1].zero_(), conv[1].zero_()
        ctx = _ctx(rt, [(at[r], n) for r, n in step], [slot[r] for r, _ in step])
        hs = torch.cat([h[r][at[r]:at[r] + n] for r, n in step]).to(DEV, rt.act_dtype).contiguous()
        out = part.forward(ctx, hs, (StateView(state), StateView(conv))).sum(0).cpu().double()
        o = 0
        for r, n in step:
            err = (out[o:o + n] - want[r][at[r]:at[r] + n]).abs().amax(dim=1) / want[r].abs().max().item()
            assert err.max().item() < tol, f"request {r} rows {at[r]}..{at[r] + n}: row {at[r] + int(err.argmax())} differs by {err.max().item():.2e}"
            o += n
            at[r] += n
    rt.check_status()


# ------------------------------------------------------------------------------------------ whole models
def _requests(name):
    vocab = tl.CONFIGS[name]["config"]["vocab"]
    return {r: traces.prompt(300 + i, n, vocab) for i, (r, n) in enumerate({"a": 150, "b": 1, "c": 23, "d": 64, "e": 97, "f": 2}.items())}


@pytest.fixture(scope="module")
def plain_logits(ldirs):
    return {name: {r: P.PlainLulenex(ldirs[name]).logits(t).numpy() for r, t in _requests(name).items()} for name in tl.CONFIGS}


def _runner(model_dir, dtype, max_tokens, page_size, **kw):
    from inference_bench_b200.trace import build_runner
    return build_runner(model_dir, dtype, max_tokens, page_size=page_size, **kw)


def _compare(got, want_by_req, dtype, what):
    errs = []
    for (r, pos), row in got.items():
        want = want_by_req[r][pos]
        err = np.abs(row - want).max() / np.abs(want_by_req[r]).max()
        assert err <= TOLERANCE[dtype], f"{what}: request {r} position {pos}: |diff| = {err:.3e} of max|logit| (allowed {TOLERANCE[dtype]:.0e})"
        errs.append(err)
    assert len(got) == sum(len(v) for v in want_by_req.values())
    if dtype == "bfloat16":
        assert float(np.median(errs)) < BF16_MEDIAN, f"{what}: the median row differs by {np.median(errs):.2e} of max|logit|"
    return max(errs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tl.CONFIGS))
def test_layers_one_by_one(ldirs, name, dtype):
    """The residual stream after every layer run (a looped layer counts each time) against the plain model's, so that a wrong layer is named."""
    from inference_bench_b200.engine.step import StepEntry
    toks = _requests(name)["e"]
    want = P.PlainLulenex(ldirs[name]).hidden_states(toks)
    runner = _runner(ldirs[name], dtype, 128, tl.CONFIGS[name]["page_size"])
    runner.cache.admit("x")
    layers = []
    runner.step([StepEntry("x", toks, list(range(len(toks))))], trace=layers)
    assert len(layers) == len(want) + 1
    for i, (g, w) in enumerate(zip(layers[1:], want)):
        err = (g.cpu().double() - w).abs().amax(dim=1) / w.abs().max().item()
        assert err.max().item() < (2e-5 if dtype == "float32" else 4e-2), f"{name}/{dtype}: the stream after layer run {i} differs by {err.max().item():.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tl.CONFIGS))
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_cut_matches_plain(ldirs, plain_logits, name, dtype, cut):
    """Whole prompts; prompts then the last tokens one by one (a tail long enough for every block of positions to pass over decoded tokens
    only); portions down to two tokens; up to four live requests of unequal length in one batch with a pool that only holds what is
    live, so pages and slots are used again by later requests."""
    reqs = _requests(name)
    steps = {"whole": traces.whole, "tail": lambda r: traces.tail_one_by_one(r, tail=60), "portions": traces.portions, "mixed": traces.mixed}[cut](reqs)
    max_tokens = traces.max_live_tokens(steps)
    runner = _runner(ldirs[name], dtype, max_tokens, tl.CONFIGS[name]["page_size"], max_requests=4)
    got = traces.run_steps(runner, steps)
    worst = _compare(got, plain_logits[name], dtype, f"{name}/{dtype}/{cut}")
    runner.cache.check()
    assert runner.cache.used_pages() == [0] * len(runner.cache.groups)
    print(f"{name}/{dtype}/{cut}: worst {worst:.3e} of max|logit|, pool {max_tokens} tokens")


def test_a_request_alone_and_in_a_batch_give_the_same_float32_logits(ldirs):
    """The float32 path adds in one order whatever shares the step: a request beside three others of other lengths, on other pages and
    in another slot, gives the bits it gives alone."""
    from inference_bench_b200.engine.step import StepEntry
    name = "A"
    reqs = _requests(name)
    runner = _runner(ldirs[name], "float32", 1024, 16, max_requests=4)
    runner.cache.admit("alone")
    alone = runner.step([StepEntry("alone", reqs["d"], [len(reqs["d"]) - 1])]).cpu()
    runner.cache.release("alone")
    for r in ("c", "f", "d", "a"):
        runner.cache.admit(r)
    rows = runner.step([StepEntry(r, reqs[r], [len(reqs[r]) - 1]) for r in ("c", "f", "d", "a")]).cpu()
    assert torch.equal(rows[2], alone[0])


# ------------------------------------------------------------------------------------------ weights made so that a fault shows
def _one_layer(tmp_path, chunk, decay, gain, sink, tag):
    """One parallel layer without a feed-forward; queries and keys scaled so that the softmax nearly picks one key."""
    cfg = {"architecture": "Lulenex", "vocab": 64, "width": 40, "norm": {"eps": 1e-6}, "loop": None,
           "layers": [{"type": "parallel", "mlp": None, "mixer": {
               "left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "mask": {"size": chunk}, "rot": {"base": 100.0, "dims": 8}, "scale": gain},
               "left_scale": 1.0, "right": {"heads": 2, "dim": 8, "vdim": 8, "decay": list(decay)}, "right_scale": 1.0}}]}
    w = tl.tensors(cfg, 77)
    w["l0.mix.left.sink"] = torch.full((2,), float(sink)).to(torch.bfloat16)
    w["l0.shift"] = torch.zeros(40).to(torch.bfloat16)
    out = tmp_path / tag
    out.mkdir()
    (out / "config.json").write_text(json.dumps(cfg))
    from inference_bench_b200.weights.safetensors_io import write_safetensors
    write_safetensors(out / "model.safetensors", w, {"format": "pt"})
    return out, cfg


@pytest.mark.parametrize("chunk,page", [(16, 16), (7, 16), (33, 8)])
def test_keys_just_inside_and_just_outside_a_block_of_positions(tmp_path, chunk, page):
    """With a softmax that nearly picks one key, a block that starts one position early or late changes the rows near every block's
    start by far more than the tolerance; the engine equals the right blocks, for whole prompts and for tokens decoded one by one."""
    from inference_bench_b200.engine.step import StepEntry
    model, cfg = _one_layer(tmp_path, chunk, (0.9, 0.5), 30.0, -1.0, "m")
    plain = P.PlainLulenex(model)
    toks = traces.prompt(11, 3 * chunk + 5, 64)
    want = plain.logits(toks)
    edge = [t for t in range(len(toks)) if t % chunk in (0, 1, chunk - 1)]
    for wrong in (chunk - 1, chunk + 1):
        bad = copy.deepcopy(plain.cfg)
        bad["layers"][0]["mixer"]["left"]["mask"]["size"] = wrong
        diff = (P.logits(bad, plain.w, toks) - want)[edge].abs().amax(dim=1) / want.abs().max()
        assert diff.max().item() > 0.05, f"blocks of {wrong} instead of {chunk} would not show ({diff.max().item():.2e})"
    for head in (len(toks), chunk + 2, 1):
        runner = _runner(model, "float32", 256, page)
        runner.cache.admit("x")
        rows = [runner.step([StepEntry("x", toks[:head], list(range(head)))]).cpu()]
        rows += [runner.step([StepEntry("x", [t], [0])]).cpu() for t in toks[head:]]
        err = (torch.cat(rows).double() - want).abs().amax(dim=1) / want.abs().max()
        assert err.max().item() < 1e-4, f"prompt of {head} then one by one: {err.max().item():.2e} at position {int(err.argmax())}"


def test_a_left_out_sink_and_a_far_key_show(tmp_path):
    """A sink as large as the largest score a key can reach takes a good part of every softmax: without it the logits differ visibly. A head whose decay is 1
    keeps the first token for ever: 400 tokens on (through the chunked form and through single tokens) it still counts."""
    from inference_bench_b200.engine.step import StepEntry
    model, cfg = _one_layer(tmp_path, 1000, (1.0, 0.97), 4.0, 64.0, "s")
    plain = P.PlainLulenex(model)
    toks = traces.prompt(12, 400, 64)
    want = plain.logits(toks)
    no_sink = dict(plain.w)
    no_sink["l0.mix.left.sink"] = torch.full((2,), -60.0, dtype=torch.float64)
    assert ((P.logits(plain.cfg, no_sink, toks) - want).abs().amax(dim=1) / want.abs().max()).min().item() > 1e-3
    other = list(toks)
    other[0] = (toks[0] + 1) % 64
    assert ((plain.logits(other) - want)[-8:].abs().amax(dim=1) / want.abs().max()).min().item() > 5e-4    # the first token still counts at the end
    for head in (400, 330):
        runner = _runner(model, "float32", 512, 16)
        runner.cache.admit("x")
        rows = [runner.step([StepEntry("x", toks[:head], list(range(head)))]).cpu()]
        rows += [runner.step([StepEntry("x", [t], [0])]).cpu() for t in toks[head:]]
        err = (torch.cat(rows).double() - want).abs().amax(dim=1) / want.abs().max()
        assert err.max().item() < 1e-4, f"{head}: {err.max().item():.2e} at {int(err.argmax())}"


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("name", list(tl.CONFIGS))
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(ldirs, name, graphs):
    """`Engine.generate`: the scheduler cuts prompts into portions, batches them beside decoded tokens, and decode steps run as captured
    graphs or not; float32 tokens equal the plain model's."""
    from inference_bench_b200 import Engine
    vocab = tl.CONFIGS[name]["config"]["vocab"]
    plain = P.PlainLulenex(ldirs[name])
    prompts = [traces.prompt(70 + i, n, vocab) for i, n in enumerate((5, 21, 40))]
    want = [plain.greedy(p, 7) for p in prompts]
    eng = Engine(ldirs[name], dtype="float32", max_ctx=128, page_size=tl.CONFIGS[name]["page_size"], use_graphs=graphs, prefill_chunk=9, max_batched_tokens=16)
    got = eng.generate(prompts, max_tokens=7)
    assert [r.tokens for r in got] == want
    assert eng.cache.used_pages() == [0] * len(eng.cache.groups)
    eng.cache.check()
    one = eng.generate(prompts[1], max_tokens=7)
    assert one.tokens == want[1]


def test_generation_in_bfloat16_runs_and_long_decoding_stays_close(ldirs):
    from inference_bench_b200 import Engine
    name = "C"
    vocab = tl.CONFIGS[name]["config"]["vocab"]
    plain = P.PlainLulenex(ldirs[name])
    prompt = traces.prompt(5, 12, vocab)
    eng = Engine(ldirs[name], dtype="bfloat16", max_ctx=256, page_size=16)
    got = eng.generate(prompt, max_tokens=120).tokens
    assert len(got) == 120
    lg = plain.logits(prompt + got)     # teacher-forced on the engine's own tokens, the plain model ranks every chosen token near the top
    span = float(lg.max() - lg.min())
    below = [float(lg[len(prompt) + i - 1].max() - lg[len(prompt) + i - 1][tok]) / span for i, tok in enumerate(got)]
    assert all(math.isfinite(b) for b in below) and max(below) < 0.2
    assert sum(b > 0.03 for b in below) <= 0.1 * len(got)


def test_trace_replay_program_and_command_line(ldirs, tmp_path):
    """bin/trace_run as a subprocess fed JSON steps (a mixed trace, float32), and `run` and `spec` of the command line, on a model folder
    of this architecture: nothing in them names an architecture."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "A"
    vocab = tl.CONFIGS[name]["config"]["vocab"]
    reqs = {r: traces.prompt(900 + i, n, vocab) for i, (r, n) in enumerate({"a": 70, "b": 9, "c": 33, "d": 64, "e": 2}.items())}
    steps = traces.mixed(reqs, seed=5)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(ldirs[name]), "--dtype", "float32", "--out", str(out),
                           "--max-tokens", str(traces.max_live_tokens(steps))],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    plain = P.PlainLulenex(ldirs[name])
    want = {r: plain.logits(t).numpy() for r, t in reqs.items()}
    at = {r: 0 for r in reqs}
    for s in steps:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
        k = 0
        for e in s["entries"]:
            for w in e["want"]:
                err = np.abs(rows[k] - want[e["id"]][at[e["id"]] + w]).max() / np.abs(want[e["id"]]).max()
                assert err <= TOLERANCE["float32"]
                k += 1
            at[e["id"]] += len(e["tokens"])
        assert k == rows.shape[0]
    env = dict(os.environ, PYTHONPATH=root)
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "run", "--model", str(ldirs[name]), "--prompt-len", "12", "--max-tokens", "5", "--json",
                        "--dtype", "float32", "--max-ctx", "64"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    r = json.loads(p.stdout)
    from inference_bench_b200.cli import _synthetic_prompt
    assert r["prompt_tokens"] == 12 and r["tokens"] == plain.greedy(_synthetic_prompt(12, vocab), 5)
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "spec", "--model", str(ldirs[name])], capture_output=True, text=True, env=env)
    assert p.returncode == 0 and json.loads(p.stdout)["layers"][1]["mixer"]["left"]["mask"]["size"] == 7
