"""Samulorn on a GPU against the plain implementation: each added kernel alone, then the engine --
the residual stream run by run, whole prompts, the tail one token at a time, prompts in portions
down to two tokens, batches of unequal requests whose shorter ones end earlier (slots, pages and
states used again), a far key among hundreds and across page borders in prompts and in decoding,
the first tokens, long decoding through the captured decode step, greedy generation through the
entry point, and the trace replay program."""
import json
import os

import pytest
import torch
import torch.nn.functional as F

from plain_samulorn import (delta_rule, dyt, gelu_tanh, over_rms, rotary_frequencies, rotate_neighbours, route,
                            short_conv)
from samulorn_helpers import (CONFIGS, NEEDLE, TOL, TOL_OF, add_portions, needle_model, needle_tokens, plain_generate_greedy,
                              plain_logits, random_tokens, safe_tokens, weights_of)
from trace_tools import (Trace, add_batches, add_tail, add_whole, compare, forced_decode, run_in_process,
                         run_trace_run)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16", "float16"]


@pytest.fixture(scope="module")
def ops():
    from yalm_b200.csrc import ops as o
    o.lib()
    return o


class B:
    """The index arrays of a ragged batch."""

    def __init__(self, q_lens, slots):
        qs = [0]
        for q in q_lens:
            qs.append(qs[-1] + q)
        self.n_seqs, self.n_tokens, self.q_lens, self.slots = len(q_lens), qs[-1], q_lens, slots
        self.is_decode = all(q == 1 for q in q_lens)
        self.q_start = torch.tensor(qs, dtype=torch.int32, device=DEV)
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
        self.token_seq = torch.tensor(sum([[i] * q for i, q in enumerate(q_lens)], []),
                                      dtype=torch.int32, device=DEV)


def _lm(cfg, w, dtype, **kw):
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    return LM(config_from_dict(cfg), dict(w), dtype=dtype, **kw)


def close(got, ref, tol):
    return (got.double().cpu() - ref.double()).abs().max().item() <= tol * max(1e-6, ref.abs().max().item())


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dim, rows", [(64, 5), (100, 3), (1000, 70), (4100, 2), (30, 4)])
def test_norm_step_forms(ops, dim, rows):
    g = torch.Generator().manual_seed(dim)
    x = torch.randn(rows, dim, generator=g, dtype=torch.float64)
    a, b = torch.randn(3, rows, dim, generator=g, dtype=torch.float64), torch.randn(2, rows, dim, generator=g, dtype=torch.float64)
    w1, b1, w2, b2 = (torch.randn(dim, generator=g, dtype=torch.float64) for _ in range(4))
    dev = lambda t: t.float().to(DEV)
    y = 0.8 * a.sum(0) - 1.3 * b.sum(0)
    forms = {"tanh": ((ops.NORM_TANH, dev(w1), dev(b1), 0.7, 0.0), lambda v: dyt(v, 0.7, w1, b1)),
             "rms": ((ops.NORM_RMS, dev(w2), None, 0.0, 1e-5), lambda v: over_rms(v, 1e-5) * w2),
             "none": ((ops.NORM_NONE, None, None, 0.0, 0.0), lambda v: v)}
    for post in forms:
        for pre in forms:
            for dt in (torch.float32, torch.bfloat16):
                xd, h = dev(x), torch.empty(rows, dim, dtype=dt, device=DEV)
                ops.norm_step(xd, [(dev(a), 3, 0.8), (dev(b), 2, -1.3)], post=forms[post][0], pre=forms[pre][0], h=h)
                new = x + forms[post][1](y)
                assert close(xd, new, 2e-6), (post, pre)
                assert close(h, forms[pre][1](new), 2e-5 if dt == torch.float32 else 1e-2), (post, pre)
    # a write alone, a read alone, and a read of some rows
    xd = dev(x)
    ops.norm_step(xd, [(dev(a), 3, 1.0)], post=forms["tanh"][0])
    assert close(xd, x + dyt(a.sum(0), 0.7, w1, b1), 2e-6)
    want = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    h = torch.empty(2, dim, device=DEV)
    ops.norm_step(dev(x), pre=forms["rms"][0], h=h, rows=want, n_rows=2)
    assert close(h, (over_rms(x, 1e-5) * w2)[[rows - 1, 0]], 2e-5)


@pytest.mark.parametrize("taps, channels", [(2, 8), (4, 100), (3, 600), (8, 33)])
def test_short_conv_ragged_steps_and_state(ops, taps, channels):
    g = torch.Generator().manual_seed(taps * 100 + channels)
    w = torch.randn(channels, taps, generator=g, dtype=torch.float64)
    bias_in, bias_out = torch.randn(channels, generator=g, dtype=torch.float64), torch.randn(channels, generator=g, dtype=torch.float64)
    n_slots, col0, row = 5, 3, channels + 7
    state = torch.zeros(n_slots, taps - 1, channels, device=DEV)
    plain_state = {s: torch.zeros(taps - 1, channels, dtype=torch.float64) for s in range(n_slots)}
    # steps of unequal sequences: longer than, as long as and shorter than the state; then one token each
    steps = [([9, 1, taps - 1, 2], [4, 0, 2, 1]), ([1, 1, 1, 1], [4, 0, 2, 1]), ([2, 5], [0, 1]), ([1], [2]),
             ([1, taps + 3], [1, 2])]
    for q_lens, slots in steps:
        b = B(q_lens, slots)
        src = torch.randn(2, b.n_tokens, row, generator=g, dtype=torch.float64)
        out32 = torch.zeros(b.n_tokens, channels + 2, device=DEV)
        blocks = 1 if channels % 4 else 4
        out16 = torch.zeros(blocks, b.n_tokens, channels // blocks, dtype=torch.bfloat16, device=DEV)
        ops.short_conv(src.float().to(DEV), 2, col0, channels, w.float().to(DEV), state, b, out32=out32, out_col0=2,
                       out16=out16, block16=channels // blocks, in_bias=bias_in.float().to(DEV),
                       out_bias=bias_out.float().to(DEV), silu=True)
        at = 0
        for ql, s in zip(q_lens, slots):
            u = src.sum(0)[at:at + ql, col0:col0 + channels] + bias_in
            y, plain_state[s] = short_conv(u, w, plain_state[s])
            y = F.silu(y + bias_out)
            assert close(out32[at:at + ql, 2:], y, 1e-5), (q_lens, s)
            got16 = out16[:, at:at + ql].permute(1, 0, 2).reshape(ql, channels)
            assert close(got16, y, 1e-2)
            assert close(state[s], plain_state[s], 1e-6), (q_lens, s)
            at += ql


@pytest.mark.parametrize("H, G, dk, dv", [(4, 2, 16, 24), (1, 1, 64, 48), (3, 1, 20, 10), (2, 2, 128, 64), (6, 3, 40, 130),
                                         (2, 1, 96, 32), (1, 1, 256, 72), (2, 2, 130, 20)])
def test_delta_rule_kernels(ops, H, G, dk, dv):
    g = torch.Generator().manual_seed(H * 1000 + dk)
    q_lens, slots = [37, 1, 18], [2, 0, 3]
    b = B(q_lens, slots)
    n, C = b.n_tokens, 2 * G * dk + H * dv
    row = ops.delta_row(H, G, dk, dv)
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=torch.float64)
    qkv, beta_z, low = rnd(n, C), rnd(2, n, H), rnd(2, n, 8)
    z, dt, a_log = rnd(3, n, H * dk + H * dv), rnd(H * dk), -4.0 + 4.0 * torch.rand(H, generator=g, dtype=torch.float64)
    S0 = 0.3 * rnd(5, H, dk, dv)
    act = torch.zeros(n, row, device=DEV)
    act[:, :C] = qkv.float().to(DEV)
    proj = torch.cat([torch.zeros(2, n, C, dtype=torch.float64), beta_z, low], -1).float().to(DEV)
    low16 = torch.empty(n, 8, dtype=torch.bfloat16, device=DEV)
    ops.delta_prep(act, proj, 2, C, C + H, 8, low16, H, G, dk, dv)
    assert close(low16, low.sum(0), 1e-2)
    state = S0.float().to(DEV)
    gate, out = torch.empty(n, H * dv, device=DEV), torch.empty(n, H * dv, device=DEV)
    ops.delta_scan(act, z.float().to(DEV), 3, dt.float().to(DEV), a_log.float().to(DEV), gate, b, state, out, H, G, dk, dv)
    zs = z.sum(0)
    assert close(gate, torch.sigmoid(zs[:, H * dk:]), 1e-5)
    qh = qkv[:, :G * dk].view(n, G, dk)
    kh = qkv[:, G * dk:2 * G * dk].view(n, G, dk)
    qh = qh / torch.sqrt((qh * qh).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    kh = kh / torch.sqrt((kh * kh).sum(-1, keepdim=True) + 1e-6)
    vh = qkv[:, 2 * G * dk:].view(n, H, dv)
    beta = torch.sigmoid(beta_z.sum(0))
    decay = torch.exp(-torch.exp(a_log)[None, :, None] * F.softplus(zs[:, :H * dk] + dt).view(n, H, dk))
    at = 0
    for ql, s in zip(q_lens, slots):
        for h in range(H):
            S = S0[s, h].clone()
            hq = h // (H // G)
            o = delta_rule(qh[at:at + ql, hq], kh[at:at + ql, hq], vh[at:at + ql, h], beta[at:at + ql, h],
                           decay[at:at + ql, h], S)
            assert close(out[at:at + ql].view(ql, H, dv)[:, h], o, 2e-5), (s, h)
            assert close(state[s, h], S, 2e-5), (s, h)
        at += ql
    assert torch.equal(state[1].cpu(), S0[1].float()) and torch.equal(state[4].cpu(), S0[4].float())


@pytest.mark.parametrize("W, blocks", [(48, 3), (64, 1), (30, 5), (512, 4)])
def test_rglru_kernels(ops, W, blocks):
    g = torch.Generator().manual_seed(W)
    bw = W // blocks
    q_lens, slots = [1, 300, 7, 2], [3, 1, 0, 2]
    b = B(q_lens, slots)
    n = b.n_tokens
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=torch.float64)
    gates, u, yx = rnd(blocks, n, 2 * bw), rnd(n, W), rnd(2, n, W + 5)
    ba, bi, by = rnd(W), rnd(W), rnd(W)
    lam = -7.0 + 7.5 * torch.rand(W, generator=g, dtype=torch.float64)          # decays from 0.9995 per token down
    S0 = rnd(4, W)
    dev = lambda t: t.float().to(DEV)
    state, coef = dev(S0), torch.empty(3, n, W, device=DEV)
    out = torch.empty(n, W, device=DEV)
    ops.rglru(dev(gates), dev(ba), dev(bi), dev(lam), dev(u), dev(yx), 2, dev(by), coef, b, state, out, W, bw, 8.0)
    r = torch.sigmoid(gates[:, :, :bw].permute(1, 0, 2).reshape(n, W) + ba)
    i = torch.sigmoid(gates[:, :, bw:].permute(1, 0, 2).reshape(n, W) + bi)
    a = torch.exp(-8.0 * r * F.softplus(lam))
    y = gelu_tanh(yx.sum(0)[:, :W] + by)
    at = 0
    for ql, s in zip(q_lens, slots):
        S = S0[s].clone()
        for t in range(at, at + ql):
            S = a[t] * S + torch.sqrt(1 - a[t] * a[t]) * i[t] * u[t]
            assert close(out[t], S * y[t], 2e-5), (s, t - at)
        assert close(state[s], S, 1e-5)
        at += ql


def test_routing_rule_kernel(ops):
    g = torch.Generator().manual_seed(5)
    for E, groups, keep, top in ((6, 3, 2, 2), (8, 4, 3, 3), (3, 1, 1, 1), (4, 2, 1, 2), (64, 8, 4, 6), (5, 5, 2, 2)):
        n = 50
        z = 2.0 * torch.randn(2, n, E, generator=g, dtype=torch.float64)
        corr = -0.8 + 0.6 * torch.randn(E, generator=g, dtype=torch.float64)      # many choice scores below zero
        choice = torch.empty(n * top, dtype=torch.int32, device=DEV)
        weight = torch.empty(n * top, device=DEV)
        counts = torch.zeros(E, dtype=torch.int32, device=DEV)
        ops.route_topk(z.float().to(DEV), 2, n, E, groups, keep, top, True, choice, weight, counts, sigmoid=True,
                       correction=corr.float().to(DEV), group_top2=True, norm_eps=1e-20, weight_scale=2.5)
        choice, weight = choice.cpu().view(n, top), weight.cpu().view(n, top)
        seen = torch.zeros(E, dtype=torch.int64)
        for t in range(n):
            chosen, w, margin = route(z.sum(0)[t], corr, groups, keep, top, 2.5)
            if margin < 1e-4:
                continue
            assert choice[t].tolist() == chosen.tolist(), (E, t)
            assert close(weight[t], w, 1e-5)
        for e in choice.reshape(-1).tolist():
            seen[e] += 1
        assert counts.cpu().tolist() == seen.tolist()


def test_head_norm_after_rotation(ops):
    g = torch.Generator().manual_seed(9)
    H, G, hd, size, dims, n = 4, 2, 32, 24, 8, 6            # heads of 24 features in rows of 32 (zeros after)
    b = B([4, 2], [1, 0])
    qkv = torch.randn(n, H + 2 * G, hd, generator=g, dtype=torch.float64)
    qkv[..., size:] = 0
    bias = torch.zeros((H + 2 * G) * hd, device=DEV)
    freq = rotary_frequencies(dims, 1e4, None)
    slot_pos = torch.tensor([7, 100], dtype=torch.int32, device=DEV)
    q_out = torch.empty(n, H * hd, device=DEV)
    kv_step = torch.empty(n, 2, G, hd, device=DEV)
    kc, vc = torch.zeros(2, G, 128, hd, device=DEV), torch.zeros(2, G, 128, hd, device=DEV)
    ops.qk_norm_rope_store(qkv.reshape(1, n, -1).float().to(DEV), 1, None, None, 1, 1, 0.0, freq.float().to(DEV), dims,
                           True, 1.0, b, q_out, kv_step, kc, vc, slot_pos, H, G, hd, True, 128, True, bias=bias,
                           head_norm=(1e-5, size))
    pos = torch.tensor([100, 101, 102, 103, 7, 8])
    rot = rotate_neighbours(qkv[:, :H + G], pos, freq)
    ref = rot / torch.sqrt((rot * rot).sum(-1, keepdim=True) / size + 1e-5)
    assert close(q_out.view(n, H, hd), ref[:, :H], 1e-5)
    assert close(kv_step[:, 0], ref[:, H:], 1e-5) and close(kv_step[:, 1], qkv[:, H + G:], 1e-6)
    assert close(kc[1, :, 100:104].permute(1, 0, 2), ref[:4, H:], 1e-5) and close(kc[0, :, 7:9].permute(1, 0, 2), ref[4:, H:], 1e-5)


# ------------------------------------------------------------------ the engine
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_residual_stream_run_by_run(name):
    cfg, seed = CONFIGS[name]
    w = weights_of(name)
    toks = random_tokens(40, cfg["vocab"], seed + 5)
    want = []
    ref, m = plain_logits(cfg, w, toks, taps=lambda ri, x: want.append(x.clone()))
    lm = _lm(cfg, w, "float32", max_context=256, max_batch=2)
    got = []
    lm.model.tap = lambda i, stream: got.append(stream.total().double().cpu())
    slots = lm.acquire(1)
    logits = lm.step([toks], slots, [list(range(len(toks)))])
    lm.model.tap = None
    assert len(got) == len(want) == len(m.runs)
    for i, (a, b) in enumerate(zip(got, want)):
        assert close(a, b, 2e-5), f"the residual stream differs after run {i} (layer {m.runs[i]})"
    assert close(logits, ref, TOL["float32"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_tail_portions_batches(name, dtype):
    cfg, seed = CONFIGS[name]
    w = weights_of(name)
    lengths = {"a": 150, "b": 1, "c": 66, "d": 23, "e": 129}           # across page borders (64, 128), one token
    reqs, refs = {}, {}
    for k, (rid, n) in enumerate(lengths.items()):
        reqs[rid], refs[rid] = safe_tokens(cfg, w, n, seed * 10 + k)
    tr = Trace()
    add_whole(tr, reqs)
    add_tail(tr, {r: reqs[r] for r in ("a", "c", "d")}, tail=40)
    for rid, sizes in (("a", [2, 3, 64, 2]), ("c", [63, 2]), ("d", [1, 2, 1, 5, 2, 2]), ("e", [64, 64])):
        add_portions(tr, rid, reqs[rid], sizes)
    # unequal requests together; the shorter end earlier; their slots and pages serve the next batch
    add_batches(tr, reqs, [["a", "b", "c"], ["d", "e", "b"], ["e", "a"]],
                {"a": 110, "b": 1, "c": 60, "d": 20, "e": 100})
    lm = _lm(cfg, w, dtype, max_context=256, max_batch=3, max_tokens=tr.max_tokens)
    got = run_in_process(lm, tr)
    compare(tr, got, refs, cfg["vocab"], TOL_OF.get(name, TOL)[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_key_in_prompts_portions_and_decoding(dtype):
    cfg, w = needle_model()
    n = 700
    toks = needle_tokens(n, 2, [63, 64, 65, 300, 511, 512, 640, 699])
    ref, _ = plain_logits(cfg, w, toks)
    blind = list(toks)
    blind[2] = 9
    lost, _ = plain_logits(cfg, w, blind)
    assert (ref[699] - lost[699]).abs().max() > 0.3 * ref.abs().max()            # a lost needle would show
    refs, reqs = {"n": ref}, {"n": toks}
    tr = Trace()
    add_whole(tr, reqs)
    add_tail(tr, reqs, tail=70)
    add_portions(tr, "n", toks, [1, 62, 1, 2, 446, 2, 127])
    lm = _lm(cfg, w, dtype, max_context=1024, max_batch=2, max_tokens=tr.max_tokens)
    compare(tr, run_in_process(lm, tr), refs, cfg["vocab"], TOL[dtype])
    # the needle as the sequence's very first token, the probe right after it
    first = needle_tokens(40, 0, [1, 39])
    ref0, _ = plain_logits(cfg, w, first)
    tr = Trace()
    add_whole(tr, {"f": first})
    add_tail(tr, {"f": first}, tail=39)
    compare(tr, run_in_process(lm, tr), {"f": ref0}, cfg["vocab"], TOL[dtype])
    assert ref0[1][NEEDLE] > 1.0 > ref0[5][NEEDLE]          # the probe at position 1 found the needle before it


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["samu_a", "samu_b"])
def test_long_decoding_through_the_captured_step(name, dtype):
    cfg, seed = CONFIGS[name]
    w = weights_of(name)
    reqs, refs = {}, {}
    for k, (rid, n) in enumerate({"x": 200, "y": 90, "z": 141}.items()):
        reqs[rid], refs[rid] = safe_tokens(cfg, w, n, seed * 7 + k)
    lm = _lm(cfg, w, dtype, max_context=256, max_batch=3)
    forced_decode(lm, reqs, {"x": 30, "y": 3, "z": 65}, refs, TOL[dtype])
    # the same slots again, other requests: nothing of the earlier states is left
    forced_decode(lm, reqs, {"x": 1, "y": 64, "z": 2}, refs, TOL[dtype], order=["z", "x", "y"])


def test_greedy_generation_through_the_entry_point():
    cfg, seed = CONFIGS["samu_a"]
    w = weights_of("samu_a")
    lm = _lm(cfg, w, "float32", max_context=128, max_batch=2)
    prompts = [random_tokens(9, cfg["vocab"], 1), random_tokens(21, cfg["vocab"], 2), random_tokens(2, cfg["vocab"], 3)]
    outs = lm.generate(prompts, max_new_tokens=12, temperature=0.0, ignore_eos=True)
    for p, o in zip(prompts, outs):
        assert list(o.tokens) == plain_generate_greedy(cfg, w, p, 12)


def test_trace_replay_program(tmp_path):
    cfg, seed = CONFIGS["samu_c"]
    w = weights_of("samu_c")
    from yalm_b200.weights import safetensors_io as st
    model_dir = tmp_path / "model"
    os.makedirs(model_dir)
    with open(model_dir / "config.json", "w") as f:
        json.dump(cfg, f)
    st.write_file(str(model_dir / "model.safetensors"), w)
    reqs, refs = {}, {}
    for k, (rid, n) in enumerate({"a": 70, "b": 9}.items()):
        reqs[rid], refs[rid] = safe_tokens(cfg, w, n, 50 + k)
    tr = Trace()
    add_whole(tr, reqs)
    add_tail(tr, reqs, tail=8)
    add_batches(tr, reqs, [["a", "b"]], {"a": 60, "b": 4})
    for dtype in ("bfloat16", "float32"):
        out = tmp_path / f"out_{dtype}"
        os.makedirs(out)
        got = run_trace_run(str(model_dir), dtype, tr, str(out))
        compare(tr, got, refs, cfg["vocab"], TOL_OF["samu_c"][dtype])
