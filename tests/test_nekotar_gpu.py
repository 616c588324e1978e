"""Nekotar on a GPU against the plain implementation: each added kernel alone, then the engine --
whole prompts, the tail one token at a time, prompts in portions down to two tokens, batches of
unequal requests whose shorter ones end earlier (slots and pages used again), keys just inside
and just outside a window and the kept first positions, in prompts and in decoding, far keys
among hundreds and at page borders, first tokens, long decoding through the captured decode
step, greedy generation through the entry point, and the trace replay program."""
import json
import os

import pytest
import torch

from nekotar_helpers import (CONFIGS, NEKO_A, TOL, add_portions, make_weights, needle_model, needle_tokens,
                             plain_generate_greedy, random_tokens, references, weights_of)
from plain_nekotar import (plain_forward, plain_gelu_tanh, plain_kept_window_mask, plain_latent, plain_norm,
                           plain_rotate, plain_softmax_mix, plain_sublayer, plain_wkv)
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
        self.q_start = torch.tensor(qs, dtype=torch.int32, device=DEV)
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
        self.token_seq = torch.tensor(sum([[i] * q for i, q in enumerate(q_lens)], []),
                                      dtype=torch.int32, device=DEV)


def _lm(cfg, w, dtype, **kw):
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    return LM(config_from_dict(cfg), dict(w), dtype=dtype, **kw)


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("copies", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dim, rows", [(64, 5), (100, 3), (1000, 70), (4100, 2), (30, 4), (2048, 300)])
def test_residual_copies_write_and_read(ops, copies, dim, rows):
    g = torch.Generator().manual_seed(dim + copies)
    X = torch.randn(copies, rows, dim, generator=g)
    y = torch.randn(3, rows, dim, generator=g)                       # a product in three slices
    w = {"hc.in": torch.randn(copies, generator=g), "hc.out": torch.randn(copies, generator=g),
         "hc.mix": torch.randn(copies, copies, generator=g)}
    nw = 1 + 0.1 * torch.randn(dim, generator=g)
    # the oracle: a sublayer that returns y, then the next sublayer's read of the new copies
    new = plain_sublayer(w, "hc", X.double(), nw, 1e-6, 0.7, lambda h: y.double().sum(0))
    u = torch.einsum("s,std->td", w["hc.in"].double(), new)
    for dt in (torch.float32, torch.bfloat16):
        Xd = X.clone().to(DEV)
        h = torch.empty(rows, dim, dtype=dt, device=DEV)
        ops.hc_step(Xd, write=(y.to(DEV), 3, w["hc.mix"].to(DEV), w["hc.out"].to(DEV), 0.7),
                    read=(w["hc.in"].to(DEV), nw.to(DEV), 1e-6, h))
        assert (Xd.cpu() - new).abs().max().item() <= 2e-5 * max(1.0, new.abs().max().item())
        ref = plain_norm(u, nw, 1e-6)
        tol = 3e-5 if dt == torch.float32 else 2e-2
        assert (h.float().cpu() - ref).abs().max().item() <= tol * ref.abs().max().item()
    # a read alone without a norm: the weighted sum itself, float32 (the model's output reads the plain sum)
    Xd = X.clone().to(DEV)
    total = torch.empty(rows, dim, device=DEV)
    ops.hc_step(Xd, read=(torch.ones(copies, device=DEV), None, 0.0, total))
    assert torch.equal(Xd.cpu(), X) and (total.cpu() - X.sum(0)).abs().max().item() <= 1e-5
    # a write alone
    ops.hc_step(Xd, write=(y.to(DEV), 3, w["hc.mix"].to(DEV), w["hc.out"].to(DEV), 0.7))
    assert (Xd.cpu() - new).abs().max().item() <= 2e-5 * max(1.0, new.abs().max().item())


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_normed_embedding_and_gelu(ops, dt):
    g = torch.Generator().manual_seed(5)
    table = torch.randn(50, 72, generator=g).to(dt)
    nw = 1 + 0.1 * torch.randn(72, generator=g)
    toks = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    x = torch.empty(4, 72, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed(toks.to(DEV), table.to(DEV), x, status)
    ops.sum_norm(x, 1.0, [], nw.to(DEV), 1e-6)
    ref = plain_norm(table.float()[toks.long()], nw, 1e-6)
    assert (x.cpu() - ref).abs().max().item() <= 1e-5 and status.item() == 0
    z = 3.0 * torch.randn(2, 7, 33, generator=g)
    out = torch.empty(7, 33, dtype=dt, device=DEV)
    ops.activation_rows(z.to(DEV), 2, out, ops.GELU_TANH)
    ref = plain_gelu_tanh(z.sum(0).double()).float()
    assert (out.float().cpu() - ref).abs().max().item() <= (1e-5 if dt == torch.float32 else 3e-2)
    ops.activation_rows(z.to(DEV), 2, out, ops.TANH)
    assert (out.float().cpu() - torch.tanh(z.sum(0))).abs().max().item() <= (1e-5 if dt == torch.float32 else 1e-2)


@pytest.mark.parametrize("H, d, rank", [(3, 16, 8), (1, 64, 16), (2, 20, 3), (2, 128, 32), (1, 200, 5), (2, 32, 1)])
def test_wkv_mixer_in_portions(ops, H, d, rank):
    """Token shift, decay, recurrence, head norm and gate through the kernels, two sequences in
    portions (one token, two tokens, many), against the plain mixer on each whole sequence."""
    g = torch.Generator().manual_seed(d + rank)
    D = 40
    cfg = {"architecture": "Nekotar", "vocab": 8, "width": D, "norm": {"eps": 1e-5}, "residual_mult": 1.0,
           "streams": 1, "layers": [{"type": "wkv", "mixer": {"heads": H, "dim": d}, "mlp": None}]}
    w = {k: v.float() for k, v in make_weights(cfg, d, torch.float32, {0: rank}).items()}
    p, m = "l0.mix", cfg["layers"][0]["mixer"]
    seqs = {2: torch.randn(41, D, generator=g), 0: torch.randn(19, D, generator=g)}
    dev = lambda name: w[f"{p}.{name}"].to(DEV)
    mu = torch.stack([dev(f"mu.{s}") for s in "rkvgw"]).contiguous()
    state = torch.zeros(4, H, d, d, device=DEV)
    prev = torch.zeros(4, D, device=DEV)
    state[1], prev[1] = 7.0, 3.0                          # another sequence's state stays as it is
    got = {s: [] for s in seqs}
    at = {s: 0 for s in seqs}
    for sizes in [{2: 17, 0: 2}, {2: 1, 0: 1}, {2: 1, 0: 1}, {2: 19, 0: 15}, {2: 3}]:
        slots = list(sizes)
        b = B([sizes[s] for s in slots], slots)
        n = b.n_tokens
        h = torch.cat([seqs[s][at[s]:at[s] + sizes[s]] for s in slots]).to(DEV)
        mixed = torch.empty(5, n, D, device=DEV)
        ops.token_shift(h, prev, mu, mixed, b)
        # the products as two unequal slices each, as a split product leaves them
        two = lambda t: torch.stack([0.25 * t, 0.75 * t]).contiguous()
        proj = [(two(mixed[i] @ dev(s).T), 2) for i, s in enumerate("rkvg")]
        z = (two(torch.tanh(mixed[4] @ dev("w1").T) @ dev("w2").T), 2)
        act = torch.empty(n, 3 * H * d + H * d, device=DEV)
        gate = torch.empty(n, H * d, device=DEV)
        o = torch.empty(n, H * d, device=DEV)
        ops.wkv(proj[0], proj[1], proj[2], proj[3], z, dev("w0"), dev("u").reshape(-1).contiguous(), act, gate,
                h, prev, b, state, o, H, d, d)
        normed = torch.empty(n, H * d, device=DEV)
        ops.wkv_out(o, dev("norm"), gate, normed, H, d, 1e-5)
        out = normed @ dev("o").T
        qs = b.q_start.tolist()
        for i, s in enumerate(slots):
            got[s].append(out[qs[i]:qs[i + 1]].cpu())
            at[s] += sizes[s]
            assert torch.equal(prev[s].cpu(), seqs[s][at[s] - 1])          # the previous input is handed on
    for s, h in seqs.items():
        ref = plain_wkv({k: v.double() for k, v in w.items()}, p, m, h.double(), 1e-5).float()
        err = (torch.cat(got[s]) - ref).abs().max(-1).values
        bad = (err > 5e-5 * max(1.0, ref.abs().max().item())).nonzero()
        assert not bad.numel(), f"sequence {s}: first wrong token {int(bad[0])}, error {float(err.max()):.3e}"
    assert bool((state[1] == 7.0).all()) and bool((prev[1] == 3.0).all())


@pytest.mark.parametrize("H, d, rd, dv, rank", [(4, 16, 8, 24, 40), (3, 32, 16, 32, 64), (5, 24, 4, 8, 20),
                                                (2, 8, 32, 16, 96), (1, 64, 0, 64, 128), (2, 32, 64, 32, 192)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_latent_mixer_in_portions(ops, H, d, rd, dv, rank, dt):
    """The cached row [normed latent | rotated key part | 0], queries moved into the latent space,
    attention with that row as key and value, expansion and gate: two sequences in portions against
    the plain mixer on each whole sequence."""
    from plain_nekotar import plain_latent_attention
    g = torch.Generator().manual_seed(d + rank)
    D, hd, cap, scale, base, eps = 48, -(-(rank + rd) // 16) * 16, 64, 0.2, 1e4, 1e-5
    m = {"heads": H, "dim": d, "rot_dim": rd, "vdim": dv, "kv_rank": rank, "scale": scale, "rot": {"base": base, "dims": rd}}
    p = "m"
    w = {f"{p}.q": torch.randn(H * (d + rd), D, generator=g) * 0.3, f"{p}.dkv": torch.randn(rank + rd, D, generator=g) * 0.3,
         f"{p}.dkv.norm": 1 + 0.1 * torch.randn(rank, generator=g), f"{p}.uk": torch.randn(H * d, rank, generator=g) * 0.3,
         f"{p}.uv": torch.randn(H * dv, rank, generator=g) * 0.3, f"{p}.g": torch.randn(H * dv, D, generator=g) * 0.3,
         f"{p}.o": torch.eye(H * dv)}
    w = {k: v.to(dt).float() for k, v in w.items()}         # values that the storage type holds exactly
    seqs = {1: torch.randn(45, D, generator=g), 3: torch.randn(36, D, generator=g)}
    freq = torch.tensor([base ** (-2.0 * i / max(rd, 2)) for i in range(max(rd // 2, 1))]).to(DEV)
    cache = torch.zeros(4, 1, cap, hd, dtype=dt, device=DEV)
    slot_pos = torch.zeros(4, dtype=torch.int32, device=DEV)
    uk = w[f"{p}.uk"].to(dt).to(DEV)
    uv = w[f"{p}.uv"].view(H, dv, rank).transpose(1, 2).contiguous().to(dt).to(DEV)
    got = {s: [] for s in seqs}
    rows = {s: [] for s in seqs}
    at = {s: 0 for s in seqs}
    for sizes in [{1: 6, 3: 1}, {1: 1, 3: 9}, {1: 2, 3: 2}, {1: 30, 3: 20}] + [{1: 1, 3: 1}] * 6:
        sizes = {s: min(n, len(seqs[s]) - at[s]) for s, n in sizes.items() if at[s] < len(seqs[s])}
        slots = list(sizes)
        b = B([sizes[s] for s in slots], slots)
        n = b.n_tokens
        h = torch.cat([seqs[s][at[s]:at[s] + sizes[s]] for s in slots]).to(DEV)
        two = lambda t: torch.stack([0.25 * t, 0.75 * t]).contiguous()
        kv_step = torch.full((n, 2, 1, hd), 9.0, dtype=dt, device=DEV)
        ops.latent_store(two(h @ w[f"{p}.dkv"].to(DEV).T), 2, w[f"{p}.dkv.norm"].to(DEV), eps, freq, b, slot_pos,
                         kv_step, cache, rank, rd, hd, cap)
        q_lat = torch.full((n, H * hd), 9.0, dtype=dt, device=DEV)
        ops.latent_absorb_q(two(h @ w[f"{p}.q"].to(DEV).T), 2, uk, freq, b, slot_pos, q_lat, H, d, rd, rank, hd)
        o_lat = torch.empty(n, H * hd, dtype=dt, device=DEV)
        nsplit = 3 if n == len(slots) else 1
        po, pml = torch.empty(n, H, nsplit, hd, device=DEV), torch.empty(n, H, nsplit, 2, device=DEV)
        ops.attention(q_lat, kv_step, cache, cache, b, slot_pos, o_lat, H, 1, hd, cap, None, nsplit, po, pml, scale=scale)
        out = torch.empty(n, H * dv, dtype=dt, device=DEV)
        ops.latent_expand(o_lat, uv, two(h @ w[f"{p}.g"].to(DEV).T), 2, out, H, rank, dv, hd)
        ops.advance(b, slot_pos)
        assert torch.equal(kv_step[:, 0], kv_step[:, 1])
        qs = b.q_start.tolist()
        for i, s in enumerate(slots):
            got[s].append(out[qs[i]:qs[i + 1]].float().cpu())
            rows[s].append(kv_step[qs[i]:qs[i + 1], 0, 0].float().cpu())
            at[s] += sizes[s]
    tol = 5e-5 if dt == torch.float32 else 4e-2
    for s, h in seqs.items():
        c, kr = plain_latent(w, p, m, h, eps)
        row = torch.cat(rows[s])
        assert (row[:, :rank] - c).abs().max().item() <= (1e-5 if dt == torch.float32 else 2e-2) * c.abs().max().item()
        if rd:
            assert (row[:, rank:rank + rd] - kr).abs().max().item() <= (1e-5 if dt == torch.float32 else 2e-2) * max(1.0, float(kr.abs().max()))
        assert not row[:, rank + rd:].any()                                  # the padding holds zeros
        assert torch.equal(cache[s, 0, :len(h)].float().cpu(), row)          # and the cache the same rows
        ref = plain_latent_attention(w, p, m, h, c, kr)
        err = (torch.cat(got[s]) - ref).abs().max(-1).values
        bad = (err > tol * ref.abs().max()).nonzero()
        assert not bad.numel(), f"sequence {s}: first wrong position {int(bad[0])}, error {float(err.max()):.3e}"


@pytest.mark.parametrize("window, keep", [(7, 3), (5, 12), (16, 1), (64, 64), (3, 70)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_window_with_kept_first_positions(ops, window, keep, dt):
    """Two sequences in portions, then one token at a time: every query sees its window and the
    kept first positions, whether they come from this step's rows or from the cache."""
    g = torch.Generator().manual_seed(window * 31 + keep)
    H, G, hd, T, cap = 4, 2, 16, 150, 192
    tol = 1e-5 if dt == torch.float32 else 2e-2
    seqs = {1: T, 3: T - 19}
    data = {s: (torch.randn(n, H, hd, generator=g).to(dt), torch.randn(n, G, hd, generator=g).to(dt),
                torch.randn(n, G, hd, generator=g).to(dt)) for s, n in seqs.items()}
    kc, vc = torch.zeros(4, G, cap, hd, dtype=dt, device=DEV), torch.zeros(4, G, cap, hd, dtype=dt, device=DEV)
    slot_pos = torch.zeros(4, dtype=torch.int32, device=DEV)
    got = {s: [] for s in seqs}
    at = {s: 0 for s in seqs}
    portions = [{1: 6, 3: 1}, {1: 1, 3: 9}, {1: 2, 3: 2}, {1: 61, 3: 70}] + [{1: 1, 3: 1}] * 100
    for sizes in portions:
        sizes = {s: min(n, seqs[s] - at[s]) for s, n in sizes.items() if at[s] < seqs[s]}
        if not sizes:
            break
        slots = list(sizes)
        b = B([sizes[s] for s in slots], slots)
        q = torch.cat([data[s][0][at[s]:at[s] + sizes[s]] for s in slots]).reshape(b.n_tokens, H * hd).to(DEV)
        kv = torch.stack([torch.cat([data[s][1][at[s]:at[s] + sizes[s]] for s in slots]),
                          torch.cat([data[s][2][at[s]:at[s] + sizes[s]] for s in slots])], 1).contiguous().to(DEV)
        ops.cache_write(kv, b, kc, vc, slot_pos, G, hd, cap)
        out = torch.empty(b.n_tokens, H * hd, dtype=dt, device=DEV)
        nsplit = 3 if b.n_tokens == len(slots) else 1
        po = torch.empty(b.n_tokens, H, nsplit, hd, device=DEV)
        pml = torch.empty(b.n_tokens, H, nsplit, 2, device=DEV)
        ops.attention(q, kv, kc, vc, b, slot_pos, out, H, G, hd, cap, window, nsplit, po, pml, scale=0.3,
                      keep_first=keep)
        ops.advance(b, slot_pos)
        qs = b.q_start.tolist()
        for i, s in enumerate(slots):
            got[s].append(out[qs[i]:qs[i + 1]].float().cpu())
            at[s] += sizes[s]
    for s, n in seqs.items():
        q, k, v = (t.float() for t in data[s])
        k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
        ref = plain_softmax_mix(q, k, v, 0.3, plain_kept_window_mask(n, window, keep))
        out = torch.cat(got[s]).view(n, H, hd)
        err = (out - ref).abs().max(-1).values.max(-1).values
        bad = (err > tol * ref.abs().max()).nonzero()
        assert not bad.numel(), f"sequence {s}: first wrong position {int(bad[0])} (window {window}, kept {keep})"


@pytest.mark.parametrize("window, keep", [(50, 70), (64, 1), (130, 64), (7, 200)])
@pytest.mark.parametrize("hd", [32, 64, 128, 256])
def test_prompt_kernel_with_kept_first_positions(ops, window, keep, hd):
    """The tensor-core kernel for prompts: kept positions in blocks of their own before the window's
    blocks, from the cache (a later portion) or from the step's rows, also more kept positions than
    a key block holds and a window that reaches back into them."""
    g = torch.Generator().manual_seed(window * 7 + keep + hd)
    dt, H, G, cap = torch.bfloat16, 4, 2, 448
    seqs = {0: 430, 2: 201}
    data = {s: (torch.randn(n, H, hd, generator=g).to(dt), torch.randn(n, G, hd, generator=g).to(dt),
                torch.randn(n, G, hd, generator=g).to(dt)) for s, n in seqs.items()}
    kc, vc = torch.zeros(3, G, cap, hd, dtype=dt, device=DEV), torch.zeros(3, G, cap, hd, dtype=dt, device=DEV)
    slot_pos = torch.zeros(3, dtype=torch.int32, device=DEV)
    got, at = {s: [] for s in seqs}, {s: 0 for s in seqs}
    for sizes in ({0: 71, 2: 2}, {0: 2, 2: 199}, {0: 193}, {0: 164}):
        slots = list(sizes)
        b = B([sizes[s] for s in slots], slots)
        q = torch.cat([data[s][0][at[s]:at[s] + sizes[s]] for s in slots]).reshape(b.n_tokens, H * hd).to(DEV)
        kv = torch.stack([torch.cat([data[s][1][at[s]:at[s] + sizes[s]] for s in slots]),
                          torch.cat([data[s][2][at[s]:at[s] + sizes[s]] for s in slots])], 1).contiguous().to(DEV)
        ops.cache_write(kv, b, kc, vc, slot_pos, G, hd, cap)
        out = torch.empty(b.n_tokens, H * hd, dtype=dt, device=DEV)
        ops.attention_exact_prefill(q, kv, kc, vc, b, slot_pos, out, H, G, hd, cap, window, scale=0.2,
                                    keep_first=keep)
        ops.advance(b, slot_pos)
        qs = b.q_start.tolist()
        for i, s in enumerate(slots):
            got[s].append(out[qs[i]:qs[i + 1]].float().cpu())
            at[s] += sizes[s]
    for s, n in seqs.items():
        q, k, v = (t.float() for t in data[s])
        k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
        ref = plain_softmax_mix(q, k, v, 0.2, plain_kept_window_mask(n, window, keep))
        err = (torch.cat(got[s]).view(n, H, hd) - ref).abs().max(-1).values.max(-1).values
        bad = (err > 2e-2 * ref.abs().max()).nonzero()
        assert not bad.numel(), f"sequence {s}: first wrong position {int(bad[0])} (window {window}, kept {keep})"


@pytest.mark.parametrize("M, N, K", [(300, 520, 264), (129, 64, 64), (2048, 1536, 512)])
@pytest.mark.parametrize("act", ["gelu", "tanh"])
def test_product_with_an_activation_on_the_way_out(ops, M, N, K, act):
    """act(a W^T) in the two-SM product's epilogue against the same in 64-bit floats: through the
    copy engine (rows of 16-byte multiples) and through the threads' own stores."""
    g = torch.Generator().manual_seed(M + N)
    a = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.2).to(torch.bfloat16)
    z = a.double() @ w.double().T
    ref = plain_gelu_tanh(z) if act == "gelu" else torch.tanh(z)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for dt, tol in ((torch.bfloat16, 1e-2), (torch.float32, 2e-5)):
        out = torch.empty(M, N, dtype=dt, device=DEV)
        ops.gemm_2sm_act(a.to(DEV), w.to(DEV), out, ops.GELU_TANH if act == "gelu" else ops.TANH, status)
        assert int(status.item()) == 0
        assert (out.double().cpu() - ref).abs().max().item() <= tol * ref.abs().max().item()


# ------------------------------------------------------------------ the engine against the plain model
def _requests(cfg, seed):
    V = cfg["vocab"]
    # (the one-token request: a sequence's first wkv output is (r . (u k)) v divided by its own root
    # mean square, i.e. v / rms(v) times the SIGN of a sum; a token whose sum nearly cancels has no
    # stable answer in 16 bits, so this seed is one whose tokens do not)
    return {"a": random_tokens(150, V, seed), "b": random_tokens(67, V, seed + 1), "c": random_tokens(1, V, seed + 7),
            "d": random_tokens(23, V, seed + 3), "e": random_tokens(131, V, seed + 4), "f": random_tokens(2, V, seed + 5)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_layer_against_the_plain_model(name, dtype):
    """The sum of the residual copies after every layer, for a prompt and for the same prompt in portions."""
    cfg, seed = CONFIGS[name]
    w = weights_of(name)
    toks = random_tokens(90, cfg["vocab"], seed + 11)
    want = []
    plain_forward(cfg, w, toks, layer_outputs=want)
    lm = _lm(cfg, w, dtype, max_context=128, max_batch=2)
    tol = 3e-5 if dtype == "float32" else 5e-2
    for cuts in ([90], [2, 63, 1, 24]):
        got = [[] for _ in want]
        lm.model.tap = lambda i, stream: got[i].append(stream.total().float().cpu())
        slot = lm.acquire(1)
        at = 0
        for n in cuts:
            lm.step([toks[at:at + n]], slot, [[]])
            at += n
        lm.release(slot)
        lm.model.tap = None
        for i, ref in enumerate(want):
            err = (torch.cat(got[i]) - ref).abs().max().item() / ref.abs().max().item()
            assert err <= tol, f"layer {i} ({cfg['layers'][i]['type']}), portions {cuts}: error {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_schedules_against_the_plain_model(name, dtype):
    cfg, seed = CONFIGS[name]
    w = weights_of(name, torch.float16 if dtype == "float16" else torch.bfloat16)
    reqs = _requests(cfg, seed)
    refs = references(cfg, w, reqs)
    tr = Trace()
    add_whole(tr, reqs)
    add_tail(tr, {k: reqs[k] for k in "abe"}, tail=48)
    add_portions(tr, "a", reqs["a"], [2, 2, 31, 64, 3, 2])
    add_portions(tr, "e", reqs["e"], [64, 1, 63, 2])
    add_portions(tr, "b", reqs["b"], [33, 32])
    add_portions(tr, "d", reqs["d"], [1, 1, 1, 2])
    add_batches(tr, reqs, [["a", "b", "c", "d"], ["e", "b", "f"], ["d", "a", "e"]],
                {"a": 100, "b": 40, "c": 1, "d": 20, "e": 66, "f": 1})
    # few slots and a page pool sized by the tokens held: slots and pages are freed and used again
    lm = _lm(cfg, w, dtype, max_context=192, max_batch=4, max_tokens=tr.max_tokens)
    got = run_in_process(lm, tr)
    compare(tr, got, refs, cfg["vocab"], TOL[dtype])
    lm.rt.check_status()
    # and with one block per sequence in place of pages
    lm2 = _lm(cfg, w, dtype, max_context=192, max_batch=4)
    tr2 = Trace()
    add_batches(tr2, reqs, [["a", "b", "c", "d"], ["e", "b"]], {"a": 100, "b": 40, "c": 1, "d": 20, "e": 66})
    compare(tr2, run_in_process(lm2, tr2), refs, cfg["vocab"], TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_does_not_depend_on_its_batch(dtype):
    cfg, seed = CONFIGS["neko_a"]
    w = weights_of("neko_a")
    reqs = _requests(cfg, seed)
    lm = _lm(cfg, w, dtype, max_context=192, max_batch=4)
    alone = {}
    for rid in "abd":
        s = lm.acquire(1)
        alone[rid] = lm.step([reqs[rid]], s, [list(range(len(reqs[rid])))]).cpu()
        lm.release(s)
    s = lm.acquire(3)
    both = lm.step([reqs[r] for r in "abd"], s, [list(range(len(reqs[r]))) for r in "abd"]).cpu()
    lm.release(s)
    at = 0
    for rid in "abd":
        n = len(reqs[rid])
        if dtype == "float32":
            assert torch.equal(both[at:at + n], alone[rid]), rid       # one chain of additions per output
        else:                                                          # the products' tiles follow the step's size
            assert (both[at:at + n] - alone[rid]).abs().max().item() <= TOL[dtype] * alone[rid].abs().max().item(), rid
        at += n


def test_a_slot_that_is_used_again_starts_from_nothing():
    """The recurrent state, the previous input and the cached rows of a finished request must not
    reach the next request in its slot."""
    cfg, seed = CONFIGS["neko_b"]
    w = weights_of("neko_b")
    reqs = _requests(cfg, seed)
    refs = references(cfg, w, reqs)
    lm = _lm(cfg, w, "float32", max_context=192, max_batch=1, max_tokens=192)
    for rid in "abeda":
        s = lm.acquire(1)
        got = lm.step([reqs[rid]], s, [list(range(len(reqs[rid])))]).cpu()
        lm.release(s)
        assert (got - refs[rid]).abs().max().item() <= TOL["float32"] * refs[rid].abs().max().item(), rid


# ------------------------------------------------------------------ one key that stands out
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size, keep, dim", [(9, 4, 16), (64, 64, 32), (70, 5, 16), (30, 40, 64), (128, 1, 16)])
def test_edges_of_the_window_and_the_kept_positions(size, keep, dim, dtype):
    cfg, w = needle_model("attention", size, keep, dim=dim)
    for at in (keep - 1, keep):                     # the last kept position (seen for ever), the first that is not
        edge = at + size                            # the first position that the window no longer covers
        n = edge + 330
        probes = sorted({edge - 1, edge, edge + 1, n - 2})      # n - 2: hundreds of positions later
        toks = needle_tokens(n, at, probes)
        ref = {"n": plain_forward(cfg, w, toks)}
        lm = _lm(cfg, w, dtype, max_context=n + 1, max_batch=2, max_tokens=2 * (n + 64))
        # in a whole prompt, in a prompt cut right at the edge, decoded token by token, and in pairs
        for cuts in ([n], [edge - 1, 1, 1], [at + 1] + [1] * (n - at - 1), [2, 2, 2] + [64] * 8):
            tr = Trace()
            add_portions(tr, "n", toks, list(cuts))
            compare(tr, run_in_process(lm, tr), ref, cfg["vocab"], TOL[dtype])
        # the same through the captured decode step
        forced_decode(lm, {"n": toks}, {"n": at + 2}, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["latent", "shared_latent"])
@pytest.mark.parametrize("at", [0, 3, 63, 64])
def test_a_far_key_of_the_latent_attention(kind, at, dtype):
    """One latent row among hundreds decides the probes' logits: at the sequence's start, and on
    both sides of a page's border; probes hundreds of positions later, in a prompt and decoded."""
    cfg, w = needle_model(kind)
    n = 520
    probes = [at + 1, 127, 128, 300, n - 2]
    toks = needle_tokens(n, at, probes)
    ref = {"n": plain_forward(cfg, w, toks)}
    lm = _lm(cfg, w, dtype, max_context=n + 1, max_batch=2, max_tokens=2 * (n + 64))
    for cuts in ([n], [at + 1, 2, 64, 61], [127] + [1] * 5 + [300], [2] * 40):
        tr = Trace()
        add_portions(tr, "n", toks, list(cuts))
        compare(tr, run_in_process(lm, tr), ref, cfg["vocab"], TOL[dtype])
    forced_decode(lm, {"n": toks}, {"n": at + 1}, ref, TOL[dtype])


# ------------------------------------------------------------------ decode path, generation, replay program
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_long_decoding_through_the_captured_step(name, dtype):
    cfg, seed = CONFIGS[name]
    w = weights_of(name)
    V = cfg["vocab"]
    reqs = {"x": random_tokens(260, V, seed + 7), "y": random_tokens(150, V, seed + 8), "z": random_tokens(40, V, seed + 9)}
    refs = references(cfg, w, reqs)
    lm = _lm(cfg, w, dtype, max_context=320, max_batch=3, max_tokens=3 * 320)
    rows = forced_decode(lm, reqs, {"x": 30, "y": 3, "z": 1}, refs, TOL[dtype])
    assert rows.shape[0] > 400
    assert lm.engine._graphs, "decode steps of a lasting batch are captured"


def test_greedy_generation_through_the_entry_point():
    cfg, seed = CONFIGS["neko_a"]
    w = weights_of("neko_a")
    lm = _lm(cfg, w, "float32", max_context=128, max_batch=3)
    prompts = [random_tokens(n, cfg["vocab"], 40 + n) for n in (9, 1, 30, 17)]
    out = lm.generate(prompts, max_new_tokens=24, temperature=0.0, ignore_eos=True)
    for p, c in zip(prompts, out):
        assert c.tokens == plain_generate_greedy(cfg, w, p, 24)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_replay_program_on_a_model_folder(tmp_path, dtype):
    from yalm_b200.weights import write_file
    cfg, seed = CONFIGS["neko_c"]
    w = weights_of("neko_c")
    folder = tmp_path / "model"
    os.makedirs(folder)
    with open(folder / "config.json", "w") as f:
        json.dump(cfg, f)
    write_file(str(folder / "model.safetensors"), w)
    reqs = {k: v for k, v in _requests(cfg, seed).items() if k in "abd"}
    refs = references(cfg, w, reqs)
    tr = Trace()
    add_whole(tr, reqs)
    add_tail(tr, {"a": reqs["a"]}, tail=40)
    add_batches(tr, reqs, [["a", "b", "d"]], {"a": 110, "b": 30, "d": 5})
    out = tmp_path / "out"
    os.makedirs(out)
    compare(tr, run_trace_run(str(folder), dtype, tr, str(out)), refs, cfg["vocab"], TOL[dtype])


def test_command_line_on_a_random_model_folder(tmp_path):
    """python -m yalm_b200: the random-weights mode writes a Nekotar model folder, greedy completion
    of token-id prompts matches the plain implementation on the weights it wrote, and sampling with
    a temperature repeats under one seed."""
    import subprocess
    import sys
    from trace_tools import ROOT
    from yalm_b200.weights import load_checkpoint
    (tmp_path / "cfg.json").write_text(json.dumps(NEKO_A))
    model = str(tmp_path / "model")
    base = [sys.executable, "-m", "yalm_b200", model, "--dtype", "float32"]
    r = subprocess.run(base + ["--random-weights", str(tmp_path / "cfg.json"), "--seed", "3",
                               "--tokens", "5,6,7;9,10", "-n", "6", "-t", "0"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "Nekotar" in r.stdout and os.path.isfile(os.path.join(model, "model.safetensors"))
    lines = [l for l in r.stdout.splitlines() if l.startswith("tokens:")]
    assert len(lines) == 2
    with open(os.path.join(model, "config.json")) as f:
        cfg = json.load(f)
    w = load_checkpoint(model)
    for line, prompt in zip(lines, ([5, 6, 7], [9, 10])):
        assert [int(t) for t in line.split("(")[0].split()[1:]] == plain_generate_greedy(cfg, w, prompt, 6)
    sampled = []
    for _ in range(2):
        r = subprocess.run(base + ["--tokens", "5,6,7", "-n", "8", "-t", "0.9", "--seed", "11"],
                           capture_output=True, text=True, cwd=ROOT, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        sampled.append([l for l in r.stdout.splitlines() if l.startswith("tokens:")])
    assert sampled[0] == sampled[1] and sampled[0]
