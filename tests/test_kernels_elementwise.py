"""The row-wise kernels and the sampler alone, against the plain implementation's functions, at
sizes other than the engine's."""
import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,E,M", [(50, 24, 7), (1000, 2050, 33)])
def test_embed_gather(V, E, M, dtype):
    from fastgguf_b200 import ops
    table = torch.randn(V, E).to(dtype).cuda()
    toks = torch.randint(0, V, (M,), dtype=torch.int32).cuda()
    got = ops.embed_gather(table, toks)
    assert got.dtype == torch.float32 and torch.equal(got.cpu(), P.plain_embedding(table.cpu().float(), toks.cpu().tolist()))


@pytest.mark.parametrize("out_dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 2 ** -8)])
@pytest.mark.parametrize("M,E,eps", [(1, 24, 1e-5), (9, 100, 1e-6), (40, 4100, 1e-3)])
def test_rmsnorm(M, E, eps, out_dtype, tol):
    from fastgguf_b200 import ops
    x = (torch.randn(M, E) * 3).cuda()
    w = (1 + 0.1 * torch.randn(E)).cuda()
    want = P.plain_rmsnorm(x.cpu().double(), w.cpu().double(), eps)
    got = ops.rmsnorm(x, w, eps, out_dtype)
    assert (got.cpu().double() - want).abs().max() <= tol * want.abs().max()
    rows = torch.tensor([M - 1, 0], dtype=torch.int32).cuda()
    picked = ops.rmsnorm(x, w, eps, out_dtype, rows=rows)
    assert torch.equal(picked, got[[M - 1, 0]])


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 2 ** -7)])
@pytest.mark.parametrize("H,KV,hd", [(3, 1, 8), (4, 2, 48), (2, 2, 128)])
def test_rope_append(H, KV, hd, dtype, tol):
    """q rotated in place; k rotated and v copied into the right page, KV head and offset."""
    from types import SimpleNamespace
    from fastgguf_b200 import ops
    from fastgguf_b200.parts import position_tables
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 64}
    cos, sin, _ = position_tables("rope", dict(head_dim=hd, theta=500000.0, scaling=scaling), 400)
    rope = SimpleNamespace(cos=torch.from_numpy(cos).cuda(), sin=torch.from_numpy(sin).cuda())
    cfg = {"rope_theta": 500000.0, "rope_scaling": scaling}
    positions = [0, 1, 63, 64, 200, 399, 5]
    row_seq = [0, 0, 0, 0, 1, 1, 2]
    table = torch.tensor([[3, 7, 0, 0, 0, 0, 0], [2, 9, 4, 8, 1, 5, 6], [10, 0, 0, 0, 0, 0, 0]], dtype=torch.int32)
    M, Q, D = len(positions), H * hd, KV * hd
    qkv = torch.randn(M, Q + 2 * D).to(dtype)
    k_pool = torch.zeros(11, KV, 64, hd, dtype=dtype).cuda()
    v_pool = torch.zeros_like(k_pool)
    dev = qkv.clone().cuda()
    ops.rope_append(dev, torch.tensor(positions, dtype=torch.int32).cuda(), torch.tensor(row_seq, dtype=torch.int32).cuda(),
                    table.cuda(), k_pool, v_pool, rope.cos, rope.sin, H, KV, hd)
    div = P.plain_rope_divisors(cfg, hd)
    src = qkv.double()
    want_q = P.plain_rope(src[:, :Q].reshape(M, H, hd), positions, 500000.0, div).reshape(M, Q)
    want_k = P.plain_rope(src[:, Q:Q + D].reshape(M, KV, hd), positions, 500000.0, div)
    assert (dev[:, :Q].cpu().double() - want_q).abs().max() <= tol * want_q.abs().max()
    written = torch.zeros(11, 64, dtype=torch.bool)
    for m, (pos, s) in enumerate(zip(positions, row_seq)):
        page, off = int(table[s, pos // 64]), pos % 64
        written[page, off] = True
        assert (k_pool[page, :, off].cpu().double() - want_k[m]).abs().max() <= tol * want_k.abs().max()
        assert torch.equal(v_pool[page, :, off].cpu(), qkv[m, Q + D:].reshape(KV, hd))
    untouched = ~written[:, None, :, None]                         # nothing else is written
    assert (k_pool.cpu() * untouched).abs().sum() == 0 and (v_pool.cpu() * untouched).abs().sum() == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 2 ** -7)])
def test_silu_mul(dtype, tol):
    from fastgguf_b200 import ops
    gu = (torch.randn(13, 2 * 37) * 4).to(dtype).cuda()
    g, u = gu.cpu().double()[:, :37], gu.cpu().double()[:, 37:]
    want = P.plain_silu(g) * u
    assert (ops.silu_mul(gu).cpu().double() - want).abs().max() <= tol * want.abs().max()


def test_argmax_takes_the_first_maximum():
    from fastgguf_b200 import ops
    lg = torch.randn(5, 70001).cuda()
    lg[0, 123] = lg[0, 69000] = 50.0
    lg[1, 0] = 60.0
    lg[2, 70000] = 70.0
    want = [P.plain_argmax(r.tolist()) for r in lg.cpu()]
    assert ops.argmax(lg).cpu().tolist() == want and want[:3] == [123, 0, 70000]


def _sampler_state(n, seeds, device="cuda"):
    rng = torch.tensor([s - (1 << 64) if s >= (1 << 63) else s for s in seeds], dtype=torch.int64, device=device)
    return rng, torch.arange(n, dtype=torch.int32, device=device)


@pytest.mark.parametrize("V", [67, 509, 40000])
@pytest.mark.parametrize("opts", [
    dict(temp=0.0, top_k=64, top_p=0.95, repeat_penalty=1.0, repeat_last_n=64),
    dict(temp=0.8, top_k=64, top_p=0.95, repeat_penalty=1.0, repeat_last_n=64),
    dict(temp=1.3, top_k=7, top_p=1.0, repeat_penalty=1.0, repeat_last_n=64),
    dict(temp=0.5, top_k=1000, top_p=0.5, repeat_penalty=1.25, repeat_last_n=8),
    dict(temp=0.0, top_k=0, top_p=1.0, repeat_penalty=1.5, repeat_last_n=5),
])
def test_sampler_matches_plain_token_for_token(V, opts):
    """Same logits, same generator state, same history: the same token, and the same next state."""
    from fastgguf_b200 import ops
    g = torch.Generator().manual_seed(V)
    B, cap = 6, max(1, opts["repeat_last_n"])
    logits = (torch.randn(B, V, generator=g) * 3).float()
    logits[2, 5] = logits[2, 40] = logits[2].max() + 1.0            # a tie at the top
    hists = [[int(t) for t in torch.randint(0, V, (n,), generator=g)] for n in (0, 3, cap, cap, 2, cap)]
    hists[3][-1] = hists[3][0]                                      # a repeated token is penalised once
    seeds = [(0x9E3779B97F4A7C15 * (i + 1)) % 2 ** 64 for i in range(B)]
    stop = [hists[1][0]] if hists[1] else []
    for rounds in range(3):                                         # states and histories carry over
        rng, rows = _sampler_state(B, seeds)
        hist = torch.zeros(B, cap, dtype=torch.int32)
        count = torch.zeros(B, dtype=torch.int32)
        for b, h in enumerate(hists):
            tail = h[-cap:]
            hist[b, :len(tail)] = torch.tensor(tail, dtype=torch.int32)
            count[b] = len(tail)
        dev = logits.clone().cuda()
        got = ops.sample(dev, seq_slot=rows, rng=rng, hist=hist.cuda(), hist_count=count.cuda(),
                         stop_ids=torch.tensor(stop, dtype=torch.int32).cuda() if stop else None, **opts).cpu().tolist()
        for b in range(B):
            tok, state = P.plain_sample(logits[b].numpy(), seeds[b], hists[b][-cap:], stop_ids=tuple(stop), **opts)
            assert got[b] == tok, (rounds, b)
            new_state = rng[b].item() % 2 ** 64
            if opts["temp"] > 0:
                assert new_state == state
            seeds[b] = state
            hists[b].append(tok)


@pytest.mark.parametrize("V,top_k", [(150001, 64), (128256, 100), (70000, 128), (4097, 65)])
def test_two_stage_top_k_at_large_vocabularies(V, top_k):
    """Segment counts that are no power of two, 128 words a segment, and the best entries crowded into one segment."""
    from fastgguf_b200 import ops
    g = torch.Generator().manual_seed(V + top_k)
    B = 3
    logits = (torch.randn(B, V, generator=g) * 2).float()
    logits[1, 5000:5000 + 200] += 30.0                               # every candidate of the row from one segment
    logits[2, V - 1] = logits[2, 0] = logits[2].max() + 2.0          # a tie between the first and the last entry
    seeds = [(0x9E3779B97F4A7C15 * (i + 3)) % 2 ** 64 for i in range(B)]
    opts = dict(temp=0.9, top_k=top_k, top_p=0.97, repeat_penalty=1.0, repeat_last_n=0)
    for rounds in range(2):
        rng, rows = _sampler_state(B, seeds)
        got = ops.sample(logits.clone().cuda(), seq_slot=rows, rng=rng, hist=None, hist_count=None, stop_ids=None, **opts).cpu().tolist()
        for b in range(B):
            tok, state = P.plain_sample(logits[b].numpy(), seeds[b], [], stop_ids=(), **opts)
            assert got[b] == tok, (rounds, b)
            assert rng[b].item() % 2 ** 64 == state
            seeds[b] = state


def test_sampler_without_top_k_follows_the_distribution():
    """top_k = 0 walks the candidates in index order: another token for the same draw, the same law."""
    from fastgguf_b200 import ops
    p = np.array([0.5, 0.3, 0.2, 1e-12])
    logits = torch.tensor(np.log(p), dtype=torch.float32).repeat(4000, 1).cuda()
    seeds = [(0x9E3779B97F4A7C15 * (i + 1)) % 2 ** 64 for i in range(4000)]
    rng, rows = _sampler_state(4000, seeds)
    toks = ops.sample(logits.clone(), temp=1.0, top_k=0, top_p=1.0, repeat_penalty=1.0, repeat_last_n=0,
                      seq_slot=rows, rng=rng, hist=None, hist_count=None, stop_ids=None).cpu().numpy()
    freq = np.bincount(toks, minlength=4) / 4000.0
    assert np.abs(freq[:3] - p[:3]).max() < 0.03 and freq[3] == 0
    toks = ops.sample(logits.clone(), temp=1.0, top_k=0, top_p=0.6, repeat_penalty=1.0, repeat_last_n=0,
                      seq_slot=rows, rng=rng, hist=None, hist_count=None, stop_ids=None).cpu().numpy()
    freq = np.bincount(toks, minlength=4) / 4000.0
    assert np.abs(freq - [0.625, 0.375, 0, 0]).max() < 0.03


def test_sampler_without_top_k_over_a_large_vocabulary():
    """The kernels that split a row over many blocks: the law of the draw, the top-p cut, rows that do not depend on
    their neighbours, and a state that is left clean for the next call."""
    from fastgguf_b200 import ops
    V, n = 20000, 3000
    p = np.array([0.5, 0.3, 0.15, 0.05])
    where = [7, 9000, 13001, V - 1]                                  # in different blocks of the row
    base = torch.full((V,), -40.0)
    for w, q in zip(where, p):
        base[w] = float(np.log(q))
    base[100] = float(np.log(0.5)) - 25.0                            # below max - 20 * temp: never a candidate
    logits = base.repeat(n, 1).cuda()
    seeds = [(0x9E3779B97F4A7C15 * (i + 1)) % 2 ** 64 for i in range(n)]
    rng, rows = _sampler_state(n, seeds)
    kw = dict(repeat_penalty=1.0, repeat_last_n=0, seq_slot=rows, rng=rng, hist=None, hist_count=None, stop_ids=None)
    toks = ops.sample(logits.clone(), temp=1.0, top_k=0, top_p=1.0, **kw).cpu().numpy()
    assert set(np.unique(toks)) <= set(where)
    freq = np.array([(toks == w).mean() for w in where])
    assert np.abs(freq - p).max() < 0.035
    toks = ops.sample(logits.clone(), temp=1.0, top_k=0, top_p=0.6, **kw).cpu().numpy()
    freq = np.array([(toks == w).mean() for w in where])
    assert np.abs(freq - [0.625, 0.375, 0, 0]).max() < 0.035
    # temperature 2: probabilities ~ sqrt(p), and the far entry is a candidate now
    toks = ops.sample(logits.clone(), temp=2.0, top_k=0, top_p=1.0, **kw).cpu().numpy()
    q = np.sqrt(np.append(p, 0.5 * np.exp(-25.0)))
    q /= q.sum()
    freq = np.array([(toks == w).mean() for w in where + [100]])
    assert np.abs(freq - q).max() < 0.035
    # random rows: alone or in a batch, the same generator state gives the same token; the second call starts clean
    g = torch.Generator().manual_seed(5)
    rnd = (torch.randn(6, 50000, generator=g) * 4).float().cuda()
    outs = []
    for rep in range(2):
        rng6, rows6 = _sampler_state(6, seeds[:6])
        outs.append(ops.sample(rnd.clone(), temp=0.8, top_k=0, top_p=0.9, repeat_penalty=1.0, repeat_last_n=0, seq_slot=rows6,
                               rng=rng6, hist=None, hist_count=None, stop_ids=None).cpu().tolist())
    assert outs[0] == outs[1]
    for b in (0, 3, 5):
        rng1, rows1 = _sampler_state(1, [seeds[b]])
        alone = ops.sample(rnd[b:b + 1].clone(), temp=0.8, top_k=0, top_p=0.9, repeat_penalty=1.0, repeat_last_n=0, seq_slot=rows1,
                           rng=rng1, hist=None, hist_count=None, stop_ids=None).cpu().tolist()
        assert alone[0] == outs[0][b]
    # the nucleus of a random row: every drawn token lies in the smallest set of most probable tokens that reaches top_p
    row = rnd[0].double().cpu().numpy() / 0.8
    pr = np.exp(row - row.max()); pr /= pr.sum()
    order = np.argsort(-pr)
    k = int(np.searchsorted(np.cumsum(pr[order]), 0.9)) + 1
    nucleus = set(order[:k + 2].tolist())                            # (entries tied with the last one within a bin are kept too)
    many = rnd[0:1].repeat(2000, 1)
    rngm, rowsm = _sampler_state(2000, seeds[:2000])
    drawn = ops.sample(many, temp=0.8, top_k=0, top_p=0.9, repeat_penalty=1.0, repeat_last_n=0, seq_slot=rowsm, rng=rngm,
                       hist=None, hist_count=None, stop_ids=None).cpu().tolist()
    assert set(drawn) <= nucleus
    assert len(set(drawn)) > k // 3                                   # and it is not stuck on a few of them


def test_decode_advance():
    from fastgguf_b200 import ops
    tokens = torch.tensor([1, 2, 3], dtype=torch.int32).cuda()
    pos = torch.tensor([10, 20, 0], dtype=torch.int32).cuda()
    ops.decode_advance(tokens, pos, torch.tensor([7, 8, 9], dtype=torch.int32).cuda(),
                       torch.tensor([1, 1, 0], dtype=torch.int32).cuda())
    assert tokens.cpu().tolist() == [7, 8, 9] and pos.cpu().tolist() == [11, 21, 0]
