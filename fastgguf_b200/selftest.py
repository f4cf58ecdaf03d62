"""``python -m fastgguf_b200 selftest``: every kernel against a plain computation of the same
operation, on random data with sane scales, one line per check.

Role of the reference's ``fastgguf selftest`` (fastgguf.c:5478-6109): "fast kernel vs an
independent plain reference", relative error measured against the right magnitude, a final
``ALL TESTS PASSED`` / ``N TESTS FAILED`` line and exit code 0 / 1 (:6107-6108).  The plain side
here is float64 tensor arithmetic written out below; nothing of it is used outside this file.
"""
from __future__ import annotations

import math

import torch


class _Run:
    def __init__(self):
        self.failed = 0

    def check(self, name: str, err: float, tol: float) -> None:
        ok = err <= tol
        self.failed += 0 if ok else 1
        print(f"{'ok  ' if ok else 'FAIL'} {name:<58} err={err:.3e} (tol {tol:.1e})")


def _rel(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double().cpu() - want.double().cpu()).abs().max() / max(float(want.abs().max()), 1e-30))


def _paged(lens, KV, hd, dtype, g):
    """Random dense K, V per sequence and the same data in shuffled pages of 64."""
    n_pages = sum((t + 63) // 64 for t in lens) + 1
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    kp = torch.zeros(n_pages, KV, 64, hd)
    vp = torch.zeros(n_pages, KV, 64, hd)
    table = torch.zeros(len(lens), max((t + 63) // 64 for t in lens), dtype=torch.int32)
    dense = []
    for s, t in enumerate(lens):
        K = torch.randn(t, KV, hd, generator=g).to(dtype).float()
        V = torch.randn(t, KV, hd, generator=g).to(dtype).float()
        dense.append((K.double(), V.double()))
        for p in range((t + 63) // 64):
            page = perm.pop()
            table[s, p] = page
            n = min(64, t - p * 64)
            kp[page, :, :n] = K[p * 64:p * 64 + n].transpose(0, 1)
            vp[page, :, :n] = V[p * 64:p * 64 + n].transpose(0, 1)
    return dense, kp.to(dtype).cuda(), vp.to(dtype).cuda(), table.cuda()


def _attn_plain(q, dense, before, new, H, KV, hd, scale):
    q = q.double().cpu().reshape(-1, H, hd)
    out = torch.zeros_like(q)
    row = 0
    for s, (K, V) in enumerate(dense):
        for i in range(new[s]):
            pos = before[s] + i
            for h in range(H):
                w = torch.softmax((K[:pos + 1, h // (H // KV)] @ q[row, h]) * scale, 0)
                out[row, h] = w @ V[:pos + 1, h // (H // KV)]
            row += 1
    return out.reshape(-1, H * hd)


def run_selftest(quick: bool = False) -> int:
    if not torch.cuda.is_available():
        print("selftest needs a CUDA device (sm_100a); none is visible")
        return 1
    from . import ops
    from .ops import fast_attention, fast_gemm
    r = _Run()
    g = torch.Generator().manual_seed(42)
    dev = "cuda"

    # ---- contractions
    for (M, N, K) in [(3, 200, 72), (70, 130, 257)]:
        a, w = torch.randn(M, K, generator=g) * 0.5, torch.randn(N, K, generator=g) * 0.5
        want = a.double() @ w.double().T
        bound = float((a.double().abs() @ w.double().abs().T).max())
        got = ops.gemm_generic(a.to(dev), w.to(dev))
        r.check(f"gemm_generic f32 {M}x{N}x{K}", float((got.double().cpu() - want).abs().max()) / bound, 2e-6)
    shapes = [(1, 256, 2048), (8, 200, 1096), (64, 384, 2048), (300, 1000, 520)] + ([] if quick else [(2048, 2048, 2048)])
    for (M, N, K) in shapes:
        a = (torch.randn(M, K, generator=g) * 0.5).bfloat16().to(dev)
        w = (torch.randn(N, K, generator=g) * 0.5).bfloat16().to(dev)
        want = a.double() @ w.double().T
        bound = float((a.double().abs() @ w.double().abs().T).max())
        got = fast_gemm.gemm_tc(a, w, out_dtype=torch.float32)
        r.check(f"gemm_tc (tcgen05) f32 out {M}x{N}x{K}", float((got.double() - want).abs().max()) / bound, 2e-6)
        res = torch.randn(M, N, generator=g).to(dev)
        acc = res.clone()
        fast_gemm.gemm_tc(a, w, out=acc, accumulate=True)
        r.check(f"gemm_tc residual add {M}x{N}x{K}", float((acc.double() - want - res.double()).abs().max()) / bound, 2e-6)
    for (M, F, K) in [(5, 192, 72), (200, 640, 512)]:
        a = (torch.randn(M, K, generator=g) * 0.5).bfloat16().to(dev)
        w = (torch.randn(2 * F, K, generator=g) * 0.5).bfloat16().to(dev)
        gg, uu = a.double() @ w[:F].double().T, a.double() @ w[F:].double().T
        want = gg / (1 + torch.exp(-gg)) * uu
        got = fast_gemm.gemm_tc(a, fast_gemm.interleave_gate_up(w[:F], w[F:]), silu=True)
        r.check(f"gemm_tc silu(gate)*up {M}x{F}x{K}", _rel(got, want), 2 ** -7)
    # an RMSNorm started by the contraction that writes the residual stream and finished by the one that reads it
    M, E, N = 8, 512, 384
    x0, a_in = torch.randn(M, E, generator=g).to(dev), (torch.randn(M, E, generator=g) * 0.5).bfloat16().to(dev)
    w1, w2 = (torch.randn(E, E, generator=g) / 16).bfloat16().to(dev), (torch.randn(N, E, generator=g) / 16).bfloat16().to(dev)
    nw = (1 + 0.1 * torch.randn(E, generator=g)).to(dev)
    x = x0.clone()
    _, started = fast_gemm.gemm_tc(a_in, w1, out=x, accumulate=True, emit_norm_weight=nw, emit_eps=1e-5)
    got = fast_gemm.gemm_tc(started.xw, w2, deferred=started, out_dtype=torch.float32)
    xd = x0.double() + a_in.double() @ w1.double().T
    want = (xd / torch.sqrt((xd * xd).mean(1, keepdim=True) + 1e-5) * nw.double()) @ w2.double().T
    r.check("gemm_tc deferred RMSNorm (started in one epilogue, finished in the next)", _rel(got, want), 2 ** -7)
    r.check("gemm_tc pipeline error flag", float(fast_gemm.pipeline_error()), 0.0)

    # ---- row-wise kernels
    x = (torch.randn(9, 300, generator=g) * 3).to(dev)
    w = (1 + 0.1 * torch.randn(300, generator=g)).to(dev)
    want = x.double() * (1.0 / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-5)) * w.double()
    r.check("rmsnorm f32", _rel(ops.rmsnorm(x, w, 1e-5, torch.float32), want), 2e-6)
    r.check("rmsnorm bf16 out", _rel(ops.rmsnorm(x, w, 1e-5, torch.bfloat16), want), 2 ** -8)
    gu = (torch.randn(13, 74, generator=g) * 4).to(dev)
    want = gu[:, :37].double() / (1 + torch.exp(-gu[:, :37].double())) * gu[:, 37:].double()
    r.check("silu_mul f32", _rel(ops.silu_mul(gu), want), 2e-6)
    table = torch.randn(50, 24, generator=g).bfloat16().to(dev)
    toks = torch.randint(0, 50, (7,), generator=g, dtype=torch.int32).to(dev)
    r.check("embed_gather bf16", _rel(ops.embed_gather(table, toks), table[toks.long()].float()), 0.0)
    # rope + append: rotation by table, placement by page table
    H, KV, hd = 4, 2, 48
    pos = torch.tensor([0, 63, 64, 200], dtype=torch.int32)
    ang = pos.double()[:, None] * torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(hd // 2) / hd)
    max_pos = 256
    full = torch.arange(max_pos).double()[:, None] * torch.pow(torch.tensor(10000.0, dtype=torch.float64),
                                                               -2.0 * torch.arange(hd // 2) / hd)
    qkv = torch.randn(4, (H + 2 * KV) * hd, generator=g)
    kp = torch.zeros(6, KV, 64, hd, device=dev)
    vp = torch.zeros_like(kp)
    tbl = torch.tensor([[1, 2, 3, 4]], dtype=torch.int32).to(dev)
    d = qkv.clone().to(dev)
    ops.rope_append(d, pos.to(dev), torch.zeros(4, dtype=torch.int32, device=dev), tbl, kp, vp,
                    torch.cos(full).float().to(dev), torch.sin(full).float().to(dev), H, KV, hd)
    qh = qkv[:, :H * hd].double().reshape(4, H, hd)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    want = torch.cat([qh[..., :hd // 2] * c - qh[..., hd // 2:] * s, qh[..., :hd // 2] * s + qh[..., hd // 2:] * c], -1)
    r.check("rope (q rotated in place)", _rel(d[:, :H * hd], want.reshape(4, -1)), 2e-6)
    r.check("cache append (v at page 4, offset 8)", _rel(vp[4, :, 8], qkv[3, (H + KV) * hd:].reshape(KV, hd)), 0.0)

    # ---- attention over the paged cache
    for (H, KV, hd, dt, tol) in [(4, 2, 16, torch.float32, 1e-5), (6, 1, 24, torch.bfloat16, 1.5e-2)]:
        before, new = [0, 70, 300], [9, 1, 3]
        lens = [b + n for b, n in zip(before, new)]
        dense, kp, vp, tbl = _paged(lens, KV, hd, dt, g)
        q = torch.randn(sum(new), H * hd, generator=g).to(dt).to(dev)
        positions = torch.tensor([b + i for b, n in zip(before, new) for i in range(n)], dtype=torch.int32).to(dev)
        row_seq = torch.tensor([s for s, n in enumerate(new) for _ in range(n)], dtype=torch.int32).to(dev)
        got = ops.attention_generic(q, positions, row_seq, tbl, kp, vp, H, KV, hd, 1 / math.sqrt(hd))
        r.check(f"attention_generic {dt} heads {H}/{KV} size {hd}",
                _rel(got, _attn_plain(q, dense, before, new, H, KV, hd, 1 / math.sqrt(hd))), tol)
    for (H, KV, hd) in [(8, 2, 64), (6, 2, 128)]:
        before = [0, 63, 700, 2047 if not quick else 500]
        dense, kp, vp, tbl = _paged([b + 1 for b in before], KV, hd, torch.bfloat16, g)
        q = torch.randn(4, H * hd, generator=g).bfloat16().to(dev)
        positions = torch.tensor(before, dtype=torch.int32).to(dev)
        want = _attn_plain(q, dense, before, [1] * 4, H, KV, hd, 1 / math.sqrt(hd))
        for splits in (1, 4, 5):
            got = fast_attention.attention_decode(q, positions, tbl, kp, vp, H, KV, hd, 1 / math.sqrt(hd), n_splits=splits)
            r.check(f"attention_decode heads {H}/{KV} size {hd} splits {splits}", _rel(got, want), 1.5e-2)
        before, new = [0, 300, 60], [200, 1, 67]
        dense, kp, vp, tbl = _paged([b + n for b, n in zip(before, new)], KV, hd, torch.bfloat16, g)
        q = torch.randn(sum(new), H * hd, generator=g).bfloat16().to(dev)
        cu = torch.tensor([0, 200, 201, 268], dtype=torch.int32).to(dev)
        got = fast_attention.attention_prefill(q, cu, torch.tensor(before, dtype=torch.int32).to(dev), tbl, kp, vp, 3, 200,
                                               H, KV, hd, 1 / math.sqrt(hd))
        want = _attn_plain(q, dense, before, new, H, KV, hd, 1 / math.sqrt(hd))
        r.check(f"attention_prefill heads {H}/{KV} size {hd}", _rel(got, want), 1.5e-2)
        got = fast_attention.attention_prefill_tc(q, cu, torch.tensor(before, dtype=torch.int32).to(dev), tbl, kp, vp, 3, 200,
                                                  H, KV, hd, 1 / math.sqrt(hd))
        r.check(f"attention_prefill_tc (tcgen05) heads {H}/{KV} size {hd}", _rel(got, want), 1.5e-2)
        r.check("attention_prefill_tc pipeline error flag", float(fast_attention.prefill_tc_error()), 0.0)
        # the decode step's kernel: rotary encoding of q and the new k, cache append and attention in one
        before = [0, 63, 64, 700]
        dense, kp, vp, tbl = _paged([b + 1 for b in before], KV, hd, torch.bfloat16, g)
        qkv = torch.randn(4, (H + 2 * KV) * hd, generator=g).bfloat16().to(dev)
        positions = torch.tensor(before, dtype=torch.int32).to(dev)
        ang = torch.arange(1024).double()[:, None] * torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(hd // 2) / hd)
        cos, sin = torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)
        k1, v1, q1 = kp.clone(), vp.clone(), qkv.clone()
        ops.rope_append(q1, positions, torch.arange(4, dtype=torch.int32, device=dev), tbl, k1, v1, cos, sin, H, KV, hd)
        want = fast_attention.attention_decode(q1, positions, tbl, k1, v1, H, KV, hd, 1 / math.sqrt(hd), n_splits=1)
        got = fast_attention.attention_decode_fused(qkv, positions, tbl, kp, vp, cos, sin, H, KV, hd, 1 / math.sqrt(hd), n_splits=4)
        r.check(f"attention_decode_fused vs rope + append + attention, heads {H}/{KV} size {hd}", _rel(got, want), 1.5e-2)
        r.check("attention_decode_fused wrote the same cache rows", float((kp != k1).sum() + (vp != v1).sum()), 0.0)

    # ---- sampler: greedy is the first maximum; draws follow the probabilities (fastgguf.c:5426-5444)
    lg = torch.randn(3, 70001, generator=g).to(dev)
    lg[0, 123] = lg[0, 69000] = 50.0
    got = ops.argmax(lg).cpu().tolist()
    r.check("argmax takes the first maximum", float(got[0] != 123 or got[1:] != lg[1:].argmax(-1).cpu().tolist()), 0.0)
    n = 4000
    p = torch.tensor([0.5, 0.3, 0.2])
    logits = torch.log(p).repeat(n, 1).to(dev)
    rng = (torch.arange(1, n + 1, dtype=torch.int64) * 0x9E3779B97F4A7C1).to(dev)
    rows = torch.arange(n, dtype=torch.int32, device=dev)
    for name, kw, want in (("temperature 1, top-k 3", dict(top_k=3, top_p=1.0), [0.5, 0.3, 0.2]),
                           ("top-p 0.6", dict(top_k=3, top_p=0.6), [0.625, 0.375, 0.0])):
        toks = ops.sample(logits.clone(), temp=1.0, repeat_penalty=1.0, repeat_last_n=0, seq_slot=rows, rng=rng, hist=None,
                          hist_count=None, stop_ids=None, **kw).cpu()
        freq = torch.bincount(toks.long(), minlength=3).double() / n
        r.check(f"sampler frequencies, {name}", float((freq - torch.tensor(want).double()).abs().max()), 0.03)
    toks = ops.sample(logits.clone(), temp=0.0, top_k=64, top_p=0.95, repeat_penalty=1.0, repeat_last_n=0, seq_slot=rows,
                      rng=rng, hist=None, hist_count=None, stop_ids=None).cpu()
    r.check("sampler temp 0 is argmax", float((toks != 0).sum()), 0.0)

    torch.cuda.synchronize()
    print("ALL TESTS PASSED" if r.failed == 0 else f"{r.failed} TESTS FAILED")
    return 0 if r.failed == 0 else 1
