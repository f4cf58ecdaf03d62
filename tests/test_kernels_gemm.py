"""The contraction kernels alone, against float64 matrix products of the same operands, at sizes
other than any model's (odd row counts, feature counts that are no multiple of the tile, a
reduction length that is no multiple of the K-block)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(M, N, K, dtype, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = (torch.randn(M, K, generator=g) * 0.5).to(dtype).cuda()
    w = (torch.randn(N, K, generator=g) * 0.5).to(dtype).cuda()
    return a, w


def _check(got, a, w, want, out_is_bf16):
    bound = (a.double().abs() @ w.double().abs().T).max().item()
    err = (got.double() - want).abs().max().item()
    tol = 2e-6 * bound + (want.abs().max().item() * 2 ** -8 if out_is_bf16 else 0.0)
    assert err <= tol, (err, tol)


@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 200, 72), (70, 130, 257), (129, 65, 64),
                                   (16, 333, 1100), (9, 1000, 4096), (2, 31, 516),        # few rows: the weight-streaming kernel
                                   (300, 260, 1000), (65, 128, 36), (200, 129, 130)])    # many rows: 128 x 128 tiles
def test_gemm_generic(M, N, K, adt, wdt):
    from fastgguf_b200 import ops
    a, _ = _operands(M, N, K, adt, 1)
    _, w = _operands(M, N, K, wdt, 1)
    want = a.double() @ w.double().T
    got = ops.gemm_generic(a, w, out_dtype=torch.float32)
    _check(got, a, w, want, False)
    res = torch.randn(M, N, device="cuda")
    acc = res.clone()
    ops.gemm_generic(a, w, out=acc, accumulate=True)
    _check(acc, a, w, want + res.double(), False)
    if adt == torch.bfloat16:
        _check(ops.gemm_generic(a, w), a, w, want, True)
    # a row's result does not depend on the other rows of the step: alone, it gives the same bits
    if M > 1:
        alone = ops.gemm_generic(a[M - 1:M].contiguous(), w, out_dtype=torch.float32)
        if (M <= 16) == (1 <= 16):                       # the same kernel serves both row counts
            assert torch.equal(alone[0], got[M - 1])
        else:
            assert (alone[0] - got[M - 1]).abs().max() <= 1e-5 * got.abs().max()


@pytest.mark.parametrize("M", [1, 5, 16, 33, 64, 100, 300, 700])
@pytest.mark.parametrize("N,K", [(200, 72), (384, 2048), (1000, 520)])
def test_gemm_tc_epilogues(M, N, K):
    from fastgguf_b200.ops import fast_gemm
    a, w = _operands(M, N, K, torch.bfloat16, 2)
    want = a.double() @ w.double().T
    got = fast_gemm.gemm_tc(a, w, out_dtype=torch.float32)
    assert got is not None
    _check(got, a, w, want, False)
    _check(fast_gemm.gemm_tc(a, w), a, w, want, True)
    res = torch.randn(M, N, device="cuda")
    acc = res.clone()
    fast_gemm.gemm_tc(a, w, out=acc, accumulate=True)
    _check(acc, a, w, want + res.double(), False)
    assert fast_gemm.pipeline_error() == 0


@pytest.mark.parametrize("splits", [2, 4, 8])
@pytest.mark.parametrize("M,N,K", [(1, 256, 2048), (8, 200, 1096), (64, 384, 8192)])
def test_gemm_tc_split_k(M, N, K, splits):
    from fastgguf_b200.ops import fast_gemm
    a, w = _operands(M, N, K, torch.bfloat16, 3)
    want = a.double() @ w.double().T
    for _ in range(2):
        got = fast_gemm.gemm_tc(a, w, out_dtype=torch.float32, force_splits=splits)
        _check(got, a, w, want, False)
    res = torch.randn(M, N, device="cuda")
    acc = res.clone()
    fast_gemm.gemm_tc(a, w, out=acc, accumulate=True, force_splits=splits)
    _check(acc, a, w, want + res.double(), False)
    assert fast_gemm.pipeline_error() == 0


@pytest.mark.parametrize("M", [1, 9, 64, 130, 513])
@pytest.mark.parametrize("F,K", [(192, 64), (320, 72), (640, 2048)])
def test_gemm_tc_silu(M, F, K):
    from fastgguf_b200.ops import fast_gemm
    a, w = _operands(M, 2 * F, K, torch.bfloat16, 4)
    g = a.double() @ w[:F].double().T
    u = a.double() @ w[F:].double().T
    want = g / (1 + torch.exp(-g)) * u
    got = fast_gemm.gemm_tc(a, fast_gemm.interleave_gate_up(w[:F], w[F:]), silu=True)
    assert got is not None and got.dtype == torch.bfloat16
    bound = (a.double().abs() @ w.double().abs().T).max().item()
    err = (got.double() - want).abs().max().item()
    assert err <= want.abs().max().item() * 2 ** -8 + 1e-5 * bound * bound
    assert fast_gemm.pipeline_error() == 0


@pytest.mark.parametrize("splits", [2, 4, 8])
@pytest.mark.parametrize("M,F,K", [(1, 192, 2048), (9, 320, 1096), (64, 640, 2048), (40, 64, 4096)])
def test_gemm_tc_silu_split_k(M, F, K, splits):
    """Gate and up partial sums of a cluster's CTAs meet in the owner of the token column before the activation."""
    from fastgguf_b200.ops import fast_gemm
    a, w = _operands(M, 2 * F, K, torch.bfloat16, 14)
    g = a.double() @ w[:F].double().T
    u = a.double() @ w[F:].double().T
    want = g / (1 + torch.exp(-g)) * u
    got = fast_gemm.gemm_tc(a, fast_gemm.interleave_gate_up(w[:F], w[F:]), silu=True, force_splits=splits)
    bound = (a.double().abs() @ w.double().abs().T).max().item()
    err = (got.double() - want).abs().max().item()
    assert err <= want.abs().max().item() * 2 ** -8 + 1e-5 * bound * bound
    assert fast_gemm.pipeline_error() == 0


def test_gemm_tc_refuses_unaligned():
    from fastgguf_b200.ops import fast_gemm
    a, w = _operands(4, 32, 36, torch.bfloat16, 5)      # K % 8 != 0: TMA cannot describe the rows
    assert fast_gemm.gemm_tc(a, w) is None
    assert fast_gemm.plan_for_weight(w) is None


@pytest.mark.parametrize("M,N,K", [(513, 3072, 256), (700, 3000, 136), (300, 1152, 2048), (129, 2048, 512)])
def test_gemm_tc_prefill_tile_widths_and_started_norm(M, N, K):
    """Prefill shapes that pick 192-wide tiles (3072, 3000 and 1152 features), whole and ragged, and 256-wide ones;
    plain, residual add through the shared-memory tiles (N % 32 == 0) and row-wise (3000), with the next norm started."""
    from fastgguf_b200.ops import fast_gemm
    a, w = _operands(M, N, K, torch.bfloat16, 6)
    want = a.double() @ w.double().T
    _check(fast_gemm.gemm_tc(a, w, out_dtype=torch.float32), a, w, want, False)
    _check(fast_gemm.gemm_tc(a, w), a, w, want, True)
    res = torch.randn(M, N, device="cuda")
    nw = (1 + 0.1 * torch.randn(N, device="cuda")).float()
    acc = res.clone()
    out, started = fast_gemm.gemm_tc(a, w, out=acc, accumulate=True, emit_norm_weight=nw, emit_eps=1e-5)
    x = want + res.double()
    _check(acc, a, w, x, False)
    assert (started.xw.double() - x * nw.double()).abs().max().item() <= 2 ** -7 * (x * nw.double()).abs().max().item()
    ss = started.ss[:started.tiles].double().sum(0)
    assert ((ss - (x * x).sum(1)).abs() / (x * x).sum(1)).max().item() < 1e-4
    assert fast_gemm.pipeline_error() == 0


@pytest.mark.parametrize("width", [-2, -4])
@pytest.mark.parametrize("M,N,K", [(512, 512, 256), (300, 384, 2048), (700, 1000, 520), (129, 256, 72), (2048, 2048, 512), (513, 3072, 264)])
def test_gemm_tc_prefill_pair_of_ctas(M, N, K, width):
    """The kernel that puts a pair of CTAs on a 256 x 256 tile (width -2) or a 256 x 192 tile (-4) (forced here; the
    engine picks it for large shapes): whole and ragged tiles in every direction, every epilogue, the next norm started."""
    from fastgguf_b200.ops import fast_gemm
    a, w = _operands(M, N, K, torch.bfloat16, 8)
    want = a.double() @ w.double().T
    _check(fast_gemm.gemm_tc(a, w, out_dtype=torch.float32, force_splits=width), a, w, want, False)
    _check(fast_gemm.gemm_tc(a, w, force_splits=width), a, w, want, True)
    res = torch.randn(M, N, device="cuda")
    nw = (1 + 0.1 * torch.randn(N, device="cuda")).float()
    acc = res.clone()
    out, started = fast_gemm.gemm_tc(a, w, out=acc, accumulate=True, emit_norm_weight=nw, emit_eps=1e-5, force_splits=width)
    x = want + res.double()
    _check(acc, a, w, x, False)
    assert (started.xw.double() - x * nw.double()).abs().max().item() <= 2 ** -7 * (x * nw.double()).abs().max().item()
    ss = started.ss[:started.tiles].double().sum(0)
    assert ((ss - (x * x).sum(1)).abs() / (x * x).sum(1)).max().item() < 1e-4
    if N % 128 == 0 and width == -2:
        F = N // 2
        gate, up = w[:F], w[F:]
        got = fast_gemm.gemm_tc(a, fast_gemm.interleave_gate_up(gate, up), silu=True, force_splits=-2)
        g, u = a.double() @ gate.double().T, a.double() @ up.double().T
        ref = g / (1 + torch.exp(-g)) * u
        bound = (a.double().abs() @ w.double().abs().T).max().item()
        assert (got.double() - ref).abs().max().item() <= ref.abs().max().item() * 2 ** -8 + 1e-5 * bound * bound
    assert fast_gemm.pipeline_error() == 0


@pytest.mark.parametrize("M,N,K", [(200, 2048, 8192), (256, 512, 4096), (384, 1000, 2048), (130, 264, 4096)])
def test_gemm_tc_prefill_split_along_k(M, N, K):
    """A few hundred rows through a projection of few output tiles: partial products over slices of K on all SMs and a
    second kernel that adds them in order and applies the epilogue - plain, bfloat16, residual add with the next norm
    started, and with a norm on the input side whose 1/rms that kernel applies (its row sums in 5 and in 40 parts)."""
    from fastgguf_b200.ops import fast_gemm
    for epi in (fast_gemm.EPI_BF16, fast_gemm.EPI_F32, fast_gemm.EPI_ADD_F32):
        assert fast_gemm.workspace_bytes(M, N, K, epi) > 0               # the shapes are ones that the split takes
    assert fast_gemm.workspace_bytes(64, N, K, fast_gemm.EPI_F32) == 0   # the decode kernel's range
    assert fast_gemm.workspace_bytes(4096, 4096, K, fast_gemm.EPI_F32) == 0      # enough tiles
    a, w = _operands(M, N, K, torch.bfloat16, 9)
    want = a.double() @ w.double().T
    got = fast_gemm.gemm_tc(a, w, out_dtype=torch.float32)
    _check(got, a, w, want, False)
    whole = fast_gemm.gemm_tc(a, w, out_dtype=torch.float32, split_k=False)
    assert (got - whole).abs().max().item() <= 2e-6 * (a.double().abs() @ w.double().abs().T).max().item()
    _check(fast_gemm.gemm_tc(a, w), a, w, want, True)
    res = torch.randn(M, N, device="cuda")
    nw = (1 + 0.1 * torch.randn(N, device="cuda")).float()
    acc = res.clone()
    out, started = fast_gemm.gemm_tc(a, w, out=acc, accumulate=True, emit_norm_weight=nw, emit_eps=1e-5)
    x = want + res.double()
    _check(acc, a, w, x, False)
    assert started.tiles == (N + 127) // 128
    assert (started.xw.double() - x * nw.double()).abs().max().item() <= 2 ** -7 * (x * nw.double()).abs().max().item()
    ss = started.ss[:started.tiles].double().sum(0)
    assert ((ss - (x * x).sum(1)).abs() / (x * x).sum(1)).max().item() < 1e-4
    # a norm on the input side: rows x (float32) arrive as bf16(x * weight) with the sums of squares of x in parts
    g = torch.Generator(device="cpu").manual_seed(10)
    xin = (torch.randn(M, K, generator=g) * torch.linspace(0.2, 3.0, M)[:, None]).cuda()
    wn = (1 + 0.1 * torch.randn(K, generator=g)).cuda()
    xw = (xin * wn).to(torch.bfloat16)
    for parts in (5, 40):
        edges = torch.linspace(0, K, parts + 1).long().tolist()
        ss_in = torch.stack([(xin[:, lo:hi].double() ** 2).sum(1).float() for lo, hi in zip(edges[:-1], edges[1:])])
        d = fast_gemm.DeferredNorm(xw, ss_in.contiguous(), parts, K, 1e-5, xin, wn)
        inv = 1.0 / torch.sqrt((xin.double() ** 2).mean(1) + 1e-5)
        want_n = (xw.double() * inv[:, None]) @ w.double().T
        got_n = fast_gemm.gemm_tc(xw, w, out_dtype=torch.float32, deferred=d)
        bound = ((xw.double().abs() * inv[:, None]) @ w.double().abs().T).max().item()
        assert (got_n.double() - want_n).abs().max().item() <= 4e-6 * bound
    assert fast_gemm.pipeline_error() == 0
