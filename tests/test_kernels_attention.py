"""The attention kernels alone (any-size, tensor-core decode, tensor-core prefill) against a plain
float64 computation over the same paged cache, at sizes other than the engine's.  Pages are handed
out in a shuffled order so that a wrong page lookup shows, and one far key per sequence is scaled
up so that a missed or doubled key changes the result visibly."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

PAGE = 64


@pytest.fixture(params=[0, 3, 7], ids=["one-score-tile", "two-score-tiles", "two-score-tiles-two-softmax-sets"])
def tc_variant(request):
    """Both forms of the tcgen05 prefill kernel at both head sizes, whatever the step's shape would choose."""
    from fastgguf_b200.ops import fast_attention
    fast_attention.prefill_tc_variant(request.param)
    yield request.param
    fast_attention.prefill_tc_variant(-1)


def make_case(lens_before, new, H, KV, hd, dtype, seed, boost=True, ramp=0.0):
    """Sequences with `lens_before[i]` cached tokens that bring `new[i]` more.  Returns everything
    the kernels need plus dense per-sequence K, V (float64) for the plain computation."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    n_seq = len(new)
    total = [a + b for a, b in zip(lens_before, new)]
    n_pages = sum((t + PAGE - 1) // PAGE for t in total) + 1
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()      # page 0 stays unused
    k_pool = torch.zeros(n_pages, KV, PAGE, hd)
    v_pool = torch.zeros(n_pages, KV, PAGE, hd)
    width = max((t + PAGE - 1) // PAGE for t in total)
    table = torch.zeros(n_seq, width, dtype=torch.int32)
    dense = []
    for s in range(n_seq):
        K = torch.randn(total[s], KV, hd, generator=g)
        V = torch.randn(total[s], KV, hd, generator=g)
        if boost and total[s] > 3:
            K[total[s] // 3] *= 4.0                                      # one key that stands out
        if ramp:
            # scores that keep growing with the key's position: the running maximum moves in every block of keys
            K += (torch.arange(total[s]) / 16.0)[:, None, None] * ramp / hd ** 0.5
        K, V = K.to(dtype).float(), V.to(dtype).float()
        dense.append((K.double(), V.double()))
        for p in range((total[s] + PAGE - 1) // PAGE):
            page = perm.pop()
            table[s, p] = page
            n = min(PAGE, total[s] - p * PAGE)
            k_pool[page, :, :n] = K[p * PAGE:p * PAGE + n].transpose(0, 1)
            v_pool[page, :, :n] = V[p * PAGE:p * PAGE + n].transpose(0, 1)
    M = sum(new)
    q = torch.randn(M, H * hd, generator=g)
    if ramp:
        q += hd ** 0.5
    q = q.to(dtype)
    positions = torch.tensor([lens_before[s] + i for s in range(n_seq) for i in range(new[s])], dtype=torch.int32)
    row_seq = torch.tensor([s for s in range(n_seq) for _ in range(new[s])], dtype=torch.int32)
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32)
    return dict(q=q.cuda(), positions=positions.cuda(), row_seq=row_seq.cuda(), cu_rows=cu.cuda(),
                seq_start=torch.tensor(lens_before, dtype=torch.int32).cuda(), table=table.cuda(),
                k_pool=k_pool.to(dtype).cuda(), v_pool=v_pool.to(dtype).cuda(), dense=dense, new=new,
                lens_before=lens_before)


def plain(case, H, KV, hd, scale, window):
    q = case["q"].double().cpu().reshape(-1, H, hd)
    out = torch.zeros_like(q)
    G, row = H // KV, 0
    for s, (K, V) in enumerate(case["dense"]):
        for i in range(case["new"][s]):
            pos = case["lens_before"][s] + i
            lo = max(0, pos - window + 1) if window else 0
            for h in range(H):
                sc = (K[lo:pos + 1, h // G] @ q[row, h]) * scale
                w = torch.softmax(sc, 0)
                out[row, h] = w @ V[lo:pos + 1, h // G]
            row += 1
    return out.reshape(-1, H * hd)


def _err(got, want):
    return (got.double().cpu() - want).abs().max().item() / want.abs().max().item()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("H,KV,hd,window", [(4, 2, 16, 0), (6, 1, 24, 0), (3, 3, 40, 50), (2, 1, 160, 0)])
def test_attention_generic(H, KV, hd, window, dtype, tol):
    from fastgguf_b200 import ops
    case = make_case([0, 70, 1300, 5], [9, 1, 3, 130], H, KV, hd, dtype, 11)
    scale = 1.0 / math.sqrt(hd)
    got = ops.attention_generic(case["q"], case["positions"], case["row_seq"], case["table"], case["k_pool"],
                                case["v_pool"], H, KV, hd, scale, window)
    assert _err(got, plain(case, H, KV, hd, scale, window)) < tol


@pytest.mark.parametrize("n_splits", [None, 1, 2, 3, 8, 16])
@pytest.mark.parametrize("H,KV,hd,window", [(8, 2, 64, 0), (3, 1, 128, 0), (24, 8, 128, 0), (20, 1, 64, 0),
                                            (4, 4, 64, 100), (4, 2, 64, 64), (4, 2, 64, 128), (8, 2, 64, 65),
                                            (6, 2, 128, 128), (3, 1, 128, 65)])
def test_attention_decode(H, KV, hd, window, n_splits):
    from fastgguf_b200.ops import fast_attention
    case = make_case([0, 63, 64, 700, 2047, 129], [1] * 6, H, KV, hd, torch.bfloat16, 12)
    scale = 1.0 / math.sqrt(hd)
    got = fast_attention.attention_decode(case["q"], case["positions"], case["table"], case["k_pool"], case["v_pool"],
                                          H, KV, hd, scale, window, n_splits=n_splits)
    want = plain(case, H, KV, hd, scale, window)
    assert _err(got, want) < 1.5e-2
    if n_splits in (2, 8):        # the same splits through scratch memory and the merge kernel
        got = fast_attention.attention_decode(case["q"], case["positions"], case["table"], case["k_pool"],
                                              case["v_pool"], H, KV, hd, scale, window, n_splits=n_splits,
                                              use_scratch=True)
        assert _err(got, want) < 1.5e-2


@pytest.mark.parametrize("H,KV,hd,window", [(8, 2, 64, 0), (3, 1, 128, 0), (24, 8, 128, 0), (20, 1, 64, 0),
                                            (4, 4, 64, 100), (4, 2, 64, 64), (4, 2, 64, 128), (8, 2, 64, 65),
                                            (6, 2, 128, 128), (3, 1, 128, 65)])
def test_attention_prefill(H, KV, hd, window):
    from fastgguf_b200.ops import fast_attention
    new = [200, 1, 67, 5]
    case = make_case([0, 300, 60, 0], new, H, KV, hd, torch.bfloat16, 13)
    scale = 1.0 / math.sqrt(hd)
    got = fast_attention.attention_prefill(case["q"], case["cu_rows"], case["seq_start"], case["table"], case["k_pool"],
                                           case["v_pool"], len(new), max(new), H, KV, hd, scale, window)
    assert _err(got, plain(case, H, KV, hd, scale, window)) < 1.5e-2


@pytest.mark.parametrize("H,KV,hd,window", [(8, 2, 64, 0), (3, 1, 128, 0), (24, 8, 128, 0), (20, 1, 64, 0),
                                            (4, 4, 64, 100), (4, 2, 64, 64), (4, 2, 64, 128), (8, 2, 64, 65),
                                            (6, 2, 128, 128), (3, 1, 128, 65)])
def test_attention_prefill_tcgen05(H, KV, hd, window, tc_variant):
    from fastgguf_b200.ops import fast_attention
    new = [200, 1, 67, 5, 300]
    case = make_case([0, 300, 60, 0, 129], new, H, KV, hd, torch.bfloat16, 14)
    scale = 1.0 / math.sqrt(hd)
    got = fast_attention.attention_prefill_tc(case["q"], case["cu_rows"], case["seq_start"], case["table"],
                                              case["k_pool"], case["v_pool"], len(new), max(new), H, KV, hd, scale, window)
    assert fast_attention.prefill_tc_error() == 0
    assert _err(got, plain(case, H, KV, hd, scale, window)) < 1.5e-2


@pytest.mark.parametrize("H,KV,hd", [(6, 2, 128), (8, 2, 64)])
def test_attention_prefill_tcgen05_batch_of_long_unequal_prompts(H, KV, hd, tc_variant):
    """Prompts of 64 to 2,048 tokens in one step: tiles of 1 to 32 iterations side by side, rows that finish long
    after the last MMA of their tile and rows that finish before it (every wait on a barrier has to name the right
    phase at either end)."""
    from fastgguf_b200.ops import fast_attention
    new = [1500, 64, 700, 2048, 300, 129]
    case = make_case([0, 0, 64, 0, 1000, 0], new, H, KV, hd, torch.bfloat16, 31)
    scale = 1.0 / math.sqrt(hd)
    got = fast_attention.attention_prefill_tc(case["q"], case["cu_rows"], case["seq_start"], case["table"],
                                              case["k_pool"], case["v_pool"], len(new), max(new), H, KV, hd, scale, 0)
    assert fast_attention.prefill_tc_error() == 0
    assert _err(got, plain(case, H, KV, hd, scale, 0)) < 1.5e-2


@pytest.mark.parametrize("n_splits", [None, 1, 4, 8])
@pytest.mark.parametrize("H,KV,hd,window", [(8, 2, 64, 0), (6, 2, 128, 0), (20, 1, 64, 0), (4, 4, 64, 100),
                                            (4, 2, 64, 64), (4, 2, 64, 128), (6, 2, 128, 65), (6, 2, 128, 128)])
def test_attention_decode_fused_with_rope_and_append(H, KV, hd, window, n_splits):
    """One kernel for RoPE, cache append and attention of a decode step, against the separate kernels."""
    from fastgguf_b200 import ops
    from fastgguf_b200.ops import fast_attention
    lens = [0, 63, 64, 700, 2047, 129]
    case = make_case(lens, [1] * 6, H, KV, hd, torch.bfloat16, 15)
    g = torch.Generator().manual_seed(16)
    qkv = torch.randn(6, (H + 2 * KV) * hd, generator=g).bfloat16().cuda()
    ang = torch.arange(2100, dtype=torch.float64)[:, None] * torch.pow(torch.tensor(10000.0, dtype=torch.float64),
                                                                       -2.0 * torch.arange(hd // 2) / hd)
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    scale = 1.0 / math.sqrt(hd)
    row_seq = torch.arange(6, dtype=torch.int32).cuda()
    # separate kernels on copies of the cache
    k1, v1, q1 = case["k_pool"].clone(), case["v_pool"].clone(), qkv.clone()
    ops.rope_append(q1, case["positions"], row_seq, case["table"], k1, v1, cos, sin, H, KV, hd)
    want = fast_attention.attention_decode(q1, case["positions"], case["table"], k1, v1, H, KV, hd, scale, window,
                                           n_splits=n_splits)
    k2, v2 = case["k_pool"].clone(), case["v_pool"].clone()
    got = fast_attention.attention_decode_fused(qkv, case["positions"], case["table"], k2, v2, cos, sin, H, KV, hd,
                                                scale, window, n_splits=n_splits)
    assert (got.float() - want.float()).abs().max() <= 2e-2 * want.float().abs().max()
    assert torch.equal(k2, k1) and torch.equal(v2, v1)          # the cache received the same rows


@pytest.mark.parametrize("H,KV,hd", [(8, 2, 64), (4, 1, 128)])
def test_attention_prefill_tcgen05_growing_maximum(H, KV, hd):
    """Scores that grow by tens of binary orders every 128 keys: every iteration moves the running base, and
    the rows of the output accumulated so far are rescaled in tensor memory."""
    from fastgguf_b200.ops import fast_attention
    scale = 1.0 / math.sqrt(hd)
    case = make_case([0, 300], [600, 200], H, KV, hd, torch.bfloat16, 21, boost=False, ramp=2.0)
    got = fast_attention.attention_prefill_tc(case["q"], case["cu_rows"], case["seq_start"], case["table"], case["k_pool"],
                                              case["v_pool"], 2, 600, H, KV, hd, scale, 0)
    assert fast_attention.prefill_tc_error() == 0
    want = plain(case, H, KV, hd, scale, 0)
    assert (got.double().cpu() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
