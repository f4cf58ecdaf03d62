"""Generality of the layer parts, shown with toy parts defined HERE and registered without touching
the framework's files: a mixer with fixed-size state of its own (no keys, no values), a schedule
that runs a layer twice (two caches) and an entry that reads another entry's cache.  The toy model
is stepped whole, in pieces and in unequal batches, and compared with a plain computation."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

E, H, KV, HD, F, V = 48, 3, 1, 16, 80, 101


def _register_toy():
    from fastgguf_b200.parts import base

    class RunningMeanMixer(base.Mixer):
        """out_t = W * mean(xn_0 .. xn_t): its state is the running sum and the count of its sequence."""

        def __init__(self, runtime, hidden_size):
            super().__init__(runtime)
            self.hidden_size = hidden_size
            self.w = None

        def tensor_specs(self):
            return {"mix.weight": base.TensorSpec((self.hidden_size, self.hidden_size))}

        def state_request(self):
            return base.StateRequest((self.hidden_size + 1,), torch.float32)

        def load(self, tensors):
            self.w = tensors["mix.weight"].float()

        def forward(self, xn, batch, io, residual):
            cu = batch.host_cu_rows
            slots = batch.slots.long()
            for s in range(batch.n_seq):
                rows = xn[cu[s]:cu[s + 1]].float()
                state = io.state[slots[s]]
                sums = state[:-1] + rows.cumsum(0)
                counts = state[-1] + torch.arange(1, rows.shape[0] + 1, device=xn.device)
                residual[cu[s]:cu[s + 1]] += (sums / counts[:, None]) @ self.w.T
                io.state[slots[s], :-1] = sums[-1]
                io.state[slots[s], -1] = counts[-1]

    base.register_mixer("toy_running_mean", RunningMeanMixer)


def _spec():
    from fastgguf_b200.engine.spec import LayerSpec, ModelSpec, PartSpec, RunSpec
    rope = PartSpec("rope", dict(head_dim=HD, theta=10000.0, scaling=None))
    norm = lambda name: PartSpec("rmsnorm", dict(size=E, eps=1e-5), {"weight": name})
    ffn = lambda p: PartSpec("swiglu", dict(hidden_size=E, d_ff=F), {f"{n}_proj.weight": f"{p}.ffn.{n}" for n in ("gate", "up", "down")})
    attn = PartSpec("gqa_attention", dict(hidden_size=E, n_heads=H, n_kv_heads=KV, head_dim=HD, position=rope),
                    {f"{n}_proj.weight": f"l0.attn.{n}" for n in "qkvo"})
    toy = PartSpec("toy_running_mean", dict(hidden_size=E), {"mix.weight": "l1.mix"})
    layers = [LayerSpec("prenorm", attn, ffn("l0"), norm("l0.n1"), norm("l0.n2")),
              LayerSpec("prenorm", toy, ffn("l1"), norm("l1.n1"), norm("l1.n2"))]
    # attention layer, toy layer, the attention layer AGAIN (its own cache), and once more reading entry 0's cache
    schedule = [RunSpec(0), RunSpec(1), RunSpec(0), RunSpec(0, cache_from=0)]
    return ModelSpec(hidden_size=E, vocab_size=V, max_positions=512,
                     embedding=PartSpec("embedding", dict(vocab_size=V, hidden_size=E), {"weight": "emb"}),
                     layers=layers, schedule=schedule, final_norm=norm("nf"),
                     head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=E), {"weight": "emb"}))


def _plain(W, toks):
    """The toy model on a whole sequence, from the plain implementation's parts."""
    W = {k: v.double() for k, v in W.items()}
    T = len(toks)
    x = P.plain_embedding(W["emb"], toks)
    pos = list(range(T))

    def attention_layer(x, shared_kv=None):
        n1 = P.plain_rmsnorm(x, W["l0.n1"], 1e-5)
        q = P.plain_rope((n1 @ W["l0.attn.q"].T).reshape(T, H, HD), pos, 10000.0, [1.0] * (HD // 2))
        if shared_kv is None:
            k = P.plain_rope((n1 @ W["l0.attn.k"].T).reshape(T, KV, HD), pos, 10000.0, [1.0] * (HD // 2))
            v = (n1 @ W["l0.attn.v"].T).reshape(T, KV, HD)
        else:
            k, v = shared_kv
        h1 = P.plain_attention(q, k, v, 1 / math.sqrt(HD)).reshape(T, H * HD) @ W["l0.attn.o"].T + x
        n2 = P.plain_rmsnorm(h1, W["l0.n2"], 1e-5)
        return P.plain_swiglu(n2, W["l0.ffn.gate"], W["l0.ffn.up"], W["l0.ffn.down"]) + h1, (k, v)

    x, kv0 = attention_layer(x)
    n1 = P.plain_rmsnorm(x, W["l1.n1"], 1e-5)
    means = n1.cumsum(0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
    h1 = means @ W["l1.mix"].T + x
    x = P.plain_swiglu(P.plain_rmsnorm(h1, W["l1.n2"], 1e-5), W["l1.ffn.gate"], W["l1.ffn.up"], W["l1.ffn.down"]) + h1
    x, _ = attention_layer(x)
    x, _ = attention_layer(x, shared_kv=kv0)
    return (P.plain_rmsnorm(x, W["nf"], 1e-5) @ W["emb"].T).numpy()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_toy_mixer_with_state_and_a_schedule_with_repeats(dtype, tol):
    from fastgguf_b200.engine.batch import StepEntry
    from fastgguf_b200.engine.model import DecoderModel
    from fastgguf_b200.parts.base import Runtime
    from fastgguf_b200.weights.loader import MemorySource
    from fastgguf_b200.weights.random_init import random_tensor
    _register_toy()
    model = DecoderModel(_spec(), Runtime(torch.device("cuda"), dtype))
    expected = model.expected_tensors()
    assert "l1.mix" in expected and len(expected) == 17            # the repeated layer's tensors appear once
    W = {n: random_tensor(n, s, 9, torch.bfloat16) * (5 if s.init[0] == "normal" else 1) for n, s in expected.items()}
    model.load_weights(MemorySource(W))
    cache = model.make_cache(max_tokens=512, n_slots=3)
    assert len(cache.groups) == 1 and cache.groups[0].entries == [0, 2]      # entry 3 borrows, entry 1 keeps no keys
    assert list(model.state.tensors) == [1] and model.state.of(1).shape == (3, E + 1)
    Wf = {k: v.float() for k, v in W.items()}
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, V, size=n).tolist() for n in (70, 5, 33)]
    want = [_plain(Wf, s) for s in seqs]

    def err(got, w):
        return float(np.abs(got - w).max() / np.abs(w).max())

    # whole, each alone
    for s, w in zip(seqs, want):
        slot = model.acquire_slot()
        got = model.step([StepEntry(slot, s, list(range(len(s))))]).cpu().numpy()
        model.release_slot(slot)
        assert err(got, w) < tol
    # an unequal batch: prompts (a prefix of each) in one step, then one token each; shorter ones end earlier
    slots = [model.acquire_slot() for _ in seqs]                   # slots used before: their state was zeroed again
    heads = [max(1, len(s) // 2) for s in seqs]
    out = model.step([StepEntry(sl, s[:h], list(range(h))) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
    got = [[r for r in out[sum(heads[:i]):sum(heads[:i + 1])]] for i in range(3)]
    fed = list(heads)
    while any(f < len(s) for f, s in zip(fed, seqs)):
        live = [i for i in range(3) if fed[i] < len(seqs[i])]
        out = model.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live]).cpu().numpy()
        for r, i in zip(out, live):
            got[i].append(r)
            fed[i] += 1
    for g, w in zip(got, want):
        assert err(np.stack(g), w) < tol
    for sl in slots:
        model.release_slot(sl)
    cache.check()


# ------------------------------------------------------------------------------------------------
# another position encoding and a feed-forward with routing, again defined and registered here

def _register_more_toys():
    from fastgguf_b200.parts import base

    class HalfRotary(base.PositionEncoding):
        """Rotates only the first `rot` pairs of a head, with positions scaled by `scale`; the other
        pairs keep their values (cos 1, sin 0).  The attention mixer only needs `cos` and `sin`
        tables [positions, head_dim / 2] after `prepare`."""

        def __init__(self, runtime, head_dim, theta, rot, scale):
            super().__init__(runtime)
            self.head_dim, self.theta, self.rot, self.scale = head_dim, theta, rot, scale
            self.cos = self.sin = None

        def prepare(self, max_positions):
            half = self.head_dim // 2
            j = torch.arange(half, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * j / self.head_dim)
            ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * self.scale * inv[None, :]
            ang[:, self.rot:] = 0.0
            self.cos = torch.cos(ang).float().to(self.runtime.device)
            self.sin = torch.sin(ang).float().to(self.runtime.device)

    class RoutedMLP(base.FeedForward):
        """Two experts, each row goes to the one its router scores higher (router logits in float32)."""

        def __init__(self, runtime, hidden_size, d_ff):
            super().__init__(runtime)
            self.hidden_size, self.d_ff = hidden_size, d_ff

        def tensor_specs(self):
            E, F = self.hidden_size, self.d_ff
            specs = {"router.weight": base.TensorSpec((2, E))}
            for e in range(2):
                specs[f"experts.{e}.up"] = base.TensorSpec((F, E))
                specs[f"experts.{e}.down"] = base.TensorSpec((E, F))
            return specs

        def load(self, tensors):
            self.t = {k: v.float() for k, v in tensors.items()}

        def forward(self, xn, batch, residual):
            x = xn.float()
            pick = (x @ self.t["router.weight"].T).argmax(-1)
            for e in range(2):
                rows = (pick == e).nonzero().squeeze(-1)
                if rows.numel():
                    h = torch.relu(x[rows] @ self.t[f"experts.{e}.up"].T)
                    residual[rows] += h @ self.t[f"experts.{e}.down"].T

    base.register_position_encoding("toy_half_rotary", HalfRotary)
    base.register_feed_forward("toy_routed", RoutedMLP)


def _spec2():
    from fastgguf_b200.engine.spec import LayerSpec, ModelSpec, PartSpec, RunSpec
    pos = PartSpec("toy_half_rotary", dict(head_dim=HD, theta=100.0, rot=5, scale=0.5))
    norm = lambda name: PartSpec("rmsnorm", dict(size=E, eps=1e-6), {"weight": name})
    attn = PartSpec("gqa_attention", dict(hidden_size=E, n_heads=H, n_kv_heads=KV, head_dim=HD, position=pos, window=40),
                    {f"{n}_proj.weight": f"a.{n}" for n in "qkvo"})
    names = {"router.weight": "r.w"}
    for e in range(2):
        names[f"experts.{e}.up"] = f"r.{e}.up"
        names[f"experts.{e}.down"] = f"r.{e}.down"
    routed = PartSpec("toy_routed", dict(hidden_size=E, d_ff=F), names)
    layers = [LayerSpec("prenorm", attn, routed, norm("n1"), norm("n2"))]
    return ModelSpec(hidden_size=E, vocab_size=V, max_positions=512,
                     embedding=PartSpec("embedding", dict(vocab_size=V, hidden_size=E), {"weight": "emb"}),
                     layers=layers, schedule=[RunSpec(0)], final_norm=norm("nf"),
                     head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=E), {"weight": "head"}))


def _plain2(W, toks):
    W = {k: v.double() for k, v in W.items()}
    T = len(toks)
    x = P.plain_embedding(W["emb"], toks)
    n1 = P.plain_rmsnorm(x, W["n1"], 1e-6)
    # half rotary: a divisor of 1 / scale on the rotated pairs, "infinite" on the others (angle 0)
    div = [2.0] * 5 + [1e300] * (HD // 2 - 5)
    pos = list(range(T))
    q = P.plain_rope((n1 @ W["a.q"].T).reshape(T, H, HD), pos, 100.0, div)
    k = P.plain_rope((n1 @ W["a.k"].T).reshape(T, KV, HD), pos, 100.0, div)
    v = (n1 @ W["a.v"].T).reshape(T, KV, HD)
    h1 = P.plain_attention(q, k, v, 1 / math.sqrt(HD), window=40).reshape(T, H * HD) @ W["a.o"].T + x
    n2 = P.plain_rmsnorm(h1, W["n2"], 1e-6)
    pick = (n2 @ W["r.w"].T).argmax(-1)
    out = h1.clone()
    for t in range(T):
        e = int(pick[t])
        out[t] += torch.relu(n2[t] @ W[f"r.{e}.up"].T) @ W[f"r.{e}.down"].T
    return (P.plain_rmsnorm(out, W["nf"], 1e-6) @ W["head"].T).numpy()


def test_toy_position_encoding_and_routed_feed_forward():
    """float32, so that the router's choice is the plain computation's; windowed attention of the framework."""
    from fastgguf_b200.engine.batch import StepEntry
    from fastgguf_b200.engine.model import DecoderModel
    from fastgguf_b200.parts.base import Runtime
    from fastgguf_b200.weights.loader import MemorySource
    from fastgguf_b200.weights.random_init import random_tensor
    _register_more_toys()
    model = DecoderModel(_spec2(), Runtime(torch.device("cuda"), torch.float32))
    W = {n: random_tensor(n, s, 4, torch.float32) * (5 if s.init[0] == "normal" else 1)
         for n, s in model.expected_tensors().items()}
    model.load_weights(MemorySource(W))
    cache = model.make_cache(max_tokens=512, n_slots=2)
    assert cache.groups[0].request.window == 40
    rng = np.random.default_rng(1)
    toks = rng.integers(0, V, size=150).tolist()
    want = _plain2(W, toks)
    slot = model.acquire_slot()
    head = model.step([StepEntry(slot, toks[:100], list(range(100)))]).cpu().numpy()
    tail = [model.step([StepEntry(slot, [t], [0])]).cpu().numpy()[0] for t in toks[100:]]
    got = np.concatenate([head, np.stack(tail)])
    assert float(np.abs(got - want).max() / np.abs(want).max()) < 5e-5
    # the windowed group gave pages back: 150 positions with a window of 40 keep at most two pages
    assert cache.free_pages(0) >= 8 - 2
    model.release_slot(slot)
    cache.check()
