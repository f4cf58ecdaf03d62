"""A plain, slow implementation of the Llama decoder, written from the formulas of the reference
engine (fastgguf.c of lawnak/FastGGUF; every function cites file:line).  Whole sequences, no
cache, one function for each part, CPU only.  It shares no code with ``fastgguf_b200``: it
parses config.json and reads the safetensors file with its own few lines.

Compared once with the reference's own C code on a tiny random model: see
``tests/golden/make_golden.py`` and ``tests/test_plain.py``.

Precision: ``dtype=torch.float64`` (default) makes it an oracle whose own rounding is
negligible; ``torch.float32`` follows the reference's mix (float everywhere, double for the
norm's sum of squares and the rotary angles).
"""
import json
import math
import os
import struct

import numpy as np
import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32,
              "I64": torch.int64}


# ------------------------------------------------------------------------------ reading
def read_safetensors(path):
    """{tensor name: CPU tensor in its stored dtype} of one safetensors file."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        data = f.read()
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        if e == b:
            tensors[name] = torch.empty(info["shape"], dtype=_ST_DTYPES[info["dtype"]])
            continue
        tensors[name] = torch.frombuffer(bytearray(data[b:e]), dtype=_ST_DTYPES[info["dtype"]]).reshape(info["shape"])
    return tensors


def write_safetensors(path, tensors):
    """The tests' own writer (for files with faults the engine's reader must name)."""
    names = {v: k for k, v in _ST_DTYPES.items()}
    header, off = {}, 0
    for name in sorted(tensors):
        t = tensors[name]
        n = t.numel() * t.element_size()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob)
        for name in sorted(tensors):
            t = tensors[name].detach().contiguous()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())


def read_model_folder(model_dir):
    """(config dict, {tensor name: float32 CPU tensor}) of a model folder."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = {k: (t.to(torch.float32) if t.dtype.is_floating_point else t)
               for k, t in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, tensors


def sizes(cfg):
    E, H = cfg["hidden_size"], cfg["num_attention_heads"]
    KV = cfg.get("num_key_value_heads") or H
    hd = cfg.get("head_dim") or E // H          # fastgguf.c:4281-4283
    return E, H, KV, hd


# ------------------------------------------------------------------------------ parts
def plain_embedding(table, tokens):
    """x = Emb[token, :] with scale 1 (fastgguf.c:4576-4581, :4652, :4219)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def plain_rmsnorm(x, w, eps):
    """rmsnorm_w (fastgguf.c:3100-3105): sum of squares in double, inv = 1/sqrt(ss/n + eps),
    y = x * inv * w."""
    ss = (x.double() * x.double()).sum(-1, keepdim=True)
    inv = (1.0 / torch.sqrt(ss / x.shape[-1] + float(eps))).to(x.dtype)
    return x * inv * w.to(x.dtype)


def plain_rope_divisors(cfg, hd):
    """Per-pair divisors of the rotary frequency.  GGUF files carry them as ``rope_freqs.weight``
    (fastgguf.c:4278) and the reference divides the angle by them (:3131); their llama3 formula
    is not in the reference: wavelength l = 2 pi theta^(2j/hd);  l < orig/high -> 1;
    l > orig/low -> factor;  else s = (orig/l - low)/(high - low), 1 / ((1 - s)/factor + s)."""
    half = hd // 2
    rs = cfg.get("rope_scaling")
    out = [1.0] * half
    if not rs or rs.get("rope_type", rs.get("type", "default")) == "default":
        return out
    assert rs.get("rope_type", rs.get("type")) == "llama3"
    theta, factor = float(cfg.get("rope_theta", 10000.0)), float(rs["factor"])
    low, high = float(rs["low_freq_factor"]), float(rs["high_freq_factor"])
    orig = float(rs["original_max_position_embeddings"])
    for j in range(half):
        wavelen = 2.0 * math.pi * theta ** (2.0 * j / hd)
        if wavelen < orig / high:
            out[j] = 1.0
        elif wavelen > orig / low:
            out[j] = factor
        else:
            s = (orig / wavelen - low) / (high - low)
            out[j] = 1.0 / ((1.0 - s) / factor + s)
    return out


def plain_rope(x, positions, theta, divisors):
    """apply_rope (fastgguf.c:3123-3145), the branch that pairs (j, j + half) (:3138-3139), over all
    of head_dim: angle = pos / theta^(2j/hd) / divisor_j in double (:3130-3131);
    (a, b) <- (a cos - b sin, a sin + b cos) (:3140-3141).  x: [T, heads, hd]."""
    T, _, hd = x.shape
    half = hd // 2
    cs, sn = np.empty((T, half)), np.empty((T, half))
    for t in range(T):
        for j in range(half):
            ang = float(positions[t]) / (float(theta) ** (2.0 * j / hd)) / divisors[j]
            cs[t, j], sn[t, j] = math.cos(ang), math.sin(ang)
    c = torch.from_numpy(cs).to(x.dtype)[:, None, :]      # rounded to the working type as :3132-3133
    s = torch.from_numpy(sn).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def plain_attention(q, k, v, scale, window=None):
    """Causal grouped-query attention of one whole sequence (fastgguf.c:3273-3326 attn_rows;
    head h uses KV head h / (H/KV), :4781; scores scale * q.k over positions [start, pos],
    :3317, :4754-4758; softmax with max subtraction, :3147-3156; o = sum w_p V[p], :3320-3323).
    q: [T, H, hd]; k, v: [T, KV, hd]; returns [T, H, hd]."""
    T, H, hd = q.shape
    G = H // k.shape[1]
    out = torch.zeros_like(q)
    for h in range(H):
        kvh = h // G
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            s = (k[lo:t + 1, kvh] @ q[t, h]) * scale
            e = torch.exp(s - s.max())
            w = e / e.sum()
            out[t, h] = w @ v[lo:t + 1, kvh]
    return out


def plain_silu(z):
    """silu_f (fastgguf.c:3118): z / (1 + exp(-z))."""
    return z / (1.0 + torch.exp(-z))


def plain_swiglu(x, w_gate, w_up, w_down):
    """Feed-forward (fastgguf.c:4870-4877): down( silu(gate x) * (up x) )."""
    return (plain_silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


# ------------------------------------------------------------------------------ the model
def plain_layer(x, W, prefix, cfg, positions, window=None):
    """One decoder layer on a whole sequence (fastgguf.c:4686-4895): attention on the normalized
    input, projection added onto the un-normalized input (:4860-4862), then the same for the
    feed-forward (:4865-4880)."""
    E, H, KV, hd = sizes(cfg)
    eps = cfg.get("rms_norm_eps", 1e-6)                        # default as fastgguf.c:4228
    theta = cfg.get("rope_theta", 10000.0)                     # default as fastgguf.c:4224
    T = x.shape[0]
    n1 = plain_rmsnorm(x, W[prefix + "input_layernorm.weight"], eps)
    q = (n1 @ W[prefix + "self_attn.q_proj.weight"].T).reshape(T, H, hd)
    k = (n1 @ W[prefix + "self_attn.k_proj.weight"].T).reshape(T, KV, hd)
    v = (n1 @ W[prefix + "self_attn.v_proj.weight"].T).reshape(T, KV, hd)
    div = plain_rope_divisors(cfg, hd)
    q, k = plain_rope(q, positions, theta, div), plain_rope(k, positions, theta, div)
    a = plain_attention(q, k, v, 1.0 / math.sqrt(hd), window).reshape(T, H * hd)   # scale :4744
    h1 = a @ W[prefix + "self_attn.o_proj.weight"].T + x
    n2 = plain_rmsnorm(h1, W[prefix + "post_attention_layernorm.weight"], eps)
    return plain_swiglu(n2, W[prefix + "mlp.gate_proj.weight"], W[prefix + "mlp.up_proj.weight"],
                        W[prefix + "mlp.down_proj.weight"]) + h1


def plain_forward(cfg, tensors, tokens, dtype=torch.float64):
    """Logits [T, vocab] of one whole sequence starting at position 0 (fastgguf.c:4648-4907):
    embedding, the layers, final norm (:4899), head = lm_head or the embedding table when tied
    (:4269-4270, :4900)."""
    W = {k: (v.to(dtype) if v.dtype.is_floating_point else v) for k, v in tensors.items()}
    x = plain_embedding(W["model.embed_tokens.weight"], tokens)
    positions = list(range(len(tokens)))
    for i in range(cfg["num_hidden_layers"]):
        x = plain_layer(x, W, f"model.layers.{i}.", cfg, positions)
    xf = plain_rmsnorm(x, W["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else W["lm_head.weight"]
    return xf @ head.T


# ------------------------------------------------------------------------------ sampling
MASK64 = (1 << 64) - 1


def plain_rng_next(state):
    """xorshift64* (fastgguf.c:3334-3339); returns (new state, output)."""
    x = state
    x ^= x >> 12
    x ^= (x << 25) & MASK64
    x ^= x >> 27
    return x, (x * 0x2545F4914F6CDD1D) & MASK64


def plain_rng_uniform(state):
    """rng_uniform (fastgguf.c:3979-3981): top 24 bits / 2^24 as float."""
    state, out = plain_rng_next(state)
    return state, np.float32(out >> 40) / np.float32(16777216.0)


def plain_argmax(v):
    """argmax_f (fastgguf.c:3328-3332): first maximum wins."""
    best, bv = 0, -math.inf
    for i, x in enumerate(v):
        if x > bv:
            best, bv = i, x
    return best


def plain_sample(logits, state, hist, *, temp, top_k, top_p, repeat_penalty, repeat_last_n, stop_ids=()):
    """sample_next (fastgguf.c:4008-4056) in float32.  ``logits``: 1-D float32 array (a copy is
    modified).  Returns (token, new rng state)."""
    f32 = np.float32
    lg = np.array(logits, dtype=np.float32)
    n = lg.shape[0]
    if repeat_penalty > 0.0 and repeat_penalty != 1.0 and repeat_last_n > 0:          # :4010-4021
        start = max(0, len(hist) - repeat_last_n)
        for i in range(start, len(hist)):
            tid = hist[i]
            if tid < 0 or tid >= n or tid in stop_ids or tid in hist[start:i]:
                continue
            lg[tid] = lg[tid] / f32(repeat_penalty) if lg[tid] > 0 else lg[tid] * f32(repeat_penalty)
    if temp <= 0.0:                                                                   # :4022
        return plain_argmax(lg), state
    if top_k > 0:                                                                     # :3989-4005
        order = sorted(range(n), key=lambda i: (-lg[i], i))[:min(top_k, n)]
    else:                                                                             # :4026-4035
        cut = lg[plain_argmax(lg)] - f32(20.0) * f32(temp)
        order = sorted([i for i in range(n) if lg[i] > cut], key=lambda i: (-lg[i], i))
    mx = lg[order[0]]
    p = [np.exp(f32(f32(lg[i] - mx) / f32(temp)), dtype=np.float32) for i in order]    # :4036-4037
    total = f32(0.0)
    for x in p:
        total = f32(total + x)
    keep = len(p)
    if 0.0 < top_p < 1.0:                                                             # :4039-4047
        cum, lim = f32(0.0), f32(f32(top_p) * total)
        for i, x in enumerate(p):
            cum = f32(cum + x)
            if cum >= lim:
                keep = i + 1
                break
    tot = f32(0.0)
    for x in p[:keep]:
        tot = f32(tot + x)
    state, u = plain_rng_uniform(state)                                               # :4049-4055
    r = f32(u * tot)
    for i in range(keep):
        r = f32(r - p[i])
        if r < 0:
            return order[i], state
    return order[keep - 1], state


def plain_generate(cfg, tensors, prompt, *, max_tokens, stop_ids=(), seed=1, dtype=torch.float64, **sampling):
    """The chat loop (fastgguf.c:5284-5309) on token ids: run the prompt, then sample, stop
    BEFORE recording a stop token (:5296), append, run again.  Recomputes the whole sequence each
    step (no cache).  Returns the generated tokens."""
    seq, out, state = list(prompt), [], seed
    for _ in range(max_tokens):
        logits = plain_forward(cfg, tensors, seq, dtype)[-1].to(torch.float32).numpy()
        tok, state = plain_sample(logits, state, seq, stop_ids=stop_ids, **sampling)
        if tok in stop_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out
