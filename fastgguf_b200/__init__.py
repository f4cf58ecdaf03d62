"""fastgguf_b200: a small model library with generation of its own for one GPU (NVIDIA B200,
sm_100a): typed configuration and an architecture registry, weights from safetensors, layers put
together from parts, a paged cache with per-sequence slots, one step function, a generation loop,
sampling, trace replay, and hand-written CUDA kernels for prefill and decode.

    from fastgguf_b200 import Engine
    engine = Engine.from_dir("model_dir", dtype="bfloat16", max_tokens=8192)
    out = engine.generate([[1, 2, 3]], temp=0, max_tokens=16)
"""
__version__ = "0.1.0"

__all__ = ["Engine", "StepEntry", "SamplingParams", "generate"]


def __getattr__(name):
    if name == "Engine":
        from .engine.api import Engine
        return Engine
    if name == "StepEntry":
        from .engine.batch import StepEntry
        return StepEntry
    if name == "SamplingParams":
        from .sampling import SamplingParams
        return SamplingParams
    if name == "generate":
        return generate
    raise AttributeError(name)


def generate(model_dir, prompts, *, ctx=2048, dtype="bfloat16", **options):
    """Load ``model_dir`` and generate for ``prompts`` (lists of token ids).  ``ctx`` and the options
    (temp, top_k, top_p, repeat_penalty, repeat_last_n, max_tokens, seed) are the reference's chat
    arguments (fastgguf.c:6957-6982)."""
    from .engine.api import Engine
    batch = min(len(prompts), 64)
    ctx = max(64, ctx)
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=batch * ((ctx + 63) // 64 * 64), max_batch=batch,
                             max_seq_len=ctx)
    return engine.generate(prompts, **options)
