"""The Python entry point: load a model folder, step it, generate from it.

``Engine`` is what every program of the framework drives - generation, the command line, trace
replay, the benchmark and the tests share its model, step function, cache and kernels.  The
option names of ``generate`` are the reference's chat options with their meanings and defaults
(``--temp 1.0`` 0 = greedy, ``--top-k 64`` 0 = off, ``--top-p 0.95``, ``--repeat-penalty 1.0``
1 = off, ``--repeat-last-n 64``, ``--max-tokens 512`` 0 = until stop, ``--seed N``;
fastgguf.c:6957-6982), and ``ctx`` is its context length argument (default 2048, at least 64;
:6972, :7085).
"""
from __future__ import annotations

from typing import Optional, Sequence, Union

import torch

from ..config.base import ModelConfig
from ..parts.base import Runtime
from ..registry import config_from_dir, spec_from_config
from ..weights.loader import FolderSource, MemorySource, TensorSource
from .batch import StepEntry
from .model import DecoderModel

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
    "f32": torch.float32,
}


def parse_dtype(name: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {name}")
        return name
    try:
        return _DTYPES[name.lower()]
    except KeyError:
        raise ValueError(f"unknown dtype '{name}' (known: bfloat16, float32)") from None


class Engine:
    """A loaded model with its cache.  ``max_tokens`` sizes the cache: the most tokens that live
    sequences hold at any time, each sequence rounded up to a page of 64."""

    def __init__(self, config: ModelConfig, source: TensorSource, *, dtype="bfloat16", max_tokens: int = 8192,
                 max_batch: int = 64, max_seq_len: Optional[int] = None, device: str = "cuda:0",
                 use_graphs: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("fastgguf_b200 runs on a CUDA device (sm_100a); no GPU is visible and there is "
                               "no CPU path")
        self.config = config
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.spec = spec_from_config(config)
        self.model = DecoderModel(self.spec, Runtime(self.device, self.dtype))
        self.model.load_weights(source)
        self.max_batch = max_batch
        self.use_graphs = use_graphs
        self._backends: dict = {}
        self.cache = self.model.make_cache(max_tokens=max_tokens, n_slots=max_batch, max_seq_len=max_seq_len)

    @classmethod
    def from_dir(cls, model_dir: str, **kw) -> "Engine":
        """The model class is chosen by ``architectures[0]`` of ``model_dir/config.json``."""
        return cls(config_from_dir(model_dir), FolderSource(model_dir), **kw)

    @classmethod
    def from_tensors(cls, config: ModelConfig, tensors: dict, **kw) -> "Engine":
        return cls(config, MemorySource(tensors), **kw)

    # ------------------------------------------------------------------ stepping
    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def acquire(self) -> int:
        return self.model.acquire_slot()

    def release(self, slot: int) -> None:
        self.model.release_slot(slot)

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        return self.model.step(entries)

    def backend(self, params, stop_ids):
        """The sampler state and captured decode graphs for one set of sampling options (kept, so
        that a second call with the same options replays the graphs of the first)."""
        from .runner import EngineBackend
        key = (params, tuple(stop_ids))
        b = self._backends.get(key)
        if b is None:
            b = self._backends[key] = EngineBackend(self, params, stop_ids)
        else:
            b.reseed()
        return b

    # ------------------------------------------------------------------ generation
    def generate(self, prompts: Sequence[Sequence[int]], *, temp: float = 1.0, top_k: int = 64, top_p: float = 0.95,
                 repeat_penalty: float = 1.0, repeat_last_n: int = 64, max_tokens: int = 512, seed: int = 0,
                 stop_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False, batch_size: Optional[int] = None,
                 on_token=None):
        """Generate for every prompt (lists of token ids); returns one ``Completion`` per prompt.
        ``on_token(request_index, token)``, if given, is called for each generated token as the host sees it."""
        from ..sampling import SamplingParams
        from .generate import generate
        params = SamplingParams(temp=temp, top_k=top_k, top_p=top_p, repeat_penalty=repeat_penalty,
                                repeat_last_n=repeat_last_n, seed=seed)
        stops = tuple(self.spec.stop_token_ids if stop_ids is None else stop_ids)
        return generate(self, prompts, params, max_tokens=max_tokens, stop_ids=() if ignore_eos else stops,
                        batch_size=batch_size or self.max_batch, on_token=on_token)
