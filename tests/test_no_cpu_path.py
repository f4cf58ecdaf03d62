"""There is no CPU fallback: without a GPU the engine and every kernel wrapper refuse loudly."""
import pytest
import torch

from helpers import TINY_A, make_model_dir

needs_no_gpu = pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour on a machine without a GPU")


@needs_no_gpu
def test_engine_refuses_to_start_without_a_gpu(tmp_path):
    from fastgguf_b200.engine.api import Engine
    d = make_model_dir(tmp_path, TINY_A, 1, torch.float32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        Engine.from_dir(d, dtype="float32", max_tokens=128, max_batch=2)


def test_kernel_wrappers_refuse_cpu_tensors():
    from fastgguf_b200 import ops
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-5, torch.float32)
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.gemm_generic(torch.zeros(2, 8), torch.zeros(4, 8))
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.embed_gather(torch.zeros(16, 8), torch.zeros(2, dtype=torch.int32))
