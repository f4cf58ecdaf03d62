"""The kernel timing module's command line (its timings need a GPU and are not asserted anywhere)."""
import pytest
import torch

from fastgguf_b200 import kernel_bench


def test_subcommand_is_required():
    with pytest.raises(SystemExit):
        kernel_bench.main([])


def test_unknown_head_size_is_refused():
    with pytest.raises(SystemExit):
        kernel_bench.main(["attention_prefill", "--head-dim", "96"])


@pytest.mark.skipif(torch.cuda.is_available(), reason="the refusal is for machines without a GPU")
def test_refuses_without_a_gpu():
    with pytest.raises(SystemExit, match="needs a GPU"):
        kernel_bench.main(["gemm"])


def test_peaks_have_a_fallback():
    hbm, tf = kernel_bench._peaks()
    assert hbm > 1000 and tf > 100
