"""Phase-trace summary and NVTX switch (host side only)."""
import torch

from coccl_b200.utils import trace


def test_summarise_takes_first_start_and_last_finish_per_phase():
    t = torch.zeros(trace.TRACE_MAX_CTAS, 4, dtype=torch.int64)
    t[0] = torch.tensor([1000, 3000, 6000, 6500])
    t[1] = torch.tensor([1200, 3500, 5000, 9000])
    s = trace.summarise(t)
    assert s["ctas"] == 2
    assert s["encode_push_us"] == (3500 - 1000) / 1e3
    assert s["decode_reduce_us"] == (6000 - 3500) / 1e3
    assert s["gather_us"] == (9000 - 6000) / 1e3
    assert s["total_us"] == (9000 - 1000) / 1e3
    assert trace.summarise(torch.zeros(trace.TRACE_MAX_CTAS, 4, dtype=torch.int64)) == {}


def test_nvtx_range_is_a_no_op_without_cuda():
    trace.enable_nvtx(True)
    with trace.nvtx_range("x"):
        pass
    trace.enable_nvtx(False)
