"""The device status word: every bounded in-kernel wait (mbarrier, peer flag) that runs out writes a code here and
makes its kernel return; the host reads the word after the step and raises.  Codes 1-5 come from
``csrc/sm100.cuh``; ``100 + r`` means "no signal from rank r" (``csrc/comm_kernels.cu``, the all-gather GEMM); 200 comes from the
expert-parallel plan kernel; 300-302 from the debug validation of index-bearing inputs (``ops.cuda.validate_row_indices``)."""
from __future__ import annotations

CODES = {
    1: "a TMA load did not arrive (full barrier)",
    2: "a shared-memory stage was not released (empty barrier)",
    3: "an accumulator in TMEM was not produced (TMEM full barrier)",
    4: "an accumulator in TMEM was not drained (TMEM empty barrier)",
    5: "a hand-off between the compute warps and the MMA thread did not happen",
}


OTHER = {
    200: "an expert-parallel rank would have received more rows than its buffer holds (raise VLMT_EP_CAPACITY)",
    300: "cu_seqlens is not a non-decreasing sequence from 0 to at most the row length",
    301: "an image-token row index lies outside the packed row",
    302: "an expert id lies outside [0, num_experts)",
}


def describe(code: int) -> str:
    if code in OTHER:
        return OTHER[code]
    if code >= 100:
        return f"no signal from rank {code - 100} within the wait limit"
    return CODES.get(code, f"unknown status code {code}")


def raise_if_set(word, what: str = "a kernel") -> int:
    """``word``: a one-element int32 tensor (device or host).  Clears it and raises if it is non-zero."""
    code = int(word.reshape(-1)[0].item())
    if code != 0:
        word.zero_()
        raise RuntimeError(f"{what} gave up on a bounded wait: {describe(code)} (status {code})")
    return code
