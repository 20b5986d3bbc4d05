"""The scan form of the gated delta rule (intra-chunk work batched, chunk-to-chunk recurrence as a scan whose backward
is the reverse scan) against the per-document chunked reference, on CPU in float32: outputs and all gradients."""
import torch

from vlm_training_b200.ops import reference as ref
from vlm_training_b200.ops.gdn_scan import doc_chunk_ranges, gated_delta_rule_scan


def test_doc_chunk_ranges_skip_empty_documents():
    dst, n, first, count = doc_chunk_ranges([0, 70, 70, 199, 290], 64)
    assert n == 2 + 3 + 2
    assert first.tolist() == [0, 2, 5] and count.tolist() == [2, 3, 2]
    assert dst[0] == 0 and dst[69] == 69 and dst[70] == 128 and dst[199] == 5 * 64
    assert len(set(dst.tolist())) == 290


def test_scan_form_matches_chunked_reference_forward_and_backward():
    torch.manual_seed(0)
    T, H, Dk, Dv = 300, 3, 16, 24
    cu = [0, 70, 70, 199, 290]           # an empty document and a tail that belongs to no document
    ins = [torch.randn(T, H, Dk), torch.randn(T, H, Dk), torch.randn(T, H, Dv), -torch.rand(T, H) * 0.5, torch.rand(T, H)]
    ins = [t.requires_grad_() for t in ins]
    want = ref.gated_delta_rule(*ins, torch.tensor(cu))
    go = torch.randn_like(want)
    want.backward(go)
    grads = [t.grad.clone() for t in ins]
    for t in ins:
        t.grad = None
    got = gated_delta_rule_scan(*ins, cu)
    got.backward(go)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    for t, w in zip(ins, grads):
        torch.testing.assert_close(t.grad, w, atol=2e-5, rtol=1e-4)
