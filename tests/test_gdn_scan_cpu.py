"""The scan form of the gated delta rule (intra-chunk work batched, chunk-to-chunk recurrence as a scan whose backward
is the reverse scan) against the per-document chunked reference, on CPU in float32: outputs and all gradients."""
import torch

from vlm_training_b200.ops import reference as ref
from vlm_training_b200.ops.gdn_scan import chunk_table, doc_chunk_ranges, gated_delta_rule_scan, native_usable


def test_doc_chunk_ranges_skip_empty_documents():
    dst, n, first, count = doc_chunk_ranges([0, 70, 70, 199, 290], 64)
    assert n == 2 + 3 + 2
    assert first.tolist() == [0, 2, 5] and count.tolist() == [2, 3, 2]
    assert dst[0] == 0 and dst[69] == 69 and dst[70] == 128 and dst[199] == 5 * 64
    assert len(set(dst.tolist())) == 290


def test_chunk_table_lists_every_chunk_slot_in_layout_order():
    """The table the chunk kernels walk: one entry per slot of the padded layout (first token, rows), consistent with the
    token -> slot map of ``doc_chunk_ranges``; empty documents have no slot, a document's last chunk may be short."""
    cu = [0, 70, 70, 199, 290, 354]
    table = chunk_table(cu, 64)
    dst, n, first, count = doc_chunk_ranges(cu, 64)
    assert table.shape == (n, 2) and table.dtype.name == "int32"
    assert table.tolist() == [[0, 64], [64, 6], [70, 64], [134, 64], [198, 1], [199, 64], [263, 27], [290, 64]]
    for slot, (tok0, rows) in enumerate(table.tolist()):
        assert dst[tok0] == slot * 64 and dst[tok0 + rows - 1] == slot * 64 + rows - 1
    assert int(table[:, 1].sum()) == cu[-1]


def test_native_chunk_kernels_are_not_chosen_off_the_gpu():
    q = torch.randn(64, 2, 128).bfloat16()
    assert not native_usable(q, q, q, 64)


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
