"""Single-GPU checks of the communication kernels: bounded flag waits that run out (nothing sets the flag; the kernel
must return, report through the status word and leave the context usable) and the all-gather -> GEMM kernel run as one
rank of two with the peer's part staged by the test (its flag already set, its rows already in the gathered buffer)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def short_waits():
    from vlm_training_b200.ops import cuda as cu

    cu.check_status(raise_on_error=False)
    cu._C.set_flag_wait_ms(50)
    cu._C.gemm_set_flag_wait_ms(50)
    yield cu
    cu._C.set_flag_wait_ms(20000)
    cu._C.gemm_set_flag_wait_ms(20000)
    cu.check_status(raise_on_error=False)


def _still_works(cu):
    a = torch.randn(256, 512, device="cuda").bfloat16()
    b = torch.randn(384, 512, device="cuda").bfloat16()
    y = cu._gemm(a, b)
    ref = a.float() @ b.float().t()
    torch.cuda.synchronize()
    assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-1)
    assert cu.check_status() == 0


def test_wait_flags_runs_out_and_reports(short_waits):
    cu = short_waits
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    cu._C.wait_flags(flags.data_ptr(), 0, 2, 1, 0)      # two ranks, collective 1, own rank 0 skipped: flag[1] never arrives
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="no signal from rank 1"):
        cu.check_status()
    assert int(cu.status_word()[0].item()) == 0           # reading the word cleared it
    _still_works(cu)


def test_pull_kernels_return_without_output_when_the_wait_runs_out(short_waits):
    cu = short_waits
    n = 1 << 16
    slot = torch.ones(2 * n, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags[0] = 1                                          # this rank signalled, the peer did not
    out = torch.zeros(2 * n, dtype=torch.bfloat16, device="cuda")
    cu._C.pull_gather([slot.data_ptr(), slot.data_ptr()], out, n, flags.data_ptr(), 1)
    torch.cuda.synchronize()
    assert cu.check_status(raise_on_error=False) == 101
    assert float(out.float().abs().sum()) == 0.0          # nothing was copied
    red = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    cu._C.pull_reduce([slot.data_ptr(), slot.data_ptr()], red, None, n, 0, flags.data_ptr(), 1)
    torch.cuda.synchronize()
    assert cu.check_status(raise_on_error=False) == 101
    assert float(red.float().abs().sum()) == 0.0
    # the same calls once the peer's flag is there
    flags[1] = 1
    cu._C.pull_gather([slot.data_ptr(), slot.data_ptr()], out, n, flags.data_ptr(), 1)
    cu._C.pull_reduce([slot.data_ptr(), slot.data_ptr()], red, None, n, 0, flags.data_ptr(), 1)
    torch.cuda.synchronize()
    assert cu.check_status() == 0
    assert float(out.float().min()) == 1.0 and float(red.float().min()) == 2.0


def test_fused_optimizer_kernel_skips_after_a_failed_wait(short_waits):
    """A wait that ran out leaves the status word set; the reduce-scatter + AdamW + all-gather kernel launched behind it
    must not touch master weights, moments or parameters."""
    cu = short_waits
    n = 8 * 1024
    g = torch.ones(n, dtype=torch.bfloat16, device="cuda")
    p = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    master, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    args = ([g.data_ptr()], [p.data_ptr()], 0, 0, 1, 0, n, master, m, v, 0, 1e-2, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001, 1.0, False)
    cu._C.wait_flags(flags.data_ptr(), 0, 2, 1, 0)
    cu._C.fused_rs_adamw_ag(*args)
    torch.cuda.synchronize()
    assert float(master.abs().sum()) == 0.0 and float(m.abs().sum()) == 0.0 and float(p.float().abs().sum()) == 0.0
    assert cu.check_status(raise_on_error=False) == 101
    cu._C.fused_rs_adamw_ag(*args)                        # status clear: the update happens
    torch.cuda.synchronize()
    assert float(m.min()) > 0.0 and float(master.max()) < 0.0


@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
def test_fused_optimizer_kernel_one_rank_matches_adamw(short_waits, state_dtype):
    """The one-kernel optimizer step on a domain of one rank (no peers): fp32 and bf16 moments against the plain AdamW
    kernel, and the gradients it consumed are cleared."""
    cu = short_waits
    n = 8 * 4096
    gen = torch.Generator(device="cuda").manual_seed(3)
    g = torch.randn(n, device="cuda", generator=gen).bfloat16()
    w0 = torch.randn(n, device="cuda", generator=gen)
    state = lambda: (w0.clone(), torch.zeros(n, device="cuda", dtype=state_dtype), torch.zeros(n, device="cuda", dtype=state_dtype))
    m1, a1, b1 = state()
    m2, a2, b2 = state()
    p1, p2 = torch.zeros(n, dtype=torch.bfloat16, device="cuda"), torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    g1, g2 = g.clone(), g.clone()
    for step in (1, 2):
        bc1, bc2 = 1 - 0.9 ** step, 1 - 0.999 ** step
        cu._C.fused_rs_adamw_ag([g1.data_ptr()], [p1.data_ptr()], 0, 0, 1, 0, n, m1, a1, b1, 0, 1e-2, 0.9, 0.999, 1e-8, 0.01, bc1, bc2,
                                0.5, True)
        cu.adamw_step_(g2, m2, a2, b2, p2, 1e-2, 0.9, 0.999, 1e-8, 0.01, step, 0.5, zero_grad=True)
        torch.cuda.synchronize()
        assert float(g1.float().abs().sum()) == 0.0       # consumed gradients are cleared
        torch.testing.assert_close(m1, m2, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(a1.float(), a2.float(), rtol=1e-2, atol=1e-6)
        assert torch.equal(p1, m1.bfloat16())
        g1.copy_(g)
        g2.copy_(g)
    assert cu.check_status() == 0


@pytest.mark.parametrize("rank", [0, 1])
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_all_gather_as_one_rank_of_two(short_waits, rank, b_mn):
    cu = short_waits
    torch.manual_seed(rank)
    R, K, N, e = 512, 1024, 768, 7
    x_all = (torch.randn(2 * R, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(K, N, device="cuda") * 0.05).bfloat16() if b_mn else (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    x_loc = x_all[rank * R:(rank + 1) * R].contiguous()
    peer = 1 - rank
    x_full = torch.zeros(2 * R, K, dtype=torch.bfloat16, device="cuda")
    x_full[peer * R:(peer + 1) * R] = x_all[peer * R:(peer + 1) * R]      # what the peer's kernel would have stored
    peer_buf = torch.zeros_like(x_full)                                    # stands for the peer's gathered buffer
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    peer_flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags[peer] = e                                                        # the peer's signal has arrived
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.empty(2 * R, N, dtype=torch.bfloat16, device="cuda")
    full_ptrs = [0, 0]
    full_ptrs[rank], full_ptrs[peer] = x_full.data_ptr(), peer_buf.data_ptr()
    flag_ptrs = [0, 0]
    flag_ptrs[rank], flag_ptrs[peer] = flags.data_ptr(), peer_flags.data_ptr()
    for _ in range(2):                                                     # twice: the CTA counter must reset itself
        cu._C.gemm_ag(x_loc, x_full, w, y, full_ptrs, flag_ptrs, 0, counter, e, rank, b_mn)
        torch.cuda.synchronize()
        assert cu.check_status() == 0
        ref = x_all.float() @ (w.float() if b_mn else w.float().t())
        assert torch.equal(x_full, x_all)
        assert torch.equal(peer_buf[rank * R:(rank + 1) * R], x_loc) and int(peer_flags[rank].item()) == e
        assert int(counter.item()) == 0
        assert ((y.float() - ref).abs().max() / ref.abs().max()).item() < 2e-2


def test_gemm_all_gather_gives_up_when_the_peer_never_signals(short_waits):
    cu = short_waits
    R, K, N = 256, 512, 384
    x_loc = torch.randn(R, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    x_full = torch.zeros(2 * R, K, dtype=torch.bfloat16, device="cuda")
    peer_buf = torch.zeros_like(x_full)
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    peer_flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.zeros(2 * R, N, dtype=torch.bfloat16, device="cuda")
    cu._C.gemm_ag(x_loc, x_full, w, y, [x_full.data_ptr(), peer_buf.data_ptr()], [flags.data_ptr(), peer_flags.data_ptr()], 0,
                  counter, 3, 0, False)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="no signal from rank 1"):
        cu.check_status()
    # the own rows were still pushed and announced, and their tiles computed
    assert torch.equal(peer_buf[:R], x_loc) and int(peer_flags[0].item()) == 3
    ref = x_loc.float() @ w.float().t()
    assert ((y[:R].float() - ref).abs().max() / ref.abs().max()).item() < 2e-2
    _still_works(cu)


@pytest.mark.parametrize("rank,world", [(0, 2), (1, 2), (2, 4)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_with_the_weight_gather_inside_as_one_rank(short_waits, rank, world, with_bias):
    """The parameter all-gather -> GEMM kernel with every rank's shard staged in local memory: the weight sits in the middle
    of a flat bucket, its region of the local whole bucket starts as NaN, and after the launch the product is right and
    the region holds the gathered weight (the rest of the bucket is untouched)."""
    cu = short_waits
    torch.manual_seed(7)
    M, N, K = 1024, 768, 512
    shard = (N * K + 4096) // world // 8 * 8 + 8           # the weight straddles every shard boundary
    total = shard * world
    w_lo = 1000 // 8 * 8
    assert w_lo + N * K <= total
    flat = (torch.randn(total, device="cuda") * 0.05).bfloat16()
    shards = [flat[r * shard:(r + 1) * shard].clone() for r in range(world)]
    bucket = torch.full((total,), float("nan"), device="cuda", dtype=torch.bfloat16)
    bucket[:w_lo] = 7.0
    bucket[w_lo + N * K:] = 7.0
    w = bucket[w_lo:w_lo + N * K].view(N, K)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16() if with_bias else None
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    sync = torch.zeros(2 * world, dtype=torch.int32, device="cuda")
    for epoch in (1, 2):                                    # a second call reuses the flags and counters
        if epoch == 2:
            bucket[w_lo:w_lo + N * K] = float("nan")
        cu._C.gemm_wgather(x, w, out, bias, bucket, [t.data_ptr() for t in shards], shard, rank, sync, epoch)
        torch.cuda.synchronize()
        assert cu.check_status() == 0
        w_ref = flat[w_lo:w_lo + N * K].view(N, K)
        assert torch.equal(w, w_ref)
        assert bool((bucket[:w_lo] == 7.0).all()) and bool((bucket[w_lo + N * K:] == 7.0).all())
        ref = x.float() @ w_ref.float().t() + (bias.float() if with_bias else 0.0)
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-1)
    _still_works(cu)


def test_debug_validation_of_index_tensors_sets_the_status_word(short_waits):
    """``VLMT_DEBUG_CHECKS``: bad ``cu_seqlens`` / image rows / expert ids are reported through the status word (no host read
    at the point of the check), good ones leave it alone."""
    cu = short_waits
    good = torch.tensor([0, 5, 5, 12], dtype=torch.int32, device="cuda")
    cu.validate_row_indices(good, 12, torch.tensor([0, 11], device="cuda"), torch.tensor([[0, 7]], device="cuda"), 8)
    assert cu.check_status() == 0
    cu.validate_row_indices(torch.tensor([0, 7, 5, 12], dtype=torch.int32, device="cuda"), 12)
    with pytest.raises(RuntimeError, match="cu_seqlens"):
        cu.check_status()
    cu.validate_row_indices(good, 12, torch.tensor([3, 12], device="cuda"))
    with pytest.raises(RuntimeError, match="image-token row"):
        cu.check_status()
    cu.validate_row_indices(None, 12, experts=torch.tensor([[0, 8]], device="cuda"), n_experts=8)
    with pytest.raises(RuntimeError, match="expert id"):
        cu.check_status()
