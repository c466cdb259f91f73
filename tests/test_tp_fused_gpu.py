"""The fused row-parallel output projection + all-reduce of a decode step (``based_tp_outproj_allreduce``).

One-GPU tier: all ranks run inside ONE cooperative launch (``based_tp_outproj_allreduce_emulated``), which exercises the
whole exchange protocol — push into every rank's workspace, per-tile flags, bounded wait, rank-ordered sum, the call
counter that the kernel advances itself — against ``sum_r x_r W_r^T`` in fp64.  The two-GPU tier (real peer memory over
NVLink, one process per GPU) is in ``test_tp_gpu.py``.  Tolerance: 2e-2 relative as for every bf16 result; the ranks'
outputs must be bit-identical to one another."""
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,M,N,K,max_rows,with_bias", [(1, 16, 64, 32, 16, False), (2, 5, 256, 96, 16, True),
                                                             (4, 64, 448, 448, 64, False), (8, 64, 256, 224, 64, True),
                                                             (8, 3, 256, 224, 64, False), (2, 33, 1024, 512, 48, False),
                                                             (1, 64, 1792, 224, 64, True)])
def test_emulated_ranks_match_the_sum_of_partial_products(world, M, N, K, max_rows, with_bias):
    """Sizes are bounded by what one GPU can keep resident at once (all ranks' blocks wait on one another); the last
    case is one rank's launch at the 1.4B model's decode size (d_model 1792, batch 64, 8-way sharded heads)."""
    from based_b200 import _capi, ops
    g = torch.Generator(device="cuda").manual_seed(world * 1000 + M)
    nbytes = ops.tp_outproj_workspace_bytes(world, max_rows, N)
    ws = [ops.tp_outproj_workspace_init_(torch.empty(nbytes, dtype=torch.uint8, device="cuda")) for _ in range(world)]
    bias = (torch.randn(N, device="cuda", generator=g) / 4).bfloat16() if with_bias else None
    for call in range(4):   # the two buffer sets alternate; the call counter lives in the workspace
        xs = [(torch.randn(M, K, device="cuda", generator=g) / 2).bfloat16() for _ in range(world)]
        wts = [(torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16() for _ in range(world)]
        outs = ops.tp_outproj_allreduce_emulated(xs, wts, bias, ws, max_rows)
        torch.cuda.synchronize()
        assert _capi.read_status() == 0
        ref = sum(x.double() @ w.double().T for x, w in zip(xs, wts))
        if bias is not None:
            ref = ref + bias.double()
        for r in range(world):
            assert outs[r].shape == (M, N) and outs[r].dtype == torch.bfloat16
            assert torch.equal(outs[r], outs[0]), f"rank {r} differs from rank 0 (call {call})"
        assert rel_err(outs[0], ref) < 2e-2, call
        # fp32 partials, one rounding: as good as rounding the exact sum
        assert rel_err(outs[0], ref) < 1e-2


def test_single_rank_equals_decode_linear():
    """world = 1 degenerates to a plain projection: same result as the library's own decode-step linear."""
    from based_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(5)
    M, N, K = 16, 512, 256
    x = (torch.randn(M, K, device="cuda", generator=g) / 2).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / 16).bfloat16()
    ws = ops.tp_outproj_workspace_init_(torch.empty(ops.tp_outproj_workspace_bytes(1, M, N), dtype=torch.uint8, device="cuda"))
    out = ops.tp_outproj_allreduce(x, w, None, [ws.data_ptr()], M, 0, 1)
    ref = ops.decode_linear(x, w)
    assert rel_err(out, ref.double()) < 4e-3
    out2 = ops.tp_outproj_allreduce(x, w, None, [ws.data_ptr()], M, 0, 1)
    assert torch.equal(out, out2)


def test_argument_checks():
    from based_b200 import _capi, ops
    with pytest.raises(ValueError):
        ops.tp_outproj_workspace_bytes(9, 16, 64)          # more ranks than one NVLink domain holds
    x = torch.zeros(4, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    ws = ops.tp_outproj_workspace_init_(torch.empty(ops.tp_outproj_workspace_bytes(1, 4, 64), dtype=torch.uint8, device="cuda"))
    with pytest.raises(ValueError):
        ops.tp_outproj_allreduce(torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16), w, None, [ws.data_ptr()], 4, 0, 1)
    with pytest.raises(TypeError):
        ops.tp_outproj_allreduce(x.float(), w, None, [ws.data_ptr()], 4, 0, 1)
    with pytest.raises(_capi.BasedLibraryError):
        ops.tp_outproj_allreduce(x, w, None, [ws.data_ptr() + 16], 4, 0, 1)   # workspace not 256-byte aligned
