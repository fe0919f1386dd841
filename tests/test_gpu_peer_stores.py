"""GPU (one device): the fused all-gather epilogue, with the "peers" played by further buffers of the same GPU.

sq_gemm with num_peer_outputs > 0 writes every finished tile to this rank's own matrix and to the same columns of every
peer's [M, N_total] matrix.  Two store forms exist: wide boxes of [16 rows x 128 bytes] (tiles 128 or 256 columns wide) and
the plain [32 rows x 16 columns] boxes (192-column tiles).  Checked for both, with both kernels, on ragged shapes, for
16-bit and fp32 outputs:
 * this rank's block is bit-identical to the same GEMM without peers (so to everything the parity tests pin),
 * every peer's column block holds the same bytes,
 * nothing outside the block is touched in a peer's matrix."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from segquant_b200 import _lib as L
from segquant_b200 import ops

DEV = "cuda:0"


def _case(kind, M, N, K, bounds, dual, group, out_dtype, seed):
    g = torch.Generator().manual_seed(seed)
    if kind == L.SQ_GEMM_W8A8_F8:
        xq = (torch.randn(M, K, generator=g) * 20).to(torch.float8_e4m3fn).view(torch.uint8)
        xn = (-torch.randn(M, K, generator=g).abs() * 2).to(torch.float8_e4m3fn).view(torch.uint8)
        wq = (torch.randn(N, K, generator=g) * 40).to(torch.float8_e4m3fn).view(torch.uint8)
    else:
        xq = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int16).to(torch.int8).view(torch.uint8)
        xn = torch.randint(-128, 1, (M, K), generator=g, dtype=torch.int16).to(torch.int8).view(torch.uint8)
        if kind == L.SQ_GEMM_W4A8:
            wq = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.int16).to(torch.uint8)
        else:
            wq = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int16).to(torch.int8).view(torch.uint8)
    S = len(bounds) - 1
    G = K // group if group else 1
    sx = torch.rand(S, generator=g) * 3 + 0.5
    sxn = torch.rand(S, generator=g) * 30 + 5
    sw = torch.rand(G, N, generator=g) * 100 + 50
    bias = torch.randn(N, generator=g)
    d = lambda t: t.to(DEV)
    args = (kind, d(xq).unsqueeze(0), d(wq).unsqueeze(0), N, bounds, d(sx), d(sw))
    kw = dict(xq_neg=d(xn).unsqueeze(0) if dual else None, sx_neg=d(sxn) if dual else None, group_size=group,
              sw_strides=(0, 0, N if group else 0, 1), bias=d(bias), out_dtype=out_dtype)
    return args, kw


# kind, M, N, K, bounds, DualScale, group, forced (bn, two_cta) or None, what store form this exercises
CASES = [
    (L.SQ_GEMM_W8A8_I8, 2500, 1352, 2304, [0, 768, 2304], False, 0, None, "pair, wide boxes, ragged M and N (N % 64 = 8)"),
    (L.SQ_GEMM_W8A8_I8, 700, 1096, 512, [0, 512], False, 0, None, "one-CTA kernel (K < 2048), wide boxes"),
    (L.SQ_GEMM_W8A8_I8, 700, 1096, 512, [0, 512], False, 0, (128, 0), "one-CTA kernel, 128-column tiles, wide boxes"),
    (L.SQ_GEMM_W8A8_F8, 1300, 840, 2560, [0, 2560], True, 0, (256, 1), "pair + DualScale, wide boxes"),
    (L.SQ_GEMM_W8A8_F8, 900, 840, 1024, [0, 1024], True, 0, (0, 0), "one-CTA kernel + DualScale, wide boxes"),
    (L.SQ_GEMM_W4A8, 900, 776, 768, [0, 256, 768], False, 128, None, "int4 weights with groups, one-CTA kernel, wide boxes"),
    (L.SQ_GEMM_W8A8_I8, 1000, 968, 2048, [0, 2048], False, 0, (192, 1), "192-column tiles forced: 16-column boxes"),
]


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kind,M,N,K,bounds,dual,group,forced,what", CASES)
def test_peer_blocks_equal_the_plain_result(native_lib, kind, M, N, K, bounds, dual, group, forced, what, out_dtype):
    args, kw = _case(kind, M, N, K, bounds, dual, group, out_dtype, seed=M + N)
    n_total, col0 = N + 2 * 264, 264          # the block sits in the middle of the peers' wider matrices (16-byte aligned offset)
    try:
        if forced is not None:
            ops.set_gemm_schedule(bn=forced[0], two_cta=forced[1])
        plain = ops.gemm(*args, **kw)[0]
        own = torch.full((M, n_total), 7.0, dtype=out_dtype, device=DEV)
        peers = [torch.full((M, n_total), float(3 + j), dtype=out_dtype, device=DEV) for j in range(3)]
        ops.gemm(*args, out=own[:, col0:col0 + N].unsqueeze(0), y_strides=(M * n_total, n_total),
                 peer_outputs=([q.data_ptr() for q in peers], n_total, col0), **kw)
        torch.cuda.synchronize()
    finally:
        ops.set_gemm_schedule()
    assert ops.device_status() == 0
    assert torch.equal(own[:, col0:col0 + N], plain), what
    assert bool((own[:, :col0] == 7.0).all()) and bool((own[:, col0 + N:] == 7.0).all()), what
    for j, q in enumerate(peers):
        assert torch.equal(q[:, col0:col0 + N], plain), (what, j)
        assert bool((q[:, :col0] == float(3 + j)).all()) and bool((q[:, col0 + N:] == float(3 + j)).all()), (what, j)


def test_peer_barrier_signals_waits_and_gives_up_within_its_bound(native_lib):
    """sq_peer_barrier on one GPU, the second rank played by the host (two kernels that wait for one another must not
    share a GPU): rank 0's kernel must store its epoch into the peer's word, pass when the peer's arrival is already
    there, and - when nobody arrives - give up after the configured number of cycles, report wait id 10 with the peer's
    rank, and leave the context usable.  Nothing faults or traps."""
    lib = L.load()
    assert ops.device_status() == 0
    flags = [torch.zeros(64, dtype=torch.int32, device=DEV) for _ in range(2)]
    ptrs = [f.data_ptr() for f in flags]
    flags[0][1] = 1                                   # "rank 1 has arrived at barrier 1"
    ops.peer_barrier(0, ptrs, 1, torch.device(DEV))
    torch.cuda.synchronize()
    assert int(flags[1][0]) == 1 and ops.device_status() == 0
    ops.peer_barrier(0, ptrs[:1], 5, torch.device(DEV))          # world of one: nothing to do
    try:
        L.check(lib.sq_set_wait_limit_cycles(1_000_000), "sq_set_wait_limit_cycles")
        ops.peer_barrier(0, ptrs, 2, torch.device(DEV))          # rank 1 never arrives at barrier 2
        with pytest.raises(L.SegQuantError) as e:
            ops.check_device()
        assert e.value.status == L.SQ_ERR_DEVICE_TIMEOUT and "wait id 10" in str(e.value) and "block 1" in str(e.value)
    finally:
        L.check(lib.sq_set_wait_limit_cycles(0), "sq_set_wait_limit_cycles")
    assert int(flags[1][0]) == 2                      # it had signalled before it waited
    assert ops.device_status() == 0                   # reading the status cleared it
    with pytest.raises(L.SegQuantError):
        ops.peer_barrier(3, ptrs, 3, torch.device(DEV))          # rank outside the world
