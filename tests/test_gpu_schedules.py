"""GPU: every schedule the host can pick, pinned bit for bit.

The host chooses a tile width (128 / 192 / 256 columns), the one-CTA or the CTA-pair kernel and, for the pair, 128- or
256-byte K stages per pipeline step; small test shapes would only ever meet one of them.  Here each combination is
forced (sq_set_gemm_schedule) on a shape with at least two rounds of tiles over the 148 SMs and ragged M and N edges,
for INT8 / FP8 / W4A8, single scale and DualScale, per-tensor and per-token activation scales:

 * the int32 accumulators written by the dump variant of the epilogue equal the CPU oracle's (fp32 accumulators of the
   e4m3 kernel: within 2e-6, the accumulation order is the hardware's);
 * the PRODUCTION epilogue variants (no dump: magic-number or cvt conversion, per-token or not) give the same output
   bytes as the dump run, which in turn is within 1e-5 of the oracle's output.

Also here: the bounded-wait path, made to run out on purpose in a stand-alone probe kernel (nothing faults or traps)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import oracle as O
from segquant_b200 import _lib as L
from segquant_b200 import ops

DEV = "cuda:0"
KIND = {"i8": (L.SQ_GEMM_W8A8_I8, O.GEMM_I8), "f8": (L.SQ_GEMM_W8A8_F8, O.GEMM_F8), "w4": (L.SQ_GEMM_W4A8, O.GEMM_W4A8)}
SCHEDULES = [(bn, cta2, ksub) for bn in (128, 192, 256) for cta2, ksub in ((0, 0), (1, 1), (1, 2))]


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def operands(kind, M, N, K, seed):
    rng = np.random.default_rng(seed)
    if kind == "f8":
        return (O.e4m3_encode(rng.standard_normal((M, K)).astype(np.float32) * 30),
                O.e4m3_encode(-np.abs(rng.standard_normal((M, K))).astype(np.float32) * 3),
                O.e4m3_encode(rng.standard_normal((N, K)).astype(np.float32) * 60), None)
    xq = rng.integers(-128, 128, (M, K)).astype(np.int8)
    xn = rng.integers(-128, 1, (M, K)).astype(np.int8)
    if kind == "w4":
        w = rng.integers(-8, 8, (N, K)).astype(np.int8)
        u = (w.astype(np.int16) & 0xF).astype(np.uint8)
        packed = (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)
        return xq, xn, packed, packed.reshape(-1)
    return xq, xn, rng.integers(-128, 128, (N, K)).astype(np.int8), None


# kind, K, segment bounds, weight group, DualScale, per-token activation scales
CASES = [
    ("i8", 1536, [0, 512, 1536], 0, False, False),       # units of 512 / 1024: cvt conversion
    ("i8", 768, [0, 768], 128, True, False),             # units of 128: magic conversion, DualScale
    ("i8", 1024, [0, 256, 1024], 0, False, True),        # per-token activation scales
    ("f8", 1536, [0, 512, 1536], 0, True, False),
    ("f8", 1024, [0, 1024], 0, False, True),
    ("w4", 768, [0, 256, 768], 128, False, False),       # int4 weights, groups of 128
    ("w4", 512, [0, 512], 0, True, False),               # int4 weights, per-channel scales, DualScale
]
M, N = 2600, 2000     # 21 x 16 tiles of 128 x 128 (336: three rounds), 11 x 8 pair tiles of 256 x 256 (88: two rounds); both edges ragged


@pytest.fixture(scope="module")
def oracle_results():
    return {}


@pytest.mark.parametrize("kind,K,bounds,group,dual,per_token", CASES)
def test_every_schedule_is_bit_exact(native_lib, kind, K, bounds, group, dual, per_token):
    S = len(bounds) - 1
    xq, xn, wq, wq_flat = operands(kind, M, N, K, seed=K + S + group)
    rng = np.random.default_rng(7)
    sx = rng.uniform(0.5, 4.0, (S, M) if per_token else (S,)).astype(np.float32)
    sxn = rng.uniform(5.0, 40.0, (S, M) if per_token else (S,)).astype(np.float32)
    G = K // group if group else 1
    sw = rng.uniform(50, 150, (G, N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    y_ref, acc_ref = O.seg_gemm(KIND[kind][1], xq, wq_flat if wq_flat is not None else wq, bounds, sx, sw if group else sw[0],
                                xq_neg=xn if dual else None, sx_neg=sxn if dual else None, group_size=group, bias=bias, want_acc=True)
    args = (KIND[kind][0], t(xq.view(np.uint8)).unsqueeze(0), t(wq.view(np.uint8)).unsqueeze(0), N, bounds, t(sx), t(sw))
    kw = dict(xq_neg=t(xn.view(np.uint8)).unsqueeze(0) if dual else None, sx_neg=t(sxn) if dual else None, per_token=per_token,
              group_size=group, sw_strides=(0, 0, N if group else 0, 1), bias=t(bias), out_dtype=torch.float32)
    seen = set()
    try:
        for bn, cta2, ksub in SCHEDULES:
            ops.set_gemm_schedule(bn=bn, two_cta=cta2, ksub=ksub)
            y_dump, acc = ops.gemm(*args, want_acc=True, **kw)
            acc = acc[0].cpu().numpy()
            if kind == "f8":
                assert np.abs(acc.view(np.float32) - acc_ref).max() <= 2e-6 * np.abs(acc_ref).max(), (bn, cta2, ksub)
            else:
                assert np.array_equal(acc, acc_ref), f"int32 accumulators differ with bn={bn} cta2={cta2} ksub={ksub}"
            y_prod = ops.gemm(*args, **kw)                     # production epilogue variant of the same schedule
            if kind == "f8":     # fp32 accumulators may differ in the last bit between schedules, never between variants
                assert torch.equal(y_prod, y_dump), (bn, cta2, ksub)
            else:
                assert torch.equal(y_prod, y_dump), f"production epilogue differs from the dump run: bn={bn} cta2={cta2} ksub={ksub}"
            rel = float(np.abs(y_prod[0].cpu().numpy() - y_ref).max() / np.abs(y_ref).max())
            assert rel < 1e-5, (bn, cta2, ksub, rel)
            seen.add(y_prod.cpu().numpy().tobytes() if kind != "f8" else b"")
            # bf16 output of the production variant: the fp32 result rounded once
            if (bn, cta2, ksub) in ((192, 1, 2), (128, 0, 0)):
                kw16 = dict(kw, out_dtype=torch.bfloat16)
                y16 = ops.gemm(*args, **kw16)
                assert torch.equal(y16, y_prod.to(torch.bfloat16)), (bn, cta2, ksub)
        assert len(seen) == 1, "integer kinds: every schedule must give the same output bytes"
    finally:
        ops.set_gemm_schedule()
    assert ops.device_status() == 0


def test_bounded_wait_gives_up_reports_and_leaves_the_context_usable(native_lib):
    """The failure path every kernel of the GEMM relies on, run once on purpose in a probe kernel: a wait on a barrier
    nobody arrives at runs out after ~1e6 cycles, the status word names it, the abort flag releases the other warp, the
    kernel returns; the status reads back once and clears; a GEMM launched afterwards is still bit-exact."""
    lib = L.load()
    assert ops.device_status() == 0
    out = torch.full((4,), -1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    L.check(lib.sq_wait_probe(1_000_000, out.data_ptr(), stream), "sq_wait_probe")
    with pytest.raises(L.SegQuantError) as e:
        ops.check_device()
    assert e.value.status == L.SQ_ERR_DEVICE_TIMEOUT and "wait id 9" in str(e.value) and "block 0" in str(e.value)
    assert out.tolist() == [1, 0, 0, 1]      # abort flag raised; both waits returned false; warp 1 left through the flag
    assert ops.device_status() == 0          # reading cleared it
    L.check(lib.sq_wait_probe(1_000_000, out.data_ptr(), stream), "sq_wait_probe")
    assert ops.device_status() == (0 << 8 | 9)
    ops.check_device()                       # cleared again: no error
    with pytest.raises(L.SegQuantError):
        L.check(lib.sq_wait_probe(10 ** 12, out.data_ptr(), stream), "sq_wait_probe")     # refused: limit too long for a probe
    with pytest.raises(L.SegQuantError):
        L.check(lib.sq_set_wait_limit_cycles(5), "sq_set_wait_limit_cycles")
    # the wait limit of the GEMM kernels is a launch parameter; a shortened (still generous) limit changes no result
    L.check(lib.sq_set_wait_limit_cycles(200_000_000), "sq_set_wait_limit_cycles")
    try:
        xq, _, wq, _ = operands("i8", 300, 272, 512, seed=1)
        sx, sw = np.array([2.0], np.float32), np.full(272, 80.0, np.float32)
        y_ref, acc_ref = O.seg_gemm(O.GEMM_I8, xq, wq, [0, 512], sx, sw, want_acc=True)
        y, acc = ops.gemm(L.SQ_GEMM_W8A8_I8, t(xq.view(np.uint8)).unsqueeze(0), t(wq.view(np.uint8)).unsqueeze(0), 272, [0, 512], t(sx), t(sw),
                          want_acc=True)
        assert np.array_equal(acc[0].cpu().numpy(), acc_ref)
    finally:
        L.check(lib.sq_set_wait_limit_cycles(0), "sq_set_wait_limit_cycles")
    assert ops.device_status() == 0
