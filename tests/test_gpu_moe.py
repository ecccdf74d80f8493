"""Mixture-of-experts block (router, bucketing, grouped quantized mat-vec, combine) against the CPU restatement of the
reference's sparse MoE forward (fuel-core/src/lazy_nn/moe.rs:92-127, 296-348)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _setup(E, H, F, seed=0):
    from fuel_b200 import GgmlDType as T, ops
    g = np.random.Generator(np.random.PCG64(seed))
    wgu = (g.standard_normal((E, 2 * F, H), dtype=np.float32) * np.float32(0.02))
    wd = (g.standard_normal((E, H, F), dtype=np.float32) * np.float32(0.02))
    bgu = ops.quantize_weights(T.Q4K, torch.from_numpy(wgu.reshape(E * 2 * F, H)).cuda())
    bd = ops.quantize_weights(T.Q4K, torch.from_numpy(wd.reshape(E * H, F)).cuda())
    return bgu, bd


def _split(blocks, E):
    b = blocks.cpu().numpy().reshape(-1)
    per = b.size // E
    return [b[e * per:(e + 1) * per] for e in range(E)]


@pytest.mark.parametrize("E,H,F,K,N", [(8, 512, 256, 2, 33), (16, 256, 256, 4, 3), (128, 2048, 768, 8, 40), (4, 256, 512, 1, 70),
                                       (128, 2048, 768, 8, 256)])   # the last: benchmark configuration 5 at its full 256 tokens
def test_moe_block_matches_reference_order(E, H, F, K, N):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import ops
    from fuel_b200.moe import QMoeBlock
    from oracle import moe_oracle as MO
    bgu, bd = _setup(E, H, F)
    g = np.random.Generator(np.random.PCG64(1))
    x = g.standard_normal((N, H), dtype=np.float32)
    logits = g.standard_normal((N, E), dtype=np.float32)
    logits[0, 1] = logits[0, 0]                       # a tie: the first index must win
    blk = QMoeBlock(E, H, F, K, bgu, bd, max_tokens=N)
    out = blk.forward(torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda())
    torch.cuda.synchronize()
    want, ids, w = MO.forward(x, logits, K, _split(bgu, E), _split(bd, E), E, H, F)
    assert np.array_equal(blk.topk_ids[:N].cpu().numpy(), ids)
    assert np.abs(blk.topk_w[:N].cpu().numpy() - w).max() <= 2e-7     # expf on the device vs exp on the host
    # bucketing: offsets are the prefix sums of the expert counts, rows inside an expert ascend
    off = blk.offsets.cpu().numpy()
    sid = blk.sorted_ids[:N * K].cpu().numpy()
    assert off[0] == 0 and off[-1] == N * K and np.array_equal(np.diff(off), np.bincount(ids.reshape(-1), minlength=E))
    for e in range(E):
        seg = sid[off[e]:off[e + 1]]
        assert np.all(np.diff(seg) > 0) and np.all(ids.reshape(-1)[seg] == e)
    got = out.cpu().numpy()
    # Two mat-vecs with a re-quantization between them: f32 summation order moves the intermediate by ~1e-7, which
    # now and then flips one 8-bit activation quant and shifts an output by one weight step. Most elements
    # agree to ~1e-7; the bound is the contract's 1e-3 of the tensor's largest value.
    err = np.abs(got - want) / np.abs(want).max()
    assert err.max() <= 1e-3 and np.quantile(err, 0.99) <= 3e-4 and np.median(err) <= 1e-6
    assert ops.device_error() == 0


def test_moe_grouped_matvec_equals_plain_matvec_per_expert():
    """The grouped kernel and the plain decode kernel compute the same dots (tolerance: summation order)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import GgmlDType as T, _lib, ops
    E, n, k, rows = 6, 384, 1024, [0, 5, 1, 16, 0, 9]
    L = _lib.lib
    g = np.random.Generator(np.random.PCG64(3))
    w = ops.quantize_weights(T.Q4K, torch.from_numpy(g.standard_normal((E * n, k), dtype=np.float32) * np.float32(0.02)).cuda())
    R = sum(rows)
    x = torch.from_numpy(g.standard_normal((R, k), dtype=np.float32)).cuda()
    off = torch.tensor(np.concatenate([[0], np.cumsum(rows)]), dtype=torch.int32, device="cuda")
    ident = torch.arange(R, dtype=torch.int32, device="cuda")
    packed = torch.zeros(L.fuelq_act_packed_bytes(int(T.Q4K), R, k), dtype=torch.uint8, device="cuda")
    _lib.check(L.fuelq_moe_quantize_rows(x.data_ptr(), k, ident.data_ptr(), 1, R, packed.data_ptr(), packed.numel(), None), "q")
    y = torch.zeros(R, n, device="cuda")
    _lib.check(L.fuelq_moe_qmatmul(int(T.Q4K), E, n, k, w.data_ptr(), packed.data_ptr(), R, off.data_ptr(), None,
                                   y.data_ptr(), None), "moe")
    per = w.numel() // E
    r0 = 0
    for e, m in enumerate(rows):
        if m:
            ref = ops.qmatmul(T.Q4K, w[e * per:(e + 1) * per], n, x[r0:r0 + m].contiguous())
            assert (y[r0:r0 + m] - ref).abs().max().item() <= 2e-6 * ref.abs().max().item()
        r0 += m
    assert ops.device_error() == 0


@pytest.mark.parametrize("E,n,k,rows", [(6, 384, 1024, [0, 5, 1, 16, 0, 9]), (3, 1536, 2048, [33, 0, 2]), (2, 100, 768, [7, 20]),
                                        (1, 37, 4096, [13]), (2, 72, 11008, [5, 20]), (1, 4096, 11008, [16])])
def test_tensor_core_grouped_kernel_matches_dp4a_grouped_kernel(E, n, k, rows):
    """Q4_K groups run on the integer tensor-core kernel; the dp4a kernel (development switch 107) computes the same
    integer dots, so the two agree up to f32 summation order."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import GgmlDType as T, _lib, ops
    L = _lib.lib
    g = np.random.Generator(np.random.PCG64(5))
    w = ops.quantize_weights(T.Q4K, torch.from_numpy(g.standard_normal((E * n, k), dtype=np.float32) * np.float32(0.02)).cuda())
    R = sum(rows)
    x = torch.from_numpy(g.standard_normal((R, k), dtype=np.float32)).cuda()
    off = torch.tensor(np.concatenate([[0], np.cumsum(rows)]), dtype=torch.int32, device="cuda")
    perm = torch.from_numpy(g.permutation(R).astype(np.int32)).cuda()
    ident = torch.arange(R, dtype=torch.int32, device="cuda")
    packed = torch.zeros(L.fuelq_act_packed_bytes(int(T.Q4K), R, k), dtype=torch.uint8, device="cuda")
    _lib.check(L.fuelq_moe_quantize_rows(x.data_ptr(), k, ident.data_ptr(), 1, R, packed.data_ptr(), packed.numel(), None), "q")
    ys = []
    for sw in (0, 1):
        if sw == 1 and k > 4096:
            break     # the dp4a grouped kernel keeps whole activation rows in shared memory: no plan for a k this large
        y = torch.full((R, n), float("nan"), device="cuda")
        try:
            L.fuelq_set_option(107, sw)
            _lib.check(L.fuelq_moe_qmatmul(int(T.Q4K), E, n, k, w.data_ptr(), packed.data_ptr(), R, off.data_ptr(),
                                           perm.data_ptr(), y.data_ptr(), None), "moe")
        finally:
            L.fuelq_set_option(107, 0)
        torch.cuda.synchronize()
        ys.append(y)
    # reference: the plain dp4a mat-vec, two rows at a time, expert by expert (k > 4096 runs the tensor-core kernel in
    # several sweeps over k)
    want = torch.full((R, n), float("nan"), device="cuda")
    per = w.numel() // E
    r0 = 0
    for e, m in enumerate(rows):
        for i in range(r0, r0 + m, 2):
            j = min(i + 2, r0 + m)
            want[perm[i:j].long()] = ops.qmatmul(T.Q4K, w[e * per:(e + 1) * per], n, x[i:j].contiguous())
        r0 += m
    for y in ys:
        assert not torch.isnan(y).any()
        assert (y - want).abs().max().item() <= 2e-6 * want.abs().max().item()
    assert ops.device_error() == 0


@pytest.mark.parametrize("P,E", [(0, 8), (1, 4), (31, 128), (33, 5), (2048, 128), (10000, 128), (20000, 128), (4096, 1024), (777, 3)])
def test_bucketing_is_a_stable_sort_by_expert(P, E):
    """fuelq_moe_bucket: pair ids ordered by expert, ascending inside an expert, offsets = prefix sums of the counts -
    for sizes that take the per-chunk count table in shared memory and for sizes that take the scanning kernel."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import _lib
    ids = np.random.Generator(np.random.PCG64(P + E)).integers(0, E, P).astype(np.int32)
    if P > 40:
        ids[7:39] = 2 % E                      # a whole warp pass of one expert
    d_ids = torch.from_numpy(ids).cuda()
    sorted_ids = torch.full((max(P, 1),), -1, dtype=torch.int32, device="cuda")
    offsets = torch.full((E + 1,), -1, dtype=torch.int32, device="cuda")
    _lib.check(_lib.lib.fuelq_moe_bucket(d_ids.data_ptr() if P else None, P, E, sorted_ids.data_ptr() if P else None,
                                         offsets.data_ptr(), torch.cuda.current_stream().cuda_stream), "fuelq_moe_bucket")
    torch.cuda.synchronize()
    want = np.argsort(ids, kind="stable").astype(np.int32)
    assert np.array_equal(sorted_ids.cpu().numpy()[:P], want)
    assert np.array_equal(offsets.cpu().numpy(), np.concatenate([[0], np.cumsum(np.bincount(ids, minlength=E))]).astype(np.int32))
