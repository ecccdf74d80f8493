"""Quantized LLaMA-architecture decode: greedy tokens against the CPU restatement of the reference's
model glue (oracle/llama_oracle.py) on a tiny random-init model in the style of the reference's own
model tests (hidden 32 / 2 layers there, fuel-core/src/lazy_quantized_llama.rs:564-652; here the
smallest sizes the k-quant block (256) and head_dim 128 allow), and CUDA-graph replay == eager."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _tiny():
    from fuel_b200.llama import LlamaConfig
    return LlamaConfig(dim=256, n_layers=2, n_heads=2, n_kv_heads=2, head_dim=128, ffn_dim=512, vocab=512, max_seq=48)


def _oracle_twin(model, oracle):
    """Rebuild the model's weights on the host: same seeded f32 tensors, quantized by the CPU quantizer."""
    from oracle.llama_oracle import OracleLlama
    from fuel_b200.llama import init_weight, q4km_mix, rope_tables
    c, dev = model.cfg, model.device
    ot = {12: oracle.Q4K, 14: oracle.Q6K}

    def q(name, li, n, k, seed):
        t = int(q4km_mix(name, li))
        blocks = oracle.quantize(ot[t], init_weight(n, k, seed, dev).cpu().numpy())
        return (ot[t], blocks, n, k)

    embed = oracle.quantize(oracle.Q4K, init_weight(c.vocab, c.dim, 1, dev).cpu().numpy())
    assert np.array_equal(embed, model.embed.cpu().numpy())      # device quantizer == CPU quantizer
    layers = []
    for li in range(c.n_layers):
        s0 = 1000 * (li + 1)
        layers.append(dict(q=q("attn_q", li, c.dim, c.dim, s0 + 1), k=q("attn_k", li, c.dim, c.dim, s0 + 2),
                           v=q("attn_v", li, c.dim, c.dim, s0 + 3), o=q("attn_output", li, c.dim, c.dim, s0 + 4),
                           gate=q("ffn_gate", li, c.ffn_dim, c.dim, s0 + 5), up=q("ffn_up", li, c.ffn_dim, c.dim, s0 + 6),
                           down=q("ffn_down", li, c.dim, c.ffn_dim, s0 + 7)))
    head = q("output", -1, c.vocab, c.dim, 2)
    cos, sin = rope_tables(c)
    return OracleLlama(c, embed, layers, head, cos, sin)


def test_greedy_tokens_match_cpu_reference_path(oracle):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200.llama import QLlama
    from fuel_b200 import ops
    dev = torch.device("cuda", 0)
    model = QLlama(_tiny(), dev)
    prompt = np.random.Generator(np.random.PCG64(3)).integers(0, 512, 8).tolist()
    got = model.generate(prompt, 12)
    twin = _oracle_twin(model, oracle)
    want = twin.generate(prompt, 12)
    assert got == want, (got, want)
    # logits of one more step agree to f32 summation-order accuracy
    _, ref_logits = twin.step(want[-1])
    model.run_step()
    torch.cuda.synchronize()
    lg = model.logits.cpu().numpy()
    assert np.abs(lg - ref_logits).max() <= 1e-4 * np.abs(ref_logits).max()
    # CUDA-graph replay and programmatic dependent launch give the same tokens as eager launches
    from fuel_b200 import _lib
    try:
        _lib.lib.fuelq_set_option(_lib.OPT_PDL, 1)
        model.capture()
        assert model.generate(prompt, 12) == got
    finally:
        _lib.lib.fuelq_set_option(_lib.OPT_PDL, 0)
    assert ops.device_error() == 0


def test_plain_step_agrees_with_fused_step():
    """The step with fused producers and tree-ordered o / down mat-vecs (what every GPU count runs for k-quant models)
    against the plain step (one call per op, plain mat-vecs; what other weight formats run): the same tokens, logits
    equal up to f32 summation order."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200.llama import QLlama
    model = QLlama(_tiny(), torch.device("cuda", 0))
    assert model.fused
    prompt = np.random.Generator(np.random.PCG64(4)).integers(0, 512, 20).tolist()
    outs = []
    for fused in (True, False):
        model.fused = fused
        toks = model.generate(prompt, 16)
        outs.append((toks, model.logits.clone()))
    assert outs[0][0] == outs[1][0]
    assert (outs[0][1] - outs[1][1]).abs().max().item() <= 1e-4 * outs[0][1].abs().max().item()


@pytest.mark.parametrize("name,n,k,world", [("q4k", 96, 4096, 1), ("q4k", 64, 4096, 2), ("q6k", 40, 11008, 4), ("q4k", 33, 11008, 8),
                                            ("q6k", 17, 1024, 2), ("q4k", 50, 2816, 8)])
def test_tree_ordered_matvec_gives_the_same_bits_for_every_split(oracle, name, n, k, world):
    """The row-parallel mat-vec: each of `world` ranks takes its aligned group of leaves of the k axis and the ranks'
    results are added pairwise in rank order (here on the host, in f32) - the value must have the bits of the
    one-GPU tree over all eight leaves, and agree with the CPU path to summation order."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ctypes
    from fuel_b200 import GgmlDType as T, _lib, ops
    from fuel_b200.llama import leaf_split, rank_leaves
    L = _lib.lib
    t, ot = {"q4k": (T.Q4K, oracle.Q4K), "q6k": (T.Q6K, oracle.Q6K)}[name]
    g = np.random.Generator(np.random.PCG64(n + k))
    w = g.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    x = g.standard_normal((1, k), dtype=np.float32)
    wb = oracle.quantize(ot, w)
    bb, nblk = t.type_size(), k // 256
    full = torch.from_numpy(wb).cuda()
    xd = torch.from_numpy(x).cuda()

    def run(world):
        parts = []
        for r in range(world):
            b0, leaves = rank_leaves(nblk, world, r)
            nb = sum(leaves)
            slab = full.view(n, nblk, bb)[:, b0:b0 + nb].contiguous().view(-1)
            packed = ops.quantize_act_packed(t, xd[:, b0 * 256:(b0 + nb) * 256].contiguous())
            y = torch.full((n,), float("nan"), device="cuda")
            arr = (ctypes.c_int32 * 8)(*leaves)
            _lib.check(L.fuelq_qmatmul_packed_tree(int(t), n, nb * 256, slab.data_ptr(), packed.data_ptr(), y.data_ptr(), len(leaves),
                                                   arr, None), "tree")
            parts.append(y.cpu().numpy())
        while len(parts) > 1:   # pairwise, in rank order, f32
            parts = [(parts[i] + parts[i + 1]).astype(np.float32) for i in range(0, len(parts), 2)]
        return parts[0]

    one = run(1)
    assert np.isfinite(one).all()
    if world > 1:
        assert np.array_equal(run(world).view(np.uint32), one.view(np.uint32))
    ref = oracle.matmul(ot, x, wb, n)[0]
    assert np.abs(one - ref).max() <= 2e-6 * np.abs(ref).max()
    assert sum(leaf_split(nblk)) == nblk
    assert ops.device_error() == 0


def test_in_kernel_exchange_single_rank_matches_fused_step():
    """comm="peer" with one rank runs the exchange protocol against itself (stamped pairs, step counter,
    stores into its own destination buffers); values must equal the plain single-GPU step, eagerly and
    as a replayed graph."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import ops
    from fuel_b200.llama import QLlama
    dev = torch.device("cuda", 0)
    prompt = np.random.Generator(np.random.PCG64(4)).integers(0, 512, 20).tolist()
    ref = QLlama(_tiny(), dev)
    want = ref.generate(prompt, 16)
    model = QLlama(_tiny(), dev, comm="peer")
    try:
        got = model.generate(prompt, 16)
        assert got == want
        assert torch.equal(model.logits, ref.logits) and torch.equal(model.x, ref.x)
        assert int(model.epoch.item()) == len(prompt) + 15
        model.capture()
        assert model.generate(prompt, 16) == want
        assert ops.device_error() == 0
    finally:
        model.release()


def test_exchange_wait_expires_with_an_error_code_and_the_context_stays_usable():
    """Failure detection without a fault: a consumer polls an exchange point that nothing ever stamps. After the
    deadline (FUELQ_OPT_PEER_WAIT_MS, shortened here) the kernel records device error 6 and finishes; the next call on
    the same context works and gives the right answer."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ctypes
    import time

    from fuel_b200 import GgmlDType as T, _lib, ops
    from oracle import oracle as O
    L = _lib.lib
    dim = 512
    x = torch.ones(dim, device="cuda")
    gain = torch.ones(dim, device="cuda")
    never_stamped = torch.zeros(2 * dim, dtype=torch.int32, device="cuda")   # a vector buffer nobody writes
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    packed = torch.zeros(L.fuelq_act_packed_bytes(int(T.Q4K), 1, dim), dtype=torch.uint8, device="cuda")
    peers = _lib.Peers()
    peers.world, peers.rank, peers.epoch = 1, 0, epoch.data_ptr()
    assert ops.device_error() == 0
    try:
        _lib.check(L.fuelq_set_option(_lib.OPT_PEER_WAIT_MS, 200), "set_option")
        t0 = time.time()
        _lib.check(L.fuelq_add_rmsnorm_q8k_peer(x.data_ptr(), never_stamped.data_ptr(), 1, gain.data_ptr(), dim, 1e-5,
                                                packed.data_ptr(), packed.numel(), ctypes.byref(peers), 3, None), "peer")
        torch.cuda.synchronize()
        dt = time.time() - t0
    finally:
        L.fuelq_set_option(_lib.OPT_PEER_WAIT_MS, 4000)
    assert 0.15 <= dt <= 3.0, dt
    assert ops.device_error() == 6          # kErrPeerWait; reading it clears it
    assert ops.device_error() == 0
    # the context is intact: an ordinary mat-vec right after gives the reference's numbers
    g = np.random.Generator(np.random.PCG64(0))
    w = g.standard_normal((64, 256), dtype=np.float32) * np.float32(0.02)
    xa = g.standard_normal((1, 256), dtype=np.float32)
    wb = O.quantize(O.Q4K, w)
    y = ops.qmatmul(T.Q4K, torch.from_numpy(wb).cuda(), 64, torch.from_numpy(xa).cuda()).cpu().numpy()
    r = O.matmul(O.Q4K, xa, wb, 64)
    assert np.abs(y - r).max() <= 2e-6 * np.abs(r).max()


@pytest.mark.parametrize("n_parts", [1, 2, 4, 8])
def test_rowpar_reduce_sums_the_parts_pairwise_in_rank_order(n_parts):
    """fuelq_rowpar_reduce on a buffer of stamped pairs written here by hand (what n_parts ranks' mat-vecs would have stored):
    the result is the balanced pairwise sum ((p0 + p1) + (p2 + p3)) + ..., bit for bit, not the left-to-right one."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ctypes

    from fuel_b200 import _lib, ops
    L = _lib.lib
    n, seq = 1000, 5
    parts = np.random.Generator(np.random.PCG64(n_parts)).standard_normal((n_parts, n), dtype=np.float32)
    parts[:, 0] = [1e8, 1.0, -1e8, 1.0, 3.0, 1e-3, -3.0, 7.0][:n_parts]      # an element where the order of the sum shows
    pairs = np.zeros((n_parts, n, 2), np.uint32)
    pairs[:, :, 0] = parts.view(np.uint32)
    pairs[:, :, 1] = 0 * _lib.PEER_MAX_SEQ + seq + 1                          # stamp of exchange point `seq` in step 0
    buf = torch.from_numpy(pairs.view(np.int32)).cuda()
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    peers = _lib.Peers()
    peers.world, peers.rank, peers.epoch = 1, 0, epoch.data_ptr()
    y = torch.full((n,), float("nan"), device="cuda")
    _lib.check(L.fuelq_rowpar_reduce(buf.data_ptr(), n_parts, n, y.data_ptr(), ctypes.byref(peers), seq, None), "fuelq_rowpar_reduce")
    torch.cuda.synchronize()
    level = [parts[q] for q in range(n_parts)]
    while len(level) > 1:
        level = [(level[i] + level[i + 1]).astype(np.float32) for i in range(0, len(level), 2)]
    assert np.array_equal(y.cpu().numpy().view(np.uint32), level[0].view(np.uint32))
    assert ops.device_error() == 0


@pytest.mark.parametrize("n_heads,n_kv,pos", [(4, 4, 0), (8, 2, 37), (4, 4, 300)])
def test_rope_fused_into_attention_matches_rope_store(n_heads, n_kv, pos):
    """fuelq_attn_decode with a rope argument = fuelq_rope_store followed by fuelq_attn_decode, bit for bit,
    and leaves the same caches behind."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ctypes

    from fuel_b200 import _lib
    from fuel_b200.llama import LlamaConfig, rope_tables
    L = _lib.lib
    hd, max_seq = 128, 512
    cos, sin = rope_tables(LlamaConfig(max_seq=max_seq))
    cos, sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    g = torch.Generator(device="cuda")
    g.manual_seed(pos)
    qkv = torch.randn((n_heads + 2 * n_kv) * hd, generator=g, device="cuda")
    kc0 = torch.randn(n_kv, max_seq, hd, generator=g, device="cuda")
    vc0 = torch.randn(n_kv, max_seq, hd, generator=g, device="cuda")
    posd = torch.tensor([pos], dtype=torch.int32, device="cuda")
    ws = torch.zeros(L.fuelq_attn_decode_workspace_bytes(n_heads), dtype=torch.uint8, device="cuda")
    scale = 1.0 / np.sqrt(hd)
    qd, kvd = n_heads * hd, n_kv * hd

    def run(fused):
        x, kc, vc = qkv.clone(), kc0.clone(), vc0.clone()
        out = torch.zeros(qd, device="cuda")
        rope = None
        if fused:
            rp = _lib.Rope()
            rp.k, rp.v = x.data_ptr() + 4 * qd, x.data_ptr() + 4 * (qd + kvd)
            rp.cos_table, rp.sin_table, rp.kcache, rp.vcache = cos.data_ptr(), sin.data_ptr(), kc.data_ptr(), vc.data_ptr()
            rope = ctypes.byref(rp)
        else:
            _lib.check(L.fuelq_rope_store(x.data_ptr(), x.data_ptr() + 4 * qd, x.data_ptr() + 4 * (qd + kvd), kc.data_ptr(),
                                          vc.data_ptr(), cos.data_ptr(), sin.data_ptr(), posd.data_ptr(), n_heads, n_kv, hd,
                                          max_seq, None), "rope_store")
        _lib.check(L.fuelq_attn_decode(x.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), posd.data_ptr(), n_heads,
                                       n_kv, hd, max_seq, scale, ws.data_ptr(), ws.numel(), rope, None), "attn_decode")
        torch.cuda.synchronize()
        return out, kc, vc

    a, b = run(False), run(True)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    assert not torch.equal(a[1], kc0)      # the cache row was really appended
